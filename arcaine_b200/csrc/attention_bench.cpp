// Attention kernel bench in the reference's kbench row format
// (src/bench/qwen35_attention_bench.cpp): Qwen3.5 full attention at 24 query
// heads / 4 KV heads / head_dim 256, inputs from the same LCG recipe
// (state = state*1664525 + 1013904223 from 42; x = (((state>>16)&1023)-512)/1024;
// Q, then K, then V), prefill lengths -p and decode depths -d, driven through the
// reference-shaped C++ interface.  With --dump DIR every cell's bf16 output is
// written to DIR/<kind>_q<seq>_kv<len>.bin so a checker can compare it with an
// independent implementation; the bench itself prints timings only.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "arcaine_attention.hpp"

using arcaine::bf16;

static uint16_t float_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    uint32_t bias = ((u >> 16) & 1u) + 0x7FFFu;
    return static_cast<uint16_t>((u + bias) >> 16);
}

static std::vector<int> parse_csv(const std::string& s) {
    std::vector<int> out;
    size_t pos = 0;
    while (pos < s.size()) {
        size_t next = s.find(',', pos);
        if (next == std::string::npos) next = s.size();
        if (next > pos) out.push_back(std::stoi(s.substr(pos, next - pos)));
        pos = next + 1;
    }
    return out;
}

#define CK(x)                                                                          \
    do {                                                                               \
        cudaError_t e_ = (x);                                                          \
        if (e_ != cudaSuccess) throw std::runtime_error(std::string(#x) + ": " + cudaGetErrorString(e_)); \
    } while (0)

static void dump(const std::string& dir, const char* kind, int seq, int kv, const bf16* dev, size_t n) {
    if (dir.empty()) return;
    std::vector<bf16> host(n);
    CK(cudaMemcpy(host.data(), dev, n * sizeof(bf16), cudaMemcpyDeviceToHost));
    std::string path = dir + "/" + kind + "_q" + std::to_string(seq) + "_kv" + std::to_string(kv) + ".bin";
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) throw std::runtime_error("cannot write " + path);
    std::fwrite(host.data(), sizeof(bf16), n, f);
    std::fclose(f);
}

int main(int argc, char** argv) {
    try {
        std::string p_csv = "128,512", d_csv = "0,512,1024", dump_dir;
        int warmup = 3, runs = 10;
        for (int i = 1; i < argc; ++i) {
            std::string arg = argv[i];
            auto next = [&]() -> std::string {
                if (i + 1 >= argc) throw std::runtime_error("missing value for " + arg);
                return argv[++i];
            };
            if (arg == "-p" || arg == "--p") p_csv = next();
            else if (arg == "-d" || arg == "--d") d_csv = next();
            else if (arg == "-w" || arg == "--w") warmup = std::stoi(next());
            else if (arg == "-r" || arg == "--r") runs = std::stoi(next());
            else if (arg == "--dump") dump_dir = next();
            else { std::fprintf(stderr, "unknown arg: %s\n", arg.c_str()); return 1; }
        }
        std::vector<int> prefills = parse_csv(p_csv), depths = parse_csv(d_csv);
        if (prefills.empty() || depths.empty() || warmup < 0 || runs <= 0)
            throw std::runtime_error("invalid benchmark arguments");

        constexpr int query_heads = 24, key_heads = 4, head_dim = 256;
        constexpr float scale = 0.0625f;
        int max_query = *std::max_element(prefills.begin(), prefills.end());
        int max_depth = *std::max_element(depths.begin(), depths.end());
        int max_kv = std::max(max_query, max_depth + 1);

        std::vector<bf16> host_q((size_t)max_query * query_heads * head_dim);
        std::vector<bf16> host_k((size_t)max_kv * key_heads * head_dim);
        std::vector<bf16> host_v(host_k.size());
        std::vector<bf16> host_g(host_q.size());
        uint32_t state = 42;
        auto fill = [&](std::vector<bf16>& values) {
            for (bf16& value : values) {
                state = state * 1664525u + 1013904223u;
                float x = (static_cast<int>((state >> 16) & 1023u) - 512) / 1024.0f;
                value = float_to_bf16(x);
            }
        };
        fill(host_q); fill(host_k); fill(host_v); fill(host_g);

        bf16 *q, *k, *v, *g, *out;
        CK(cudaMalloc(&q, host_q.size() * 2));
        CK(cudaMalloc(&k, host_k.size() * 2));
        CK(cudaMalloc(&v, host_v.size() * 2));
        CK(cudaMalloc(&g, host_g.size() * 2));
        CK(cudaMalloc(&out, host_q.size() * 2));
        CK(cudaMemcpy(q, host_q.data(), host_q.size() * 2, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(k, host_k.data(), host_k.size() * 2, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(v, host_v.data(), host_v.size() * 2, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(g, host_g.data(), host_g.size() * 2, cudaMemcpyHostToDevice));
        cudaStream_t stream;
        CK(cudaStreamCreate(&stream));
        arcaine::SdpaWorkspace ws;

        std::printf("[bench] Qwen3.5 full attention: q_heads=24 kv_heads=4 head_dim=256\n");
        auto cell = [&](const char* kind, int seq, int past, bool gated) {
            auto run = [&]() {
                if (gated)
                    arcaine::qwen35_xmx_attention_decode_gqa(stream, q, k, v, out, past, query_heads, key_heads,
                                                             head_dim, scale, g, ws);
                else
                    arcaine::qwen35_xmx_attention(stream, q, k, v, out, seq, past, query_heads, key_heads, head_dim,
                                                  scale, ws);
            };
            run();
            CK(cudaStreamSynchronize(stream));
            dump(dump_dir, kind, seq, past + seq, out, (size_t)seq * query_heads * head_dim);
            for (int i = 0; i < warmup; ++i) run();
            CK(cudaStreamSynchronize(stream));
            std::vector<double> samples;
            for (int i = 0; i < runs; ++i) {
                auto start = std::chrono::steady_clock::now();
                run();
                CK(cudaStreamSynchronize(stream));
                samples.push_back(
                    std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - start).count());
            }
            double mean = 0, sd = 0;
            for (double s : samples) mean += s;
            mean /= samples.size();
            for (double s : samples) sd += (s - mean) * (s - mean);
            sd = std::sqrt(sd / samples.size());
            std::printf("qwen35_attention kind=%s kernel=sm100 q=%d kv=%d mean_ms=%.3f sd_ms=%.3f\n", kind, seq,
                        past + seq, mean, sd);
        };
        for (int seq : prefills) cell("prefill", seq, 0, false);
        for (int depth : depths) cell("decode", 1, depth, false);
        for (int depth : depths) cell("decode_gated", 1, depth, true);
        CK(cudaStreamSynchronize(stream));
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "attention_bench: %s\n", e.what());
        return 2;
    }
}
