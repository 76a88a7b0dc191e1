// Kernel-bench entry for the attention library, in the row format of the reference's bench program
// (src/bench/qwen35_attention_bench.cpp:155-158; benches are named and listed like
// src/common/bench/registry.hpp):
//
//   <bench> kind=<prefill|decode> kernel=<name> q=<tokens> kv=<keys> mean_ms=.. sd_ms=.. max_abs=.. max_rel=..
//
//   arc_attention_bench --list
//   arc_attention_bench qwen35-attention [--runs N] [--warmup W] [--dump DIR]
//   arc_attention_bench sdpa-prefill | sdpa-decode [--runs N] [--warmup W] [--no-baseline]
//
// Every cell is run by two kernels: `baseline`, a scalar online-softmax kernel that lives in this file
// (one warp per query row, the formulation of src/modeling/qwen3_5/kernels.hpp:621-679 generalised to
// batches, windows and a gate) and `sdpa`, the library through its reference-shaped C++ interface.
// max_abs / max_rel compare the two outputs, as the reference's bench compares its kernels with its
// scalar one.  Times are CUDA-event times of single calls.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/arc_sdpa.h"
#include "arcaine_attention.hpp"

namespace {

using arcaine::bf16;

#define CK(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) throw std::runtime_error(std::string(#call) + ": " + cudaGetErrorString(e_)); \
    } while (0)

__device__ __forceinline__ float bf2f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t f2bf(float f) {  // round to nearest even (src/common/gpu/buffer.hpp:17-23)
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

struct Shape {
    int batch, seq, nq, nkv, hd;
    int window;          // keys a query sees, itself included; INT_MAX = all
    bool causal;         // false: every query sees every key
    const int* kv_len;   // device [batch] or nullptr (kv_uniform)
    const long long* kv_off;  // device [batch] first cache row of each sequence, or nullptr (b * kv_uniform)
    int kv_uniform;
    float scale;
};

// One warp per (sequence, token, head).  Lane l holds head-dim elements l, l + 32, ...; per key the
// partial dot products meet in a shuffle reduction and every lane keeps the same running max and sum.
__global__ void baseline_attention(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* gate,
                                   uint16_t* out, Shape s) {
    const long long row = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const long long rows = (long long)s.batch * s.seq * s.nq;
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const int h = (int)(row % s.nq);
    const int t = (int)((row / s.nq) % s.seq);
    const int b = (int)(row / ((long long)s.nq * s.seq));
    const int kvh = h / (s.nq / s.nkv);
    const int len = s.kv_len ? s.kv_len[b] : s.kv_uniform;
    const long long row0 = s.kv_off ? s.kv_off[b] : (long long)b * s.kv_uniform;
    const int self = len - s.seq + t;  // the query's own key position (the last seq keys are the queries')
    int hi = s.causal ? self + 1 : len;
    int lo = (s.causal && s.window != 0x7fffffff) ? self - s.window + 1 : 0;
    if (lo < 0) lo = 0;
    if (hi > len) hi = len;
    const int per = s.hd / 32;
    float qv[8], acc[8];
    const uint16_t* qp = q + ((long long)(b * s.seq + t) * s.nq + h) * s.hd;
    for (int i = 0; i < per; ++i) {
        qv[i] = bf2f(qp[lane + 32 * i]);
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = lo; j < hi; ++j) {
        const uint16_t* kp = k + ((row0 + j) * s.nkv + kvh) * s.hd;
        float d = 0.f;
        for (int i = 0; i < per; ++i) d += qv[i] * bf2f(kp[lane + 32 * i]);
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float x = d * s.scale;
        const float mn = fmaxf(m, x);
        const float a = expf(m - mn), p = expf(x - mn);
        l = l * a + p;
        const uint16_t* vp = v + ((row0 + j) * s.nkv + kvh) * s.hd;
        for (int i = 0; i < per; ++i) acc[i] = acc[i] * a + p * bf2f(vp[lane + 32 * i]);
        m = mn;
    }
    uint16_t* op = out + ((long long)(b * s.seq + t) * s.nq + h) * s.hd;
    const uint16_t* gp = gate ? gate + ((long long)(b * s.seq + t) * s.nq + h) * s.hd : nullptr;
    for (int i = 0; i < per; ++i) {
        uint16_t r = f2bf(l > 0.f ? acc[i] / l : 0.f);
        if (gp) r = f2bf(bf2f(r) / (1.0f + expf(-bf2f(gp[lane + 32 * i]))));  // src/modeling/qwen3_5_moe/kernels.hpp:80-88
        op[lane + 32 * i] = r;
    }
}

// The reference bench's input recipe (src/bench/qwen35_attention_bench.cpp:86-94): a linear congruential
// generator, ten bits of it per value, centred and scaled to [-0.5, 0.5).
struct Lcg {
    uint32_t state;
    explicit Lcg(uint32_t seed) : state(seed) {}
    float next() {
        state = state * 1664525u + 1013904223u;
        return (float)((int)((state >> 16) & 1023u) - 512) / 1024.0f;
    }
};

uint16_t host_f2bf(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float host_bf2f(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

struct DeviceBf16 {
    uint16_t* p = nullptr;
    size_t n = 0;
    DeviceBf16() = default;
    explicit DeviceBf16(size_t count) : n(count) { CK(cudaMalloc(&p, count * 2)); }
    DeviceBf16(const DeviceBf16&) = delete;
    DeviceBf16& operator=(const DeviceBf16&) = delete;
    ~DeviceBf16() { cudaFree(p); }
    void fill(Lcg& g) {
        std::vector<uint16_t> h(n);
        for (auto& x : h) x = host_f2bf(g.next());
        CK(cudaMemcpy(p, h.data(), n * 2, cudaMemcpyHostToDevice));
    }
    std::vector<uint16_t> host() const {
        std::vector<uint16_t> h(n);
        CK(cudaMemcpy(h.data(), p, n * 2, cudaMemcpyDeviceToHost));
        return h;
    }
};

struct Options {
    int runs = 20, warmup = 3;
    bool baseline = true;
    std::string dump;  // directory for the sdpa outputs of qwen35-attention (one .bin of bf16 bits per cell)
};

struct Timing {
    double mean, sd;
};

template <typename F>
Timing time_calls(F&& call, const Options& opt, cudaStream_t stream) {
    for (int i = 0; i < opt.warmup; ++i) call();
    CK(cudaStreamSynchronize(stream));
    cudaEvent_t a, b;
    CK(cudaEventCreate(&a));
    CK(cudaEventCreate(&b));
    double sum = 0, sq = 0;
    for (int i = 0; i < opt.runs; ++i) {
        CK(cudaEventRecord(a, stream));
        call();
        CK(cudaEventRecord(b, stream));
        CK(cudaEventSynchronize(b));
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, a, b));
        sum += ms;
        sq += (double)ms * ms;
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    const double mean = sum / opt.runs;
    const double var = opt.runs > 1 ? (sq - opt.runs * mean * mean) / (opt.runs - 1) : 0.0;
    return {mean, std::sqrt(var > 0 ? var : 0)};
}

void print_row(const char* bench, const char* kind, const char* kernel, long long q, long long kv, Timing t,
               double max_abs, double max_rel) {
    std::printf("%s kind=%s kernel=%s q=%lld kv=%lld mean_ms=%.3f sd_ms=%.3f max_abs=%.6f max_rel=%.6f\n", bench, kind,
                kernel, q, kv, t.mean, t.sd, max_abs, max_rel);
    std::fflush(stdout);
}

void compare(const std::vector<uint16_t>& want, const std::vector<uint16_t>& got, double& max_abs, double& max_rel) {
    max_abs = max_rel = 0;
    for (size_t i = 0; i < want.size(); ++i) {
        const double e = host_bf2f(want[i]), a = host_bf2f(got[i]);
        const double err = std::fabs(e - a);
        if (err > max_abs) max_abs = err;
        const double rel = err / std::fmax(1e-3, std::fabs(e));
        if (rel > max_rel) max_rel = rel;
    }
}

void launch_baseline(const DeviceBf16& q, const DeviceBf16& k, const DeviceBf16& v, const uint16_t* gate, DeviceBf16& out,
                     const Shape& s, cudaStream_t stream) {
    const long long rows = (long long)s.batch * s.seq * s.nq;
    baseline_attention<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(q.p, k.p, v.p, gate, out.p, s);
    CK(cudaGetLastError());
}

// ---- qwen35-attention: the reference bench's cells (24Q / 4KV / D256, prefill 128 and 512, decode at
// depths 0, 512, 1024), inputs from its recipe with seed 42: Q, then K, then V.
int bench_qwen35(const Options& opt) {
    const int nq = 24, nkv = 4, hd = 256, max_q = 512, max_kv = 1025;
    const float scale = 0.0625f;
    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    Lcg g(42);
    DeviceBf16 q((size_t)max_q * nq * hd), k((size_t)max_kv * nkv * hd), v((size_t)max_kv * nkv * hd);
    q.fill(g);
    k.fill(g);
    v.fill(g);
    DeviceBf16 gate(q.n), out(q.n), ref(q.n);
    gate.fill(g);
    arcaine::SdpaWorkspace ws;
    std::printf("[bench] Qwen3.5 full attention: q_heads=%d kv_heads=%d head_dim=%d\n", nq, nkv, hd);
    auto dump = [&](const char* kind, int seq, int kv, const std::vector<uint16_t>& bits) {
        if (opt.dump.empty()) return;
        const std::string path = opt.dump + "/" + kind + "_q" + std::to_string(seq) + "_kv" + std::to_string(kv) + ".bin";
        FILE* f = std::fopen(path.c_str(), "wb");
        if (!f) throw std::runtime_error("cannot write " + path);
        std::fwrite(bits.data(), 2, bits.size(), f);
        std::fclose(f);
    };
    auto cell = [&](const char* kind, int seq, int past) {
        Shape s{1, seq, nq, nkv, hd, 0x7fffffff, true, nullptr, nullptr, past + seq, scale};
        const size_t n = (size_t)seq * nq * hd;
        for (int gated = 0; gated < (seq == 1 ? 2 : 1); ++gated) {
            const uint16_t* gp = gated ? gate.p : nullptr;
            launch_baseline(q, k, v, gp, ref, s, stream);
            CK(cudaStreamSynchronize(stream));
            std::vector<uint16_t> want = ref.host();
            want.resize(n);
            print_row("qwen35_attention", kind, gated ? "baseline-gated" : "baseline", seq, past + seq,
                      time_calls([&] { launch_baseline(q, k, v, gp, ref, s, stream); }, opt, stream), 0.0, 0.0);
            auto sdpa = [&] {
                if (gated)  // the decode kernel with the sigmoid gate of src/modeling/qwen3_5/operators.hpp:160 fused
                    arcaine::qwen35_xmx_attention_decode_gqa(stream, q.p, k.p, v.p, out.p, past, nq, nkv, hd, scale, gate.p, ws);
                else
                    arcaine::qwen35_xmx_attention(stream, q.p, k.p, v.p, out.p, seq, past, nq, nkv, hd, scale, ws);
            };
            sdpa();
            CK(cudaStreamSynchronize(stream));
            std::vector<uint16_t> got = out.host();
            got.resize(n);
            double ma = 0, mr = 0;
            compare(want, got, ma, mr);
            dump(gated ? "decode_gated" : kind, seq, past + seq, got);
            print_row("qwen35_attention", kind, gated ? "sdpa-gated" : "sdpa", seq, past + seq, time_calls(sdpa, opt, stream), ma, mr);
        }
    };
    for (int seq : {128, 512}) cell("prefill", seq, 0);
    for (int depth : {0, 512, 1024}) cell("decode", 1, depth);
    cudaStreamDestroy(stream);
    return 0;
}

// ---- sdpa-prefill: the sliding-window prefill shape (batch 4, 32Q / 16KV, D128, 8192 tokens, window 1024)
// and the canvas-over-prompt shape (16Q / 8KV, D256, 256 queries over 2304 keys, no mask, no scale).
int bench_prefill(const Options& opt) {
    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    arcaine::SdpaWorkspace ws;
    struct Case { const char* label; int batch, seq, kv, nq, nkv, hd, window; bool causal; float scale; };
    const Case cases[] = {{"window", 4, 8192, 8192, 32, 16, 128, 1024, true, 0.08838834764831845f},
                          {"canvas", 1, 256, 2304, 16, 8, 256, 0x7fffffff, false, 1.0f}};
    for (const Case& c : cases) {
        Lcg g(7);
        DeviceBf16 q((size_t)c.batch * c.seq * c.nq * c.hd), k((size_t)c.batch * c.kv * c.nkv * c.hd), v(k.n);
        q.fill(g);
        k.fill(g);
        v.fill(g);
        DeviceBf16 out(q.n), ref(q.n);
        arc_sdpa_prefill_params p{};
        p.q = q.p; p.k = k.p; p.v = v.p; p.out = out.p;
        p.batch = c.batch; p.seq = c.seq; p.kv_len = c.kv; p.nq = c.nq; p.nkv = c.nkv; p.hd = c.hd;
        p.q_stride_t = p.o_stride_t = (int64_t)c.nq * c.hd;
        p.k_stride_t = p.v_stride_t = (int64_t)c.nkv * c.hd;
        p.q_stride_b = p.o_stride_b = (int64_t)c.seq * c.nq * c.hd;
        p.k_stride_b = p.v_stride_b = (int64_t)c.kv * c.nkv * c.hd;
        p.scale = c.scale;
        p.mask_type = c.causal ? ARC_MASK_CAUSAL : ARC_MASK_NONE;
        p.window = c.window;
        const size_t need = arc_sdpa_prefill_workspace_bytes(&p);
        if (need) { p.workspace = ws.reserve(need); p.workspace_bytes = ws.capacity(); }
        auto sdpa = [&] {
            const int rc = arc_sdpa_prefill(&p, stream);
            if (rc != ARC_OK) throw std::runtime_error(std::string("arc_sdpa_prefill: ") + arc_sdpa_status_string(rc));
        };
        double ma = 0, mr = 0;
        std::string kind = std::string("prefill-") + c.label;
        if (opt.baseline) {
            Shape s{c.batch, c.seq, c.nq, c.nkv, c.hd, c.window, c.causal, nullptr, nullptr, c.kv, c.scale};
            Options once = opt;
            once.runs = 2;
            once.warmup = 1;
            print_row("sdpa_prefill", kind.c_str(), "baseline", (long long)c.batch * c.seq, c.kv,
                      time_calls([&] { launch_baseline(q, k, v, nullptr, ref, s, stream); }, once, stream), 0.0, 0.0);
            sdpa();
            CK(cudaStreamSynchronize(stream));
            compare(ref.host(), out.host(), ma, mr);
        }
        print_row("sdpa_prefill", kind.c_str(), "sdpa", (long long)c.batch * c.seq, c.kv, time_calls(sdpa, opt, stream), ma, mr);
    }
    cudaStreamDestroy(stream);
    return 0;
}

// ---- sdpa-decode: gated decode (batch 64, 24Q / 4KV, D256, lengths 1024..32768 from the recipe's
// generator) and long-context decode (batch 4, 16Q / 2KV, D128, 524288 keys per sequence).
int bench_decode(const Options& opt) {
    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    arcaine::SdpaWorkspace ws;
    struct Case { const char* label; int batch, nq, nkv, hd, len_lo, len_hi; bool gate; };
    const Case cases[] = {{"gated", 64, 24, 4, 256, 1024, 32768, true}, {"long", 4, 16, 2, 128, 524288, 524288, false}};
    for (const Case& c : cases) {
        Lcg g(11);
        std::vector<int> lens(c.batch);
        std::vector<long long> offs(c.batch);
        long long total = 0;
        for (int b = 0; b < c.batch; ++b) {
            g.next();
            lens[b] = c.len_lo + (int)(g.state % (uint32_t)(c.len_hi - c.len_lo + 1));
            offs[b] = total;
            total += lens[b];
        }
        DeviceBf16 q((size_t)c.batch * c.nq * c.hd), k((size_t)total * c.nkv * c.hd), v(k.n), gate(q.n), out(q.n), ref(q.n);
        q.fill(g);
        k.fill(g);
        v.fill(g);
        gate.fill(g);
        int* d_len = nullptr;
        long long* d_off = nullptr;
        CK(cudaMalloc(&d_len, c.batch * sizeof(int)));
        CK(cudaMalloc(&d_off, c.batch * sizeof(long long)));
        CK(cudaMemcpy(d_len, lens.data(), c.batch * sizeof(int), cudaMemcpyHostToDevice));
        CK(cudaMemcpy(d_off, offs.data(), c.batch * sizeof(long long), cudaMemcpyHostToDevice));
        const float scale = 1.0f / std::sqrt((float)c.hd);
        arc_sdpa_decode_params p{};
        p.q = q.p; p.k = k.p; p.v = v.p; p.out = out.p;
        p.gate = c.gate ? gate.p : nullptr;
        p.kv_len = d_len;
        p.kv_row_offset = reinterpret_cast<const int64_t*>(d_off);
        p.batch = c.batch; p.nq = c.nq; p.nkv = c.nkv; p.hd = c.hd;
        p.max_kv_len = c.len_hi;
        p.q_stride_b = p.o_stride_b = (int64_t)c.nq * c.hd;
        p.kv_stride_t = (int64_t)c.nkv * c.hd;
        p.kv_rows_total = total;
        p.scale = scale;
        const size_t need = arc_sdpa_decode_workspace_bytes(&p);
        p.workspace = ws.reserve(need);
        p.workspace_bytes = ws.capacity();
        auto sdpa = [&] {
            const int rc = arc_sdpa_decode(&p, stream);
            if (rc != ARC_OK) throw std::runtime_error(std::string("arc_sdpa_decode: ") + arc_sdpa_status_string(rc));
        };
        double ma = 0, mr = 0;
        std::string kind = std::string("decode-") + c.label;
        long long kv_mean = total / c.batch;
        if (opt.baseline) {
            Shape s{c.batch, 1, c.nq, c.nkv, c.hd, 0x7fffffff, true, d_len, d_off, 0, scale};
            Options once = opt;
            once.runs = 2;
            once.warmup = 1;
            print_row("sdpa_decode", kind.c_str(), "baseline", c.batch, kv_mean,
                      time_calls([&] { launch_baseline(q, k, v, c.gate ? gate.p : nullptr, ref, s, stream); }, once, stream), 0.0, 0.0);
            sdpa();
            CK(cudaStreamSynchronize(stream));
            compare(ref.host(), out.host(), ma, mr);
        }
        print_row("sdpa_decode", kind.c_str(), "sdpa", c.batch, kv_mean, time_calls(sdpa, opt, stream), ma, mr);
        cudaFree(d_len);
        cudaFree(d_off);
    }
    cudaStreamDestroy(stream);
    return 0;
}

struct Bench {
    const char* name;
    const char* description;
    int (*run)(const Options&);
};

const Bench kBenches[] = {
    {"qwen35-attention", "Qwen3.5 full attention at 24Q/4KV/D256: scalar baseline and the sdpa library", bench_qwen35},
    {"sdpa-prefill", "sliding-window prefill (batch 4, 32Q/16KV, D128, 8192 tokens) and the canvas step (D256)", bench_prefill},
    {"sdpa-decode", "gated decode (batch 64, D256, ragged lengths) and long-context decode (524288 keys)", bench_decode},
};

}  // namespace

int main(int argc, char** argv) {
    Options opt;
    const Bench* chosen = nullptr;
    bool list = argc < 2;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto value = [&]() -> int {
            if (i + 1 >= argc) throw std::runtime_error("missing value after " + a);
            return std::atoi(argv[++i]);
        };
        try {
            if (a == "--list") list = true;
            else if (a == "--runs") opt.runs = value();
            else if (a == "--warmup") opt.warmup = value();
            else if (a == "--no-baseline") opt.baseline = false;
            else if (a == "--dump") {
                if (i + 1 >= argc) throw std::runtime_error("missing directory after --dump");
                opt.dump = argv[++i];
            }
            else {
                for (const Bench& b : kBenches)
                    if (a == b.name) chosen = &b;
                if (!chosen) throw std::runtime_error("unknown bench or option: " + a);
            }
        } catch (const std::exception& e) {
            std::fprintf(stderr, "%s\n", e.what());
            return 2;
        }
    }
    if (list || !chosen) {
        for (const Bench& b : kBenches) std::printf("%-18s %s\n", b.name, b.description);
        return chosen || list ? 0 : 2;
    }
    if (opt.runs < 1) opt.runs = 1;
    try {
        return chosen->run(opt);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "%s: %s\n", chosen->name, e.what());
        return 1;
    }
}
