// Reference-shaped C++ wrappers over the C ABI (see arcaine_attention.hpp).
#include "arcaine_attention.hpp"

#include <stdexcept>
#include <string>

#include "../../include/arc_sdpa.h"

namespace arcaine {

namespace {

void throw_on(int status, const char* where) {
    if (status != ARC_OK)
        throw std::runtime_error(std::string(where) + ": " + arc_sdpa_status_string(status));
}

// One sequence, token-major contiguous tensors: (tokens, heads, hd).
void run_prefill(cudaStream_t stream, const bf16* q, const bf16* k, const bf16* v, bf16* out, const bf16* gate,
                 const float* mask, int seq, int kv_len, int nq, int nkv, int hd, float scale, int mask_type,
                 int window, SdpaWorkspace& ws, const char* where, const int32_t* block_ids = nullptr,
                 int block_ids_offset = 0) {
    arc_sdpa_prefill_params p{};
    p.q = q;
    p.k = k;
    p.v = v;
    p.out = out;
    p.gate = gate;
    p.mask = mask;
    p.batch = 1;
    p.seq = seq;
    p.kv_len = kv_len;
    p.nq = nq;
    p.nkv = nkv;
    p.hd = hd;
    p.q_stride_t = p.o_stride_t = (int64_t)nq * hd;
    p.k_stride_t = p.v_stride_t = (int64_t)nkv * hd;
    p.q_stride_b = p.o_stride_b = (int64_t)seq * nq * hd;
    p.k_stride_b = p.v_stride_b = (int64_t)kv_len * nkv * hd;
    p.scale = scale;
    p.mask_type = mask_type;
    p.window = window;
    p.num_splits = 0;
    p.block_ids = block_ids;
    p.block_ids_offset = block_ids_offset;
    const size_t need = arc_sdpa_prefill_workspace_bytes(&p);
    if (need) {
        p.workspace = ws.reserve(need);
        p.workspace_bytes = ws.capacity();
    }
    throw_on(arc_sdpa_prefill(&p, stream), where);
}

void run_decode(cudaStream_t stream, const bf16* q, const bf16* k, const bf16* v, bf16* out, const bf16* gate,
                int kv_len, int nq, int nkv, int hd, float scale, SdpaWorkspace& ws, const char* where) {
    arc_sdpa_decode_params p{};
    p.q = q;
    p.k = k;
    p.v = v;
    p.out = out;
    p.gate = gate;
    p.batch = 1;
    p.nq = nq;
    p.nkv = nkv;
    p.hd = hd;
    p.kv_len_uniform = kv_len;
    p.max_kv_len = kv_len;
    p.q_stride_b = p.o_stride_b = (int64_t)nq * hd;
    p.kv_stride_b = kv_len;
    p.kv_stride_t = (int64_t)nkv * hd;
    p.kv_rows_total = kv_len;
    p.scale = scale;
    const size_t need = arc_sdpa_decode_workspace_bytes(&p);
    if (need == 0) throw_on(arc_sdpa_decode(&p, stream), where);  // reports the reason
    p.workspace = ws.reserve(need);
    p.workspace_bytes = ws.capacity();
    throw_on(arc_sdpa_decode(&p, stream), where);
}

}  // namespace

SdpaWorkspace::~SdpaWorkspace() {
    if (ptr_ && owned_) cudaFree(ptr_);
}

void* SdpaWorkspace::reserve(size_t bytes) {
    if (bytes > bytes_) {
        if (!owned_) throw std::runtime_error("SdpaWorkspace: the borrowed region is too small for this call");
        if (ptr_) cudaFree(ptr_);
        ptr_ = nullptr;
        bytes_ = 0;
        if (cudaMalloc(&ptr_, bytes) != cudaSuccess) throw std::runtime_error("SdpaWorkspace: cudaMalloc failed");
        bytes_ = bytes;
    }
    return ptr_;
}

void gqa_attention_sdpa(CudaEngine& ctx, const bf16* Q, int seq, int nq, int hd, const bf16* Kc,
                        const bf16* Vc, int kv_len, int nkv, const float* mask, int mask_type, bf16* out,
                        SdpaWorkspace& ws) {
    run_prefill(ctx.stream, Q, Kc, Vc, out, nullptr, mask, seq, kv_len, nq, nkv, hd, 1.0f, mask_type,
                ARC_NO_WINDOW, ws, "gqa_attention_sdpa");
}

void gqa_attention(CudaEngine& ctx, const bf16* Q, int seq, int nq, int hd, const bf16* Kc, const bf16* Vc,
                   int kv_len, int nkv, int /*past_offset*/, int sliding_window, bool causal, bf16* out,
                   SdpaWorkspace& ws) {
    // Query and key positions share past_offset, so it cancels out of the rule.
    run_prefill(ctx.stream, Q, Kc, Vc, out, nullptr, nullptr, seq, kv_len, nq, nkv, hd, 1.0f,
                causal ? ARC_MASK_CAUSAL : ARC_MASK_NONE, causal ? sliding_window : ARC_NO_WINDOW, ws,
                "gqa_attention");
}

void batched_attention(CudaEngine& ctx, const bf16* Q_dev, int seq_len, int nq_heads, int q_head_dim,
                       const bf16* K_dev, const bf16* V_dev, int kv_len, int nkv_heads, int kv_head_dim,
                       int past_offset, int sliding_window, float scale, bool skip_mask,
                       const int32_t* block_ids, bf16* out, SdpaWorkspace& ws) {
    if (q_head_dim != kv_head_dim) throw std::runtime_error("batched_attention: q and kv head_dim differ");
    if (skip_mask) block_ids = nullptr;  // the reference builds no mask at all then
    // key j of K_dev sits at absolute position past_offset - (kv_len - seq_len) + j
    const int ids_offset = past_offset - (kv_len - seq_len);
    if (block_ids && ids_offset < 0) throw std::runtime_error("batched_attention: block ids start before position 0");
    run_prefill(ctx.stream, Q_dev, K_dev, V_dev, out, nullptr, nullptr, seq_len, kv_len, nq_heads, nkv_heads,
                q_head_dim, scale, skip_mask ? ARC_MASK_NONE : ARC_MASK_CAUSAL,
                skip_mask ? ARC_NO_WINDOW : sliding_window, ws, "batched_attention", block_ids,
                block_ids ? ids_offset : 0);
}

void gemma4_sliding_decode_attention(CudaEngine& ctx, const bf16* Q_dev, const bf16* K_cache, const bf16* V_cache,
                                     int kv_len, int kv_start, int nq_heads, int nkv_heads, int head_dim, bf16* out,
                                     SdpaWorkspace& ws) {
    const size_t row = (size_t)nkv_heads * head_dim;
    run_decode(ctx.stream, Q_dev, K_cache + (size_t)kv_start * row, V_cache + (size_t)kv_start * row, out, nullptr,
               kv_len, nq_heads, nkv_heads, head_dim, 1.0f, ws, "gemma4_sliding_decode_attention");
}

void qwen35_xmx_attention(cudaStream_t stream, const bf16* query, const bf16* key, const bf16* value,
                          bf16* output, int seq, int past, int query_heads, int key_heads, int head_dim,
                          float scale, SdpaWorkspace& ws) {
    if (key_heads <= 0 || query_heads % key_heads != 0)
        throw std::runtime_error("Qwen3.5 attention requires integral GQA ratio");
    if (seq == 1)
        run_decode(stream, query, key, value, output, nullptr, past + 1, query_heads, key_heads, head_dim, scale,
                   ws, "qwen35_xmx_attention");
    else
        run_prefill(stream, query, key, value, output, nullptr, nullptr, seq, past + seq, query_heads, key_heads,
                    head_dim, scale, ARC_MASK_CAUSAL, ARC_NO_WINDOW, ws, "qwen35_xmx_attention");
}

void qwen35_online_attention(cudaStream_t stream, const bf16* query, const bf16* key, const bf16* value,
                             bf16* output, int seq, int past, int query_heads, int key_heads, int head_dim,
                             float scale, SdpaWorkspace& ws) {
    qwen35_xmx_attention(stream, query, key, value, output, seq, past, query_heads, key_heads, head_dim, scale, ws);
}

void qwen35_xmx_attention_decode_gqa(cudaStream_t stream, const bf16* query, const bf16* key,
                                     const bf16* value, bf16* output, int past, int query_heads,
                                     int key_heads, int head_dim, float scale, const bf16* gate,
                                     SdpaWorkspace& ws) {
    if (key_heads <= 0 || query_heads % key_heads != 0)
        throw std::runtime_error("Qwen3.5 attention requires integral GQA ratio");
    run_decode(stream, query, key, value, output, gate, past + 1, query_heads, key_heads, head_dim, scale, ws,
               "qwen35_xmx_attention_decode_gqa");
}

void mul_sigmoid_inplace(cudaStream_t stream, bf16* a, const bf16* gate, size_t n) {
    throw_on(arc_mul_sigmoid_inplace(a, gate, (int64_t)n, stream), "mul_sigmoid_inplace");
}

void fill_causal_mask(cudaStream_t stream, float* mask, int q_len, int kv_len, int past_offset,
                      int sliding_window) {
    throw_on(arc_fill_causal_mask(mask, q_len, kv_len, past_offset, sliding_window, stream), "fill_causal_mask");
}

void rms_norm(cudaStream_t stream, const bf16* x, const bf16* weight, bf16* out, int rows, int H, float eps) {
    // One "head" per row; out of place is the K path of the kernel (source and destination rows differ).
    arc_qkv_prepare_params p{};
    p.batch = 1;
    p.seq = rows;
    p.hd = H;
    p.eps = eps;
    if (x == out) {
        p.q = out;
        p.nq = 1;
        p.q_stride_t = H;
        p.q_weight = weight;
    } else {
        p.k_src = x;
        p.k_dst = out;
        p.nkv = 1;
        p.k_src_stride_t = p.k_dst_stride_t = H;
        p.k_weight = weight;
    }
    throw_on(arc_qkv_prepare(&p, stream), "rms_norm");
}

void fused_norm_rope_inplace(cudaStream_t stream, bf16* x, const bf16* weight, int seq, int nheads, int hd,
                             int offset, float theta, float partial, float eps, const float* rope_cos,
                             const float* rope_sin) {
    arc_qkv_prepare_params p{};
    p.q = x;
    p.q_weight = weight;
    p.batch = 1;
    p.seq = seq;
    p.nq = nheads;
    p.hd = hd;
    p.q_stride_t = (int64_t)nheads * hd;
    p.n_active_pairs = static_cast<int>(partial * hd / 2.0f);
    p.rope_cos = rope_cos;
    p.rope_sin = rope_sin;
    p.pos0 = offset;
    p.theta = theta;
    p.eps = eps;
    throw_on(arc_qkv_prepare(&p, stream), "fused_norm_rope_inplace");
}

void qkv_norm_rope_append(cudaStream_t stream, bf16* Q, const bf16* K, const bf16* V, bf16* k_cache, bf16* v_cache,
                          int seq, int past_len, int nq, int nkv, int hd, const bf16* q_norm, const bf16* k_norm,
                          float theta, float partial, float eps, const float* rope_cos, const float* rope_sin) {
    arc_qkv_prepare_params p{};
    const int64_t row = (int64_t)nkv * hd;
    p.q = Q;
    p.k_src = K;
    p.v_src = V;
    p.k_dst = k_cache + (int64_t)past_len * row;
    p.v_dst = v_cache + (int64_t)past_len * row;
    p.q_weight = q_norm;
    p.k_weight = k_norm;
    p.batch = 1;
    p.seq = seq;
    p.nq = nq;
    p.nkv = nkv;
    p.hd = hd;
    p.q_stride_t = (int64_t)nq * hd;
    p.k_src_stride_t = p.v_src_stride_t = p.k_dst_stride_t = p.v_dst_stride_t = row;
    p.n_active_pairs = static_cast<int>(partial * hd / 2.0f);
    p.rope_cos = rope_cos;
    p.rope_sin = rope_sin;
    p.pos0 = past_len;
    p.theta = theta;
    p.eps = eps;
    throw_on(arc_qkv_prepare(&p, stream), "qkv_norm_rope_append");
}

void qwen35_norm_mrope_append(cudaStream_t stream, bf16* query, const bf16* key, const bf16* value, bf16* key_cache,
                              bf16* value_cache, const int32_t* positions, int seq, int past, int query_heads,
                              int key_heads, int head_dim, int rotary_dim, float theta, const int sections[3],
                              const bf16* q_norm, const bf16* k_norm, float eps) {
    if (!sections) throw std::runtime_error("Qwen3.5 MRoPE needs three sections");
    arc_qkv_prepare_params p{};
    const int64_t row = (int64_t)key_heads * head_dim;
    p.q = query;
    p.k_src = key;
    p.v_src = value;
    p.k_dst = key_cache + (int64_t)past * row;
    p.v_dst = value_cache + (int64_t)past * row;
    p.q_weight = q_norm;
    p.k_weight = k_norm;
    p.batch = 1;
    p.seq = seq;
    p.nq = query_heads;
    p.nkv = key_heads;
    p.hd = head_dim;
    p.q_stride_t = (int64_t)query_heads * head_dim;
    p.k_src_stride_t = p.v_src_stride_t = p.k_dst_stride_t = p.v_dst_stride_t = row;
    p.n_active_pairs = rotary_dim / 2;
    p.rot_half = rotary_dim / 2;
    p.freq_denom = rotary_dim;
    p.mrope_positions = positions;
    for (int i = 0; i < 3; ++i) p.mrope_section[i] = sections[i];
    p.v_copy = 1;
    p.theta = theta;
    p.eps = eps;
    throw_on(arc_qkv_prepare(&p, stream), "qwen35_norm_mrope_append");
}

arc_head_shard plan_head_shards(int nq, int nkv, int batch, int world, int rank) {
    arc_head_shard sh{};
    throw_on(arc_plan_head_shards(nq, nkv, batch, world, rank, &sh), "plan_head_shards");
    return sh;
}

void plan_seq_shards(long long kv_len, int world, int rank, long long* begin, long long* end) {
    int64_t b = 0, e = 0;
    throw_on(arc_plan_seq_shards(kv_len, world, rank, 0, &b, &e), "plan_seq_shards");
    *begin = b;
    *end = e;
}

void allgather_merge(cudaStream_t stream, const float* record, float* gathered, int world, int batch, int nq, int hd,
                     const bf16* gate, bf16* out, void* nccl_comm) {
    throw_on(arc_sdpa_allgather_merge(record, gathered, world, batch, nq, hd, gate, out, nccl_comm, stream),
             "allgather_merge");
}

}  // namespace arcaine
