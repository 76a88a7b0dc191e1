// C++ host interface of the attention path, shaped like the reference's own
// free functions so a call site changes its context type and nothing else:
// raw device pointers to bf16-as-uint16_t, int dimensions, enqueue-only on the
// engine's stream, std::runtime_error on failure.  Every function forwards to
// the C ABI in include/arc_sdpa.h; there is no other backend and no CPU path.
//
//   reference                                              here
//   GpuEngine {engine, stream, queue, index}               CudaEngine {index, stream}
//     (src/common/gpu/engine.hpp:10-19)
//   diffarena::Alloc<bf16> result from the per-GPU arena   caller-provided `out`
//     (src/modeling/diffusion_gemma/attention.cpp:940-942)
#pragma once
#include <cuda_runtime.h>

#include "../../include/arc_sdpa.h"

#include <climits>
#include <cstddef>
#include <cstdint>

namespace arcaine {

using bf16 = uint16_t;  // raw bits, src/common/gpu/buffer.hpp:8

// Stand-in for GpuEngine: which GPU, and the in-order stream work is enqueued on.
struct CudaEngine {
    int index = 0;
    cudaStream_t stream = nullptr;
};

// Grow-only device scratch for split-KV partials.  The reference learned that
// per-call allocation costs throughput (persistent attention scratch, notes/
// diffusion_gemma/NVFP4_DPAS_KERNEL.md:243-250); this buffer reallocates only
// when a call needs more than any call before it.
class SdpaWorkspace {
public:
    SdpaWorkspace() = default;
    // A region the caller owns (an arena slice sized from arc_sdpa_*_workspace_bytes): never freed or grown
    // here; a call that needs more throws.
    SdpaWorkspace(void* borrowed, size_t bytes) : ptr_(borrowed), bytes_(bytes), owned_(false) {}
    ~SdpaWorkspace();
    SdpaWorkspace(const SdpaWorkspace&) = delete;
    SdpaWorkspace& operator=(const SdpaWorkspace&) = delete;
    void* reserve(size_t bytes);  // throws std::runtime_error on allocation failure
    size_t capacity() const { return bytes_; }

private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
    bool owned_ = true;
};

// src/modeling/diffusion_gemma/attention.cpp:930-995.  O = softmax(Q K^T + mask) V,
// no scale (Q and K arrive RMS-normed), GQA with nkv KV heads.  mask_type: 0 none,
// 1 explicit additive f32 (seq, kv_len), 3 causal aligned bottom-right.
void gqa_attention_sdpa(CudaEngine& ctx, const bf16* Q, int seq, int nq, int hd, const bf16* Kc,
                        const bf16* Vc, int kv_len, int nkv, const float* mask, int mask_type, bf16* out,
                        SdpaWorkspace& ws);

// src/modeling/diffusion_gemma/attention.cpp:706-821.  Same result through inline
// causal / sliding-window masking: query i sits at absolute position
// past_offset + i, key 0 at past_offset - (kv_len - seq).
void gqa_attention(CudaEngine& ctx, const bf16* Q, int seq, int nq, int hd, const bf16* Kc, const bf16* Vc,
                   int kv_len, int nkv, int past_offset, int sliding_window, bool causal, bf16* out,
                   SdpaWorkspace& ws);

// src/common/layers/attention_batched.hpp:71-136.  scores*scale + causal/window
// mask (skip_mask: no mask).  block_ids (device int32 per absolute position, -1 = text): Gemma4's
// bidirectional vision blocks (src/common/kernels/attention_mask.hpp:44-73), evaluated inside the
// kernel; key j of K_dev sits at absolute position past_offset - (kv_len - seq_len) + j.
void batched_attention(CudaEngine& ctx, const bf16* Q_dev, int seq_len, int nq_heads, int q_head_dim,
                       const bf16* K_dev, const bf16* V_dev, int kv_len, int nkv_heads, int kv_head_dim,
                       int past_offset, int sliding_window, float scale, bool skip_mask,
                       const int32_t* block_ids, bf16* out, SdpaWorkspace& ws);

// sliding_decode_attention, src/modeling/gemma4_unified/attention.cpp:93-137: one token over cache rows
// [kv_start, kv_start + kv_len), no scale.  Takes the token-major cache (max_seq, nkv, hd) of
// src/modeling/gemma4_unified/kv_cache.hpp:8-9 directly: the head-major K copy and the transposed V copy the
// reference keeps for its strided GEMMs (kv_cache.hpp:10-11) are not needed.
void gemma4_sliding_decode_attention(CudaEngine& ctx, const bf16* Q_dev, const bf16* K_cache, const bf16* V_cache,
                                     int kv_len, int kv_start, int nq_heads, int nkv_heads, int head_dim, bf16* out,
                                     SdpaWorkspace& ws);

// src/modeling/qwen3_5/kernels.hpp:621-679 / 761-905.  Causal GQA attention of
// `seq` new tokens over a cache holding past + seq positions; `output` may alias
// `query`.  seq == 1 takes the split-KV decode kernel, seq > 1 the prefill kernel.
void qwen35_xmx_attention(cudaStream_t stream, const bf16* query, const bf16* key, const bf16* value,
                          bf16* output, int seq, int past, int query_heads, int key_heads, int head_dim,
                          float scale, SdpaWorkspace& ws);
void qwen35_online_attention(cudaStream_t stream, const bf16* query, const bf16* key, const bf16* value,
                             bf16* output, int seq, int past, int query_heads, int key_heads, int head_dim,
                             float scale, SdpaWorkspace& ws);

// src/modeling/qwen3_5/kernels.hpp:910-1054 (single-token decode), with the
// sigmoid output gate of src/modeling/qwen3_5/operators.hpp:160 optionally fused
// (gate == nullptr: plain attention).
void qwen35_xmx_attention_decode_gqa(cudaStream_t stream, const bf16* query, const bf16* key,
                                     const bf16* value, bf16* output, int past, int query_heads,
                                     int key_heads, int head_dim, float scale, const bf16* gate,
                                     SdpaWorkspace& ws);

// src/modeling/qwen3_5_moe/kernels.hpp:80-88
void mul_sigmoid_inplace(cudaStream_t stream, bf16* a, const bf16* gate, size_t n);

// src/common/kernels/attention_mask.hpp:12-38
void fill_causal_mask(cudaStream_t stream, float* mask, int q_len, int kv_len, int past_offset,
                      int sliding_window);

// src/common/kernels/rms_norm.hpp:9-56 (weight == nullptr: rms_norm_no_scale).  H in {128, 256, 512}.
void rms_norm(cudaStream_t stream, const bf16* x, const bf16* weight, bf16* out, int rows, int H, float eps);

// src/modeling/diffusion_gemma/attention_kernels.hpp:99-153.  rope_cos / rope_sin: (seq, n_active_pairs)
// tables or nullptr (angles computed from theta).
void fused_norm_rope_inplace(cudaStream_t stream, bf16* x, const bf16* weight, int seq, int nheads, int hd,
                             int offset, float theta, float partial, float eps, const float* rope_cos,
                             const float* rope_sin);

// The post-projection half of project_qkv plus the cache append of encoder_attention_forward
// (src/modeling/diffusion_gemma/attention.cpp:529-610, 1017-1020) in one launch: Q normed and rotated in
// place, K normed and rotated and V unit-normed straight into cache rows past_len .. past_len + seq of
// (max_seq, nkv, hd) caches.  v == nullptr: V is taken from the raw K projection (full-attention layers).
void qkv_norm_rope_append(cudaStream_t stream, bf16* Q, const bf16* K, const bf16* V, bf16* k_cache, bf16* v_cache,
                          int seq, int past_len, int nq, int nkv, int hd, const bf16* q_norm, const bf16* k_norm,
                          float theta, float partial, float eps, const float* rope_cos, const float* rope_sin);

// Qwen3.5 layer call (src/modeling/qwen3_5/operators.hpp:127-140) in one launch: rms_norm of Q and K with
// their weights, qwen35_apply_mrope (src/modeling/qwen3_5/kernels.hpp:585-617) and the two cache memcpys.
// positions: device int32 (3, seq); sections: the three mrope_section values.
void qwen35_norm_mrope_append(cudaStream_t stream, bf16* query, const bf16* key, const bf16* value, bf16* key_cache,
                              bf16* value_cache, const int32_t* positions, int seq, int past, int query_heads,
                              int key_heads, int head_dim, int rotary_dim, float theta, const int sections[3],
                              const bf16* q_norm, const bf16* k_norm, float eps);

// ---- multi-GPU (one process per GPU): thin forms of the C helpers that throw like the calls above ----

// Which KV heads (with their query heads) and sequences rank `rank` of `world` computes in a prefill.
arc_head_shard plan_head_shards(int nq, int nkv, int batch, int world, int rank);
// Key range [begin, end) of rank `rank` in a sequence-sharded decode.
void plan_seq_shards(long long kv_len, int world, int rank, long long* begin, long long* end);
// Sequence-sharded decode through NCCL: `record` is this rank's packed [out f32 | lse f32] partial
// (arc_sdpa_record_floats() floats, written by arc_sdpa_decode through out_f32 / out_lse), `gathered` room
// for `world` of them; all-gather, merge, optional gate.  Replaces the host-staged copies between GPUs of
// src/modeling/diffusion_gemma/model.cpp:33-46 for this path.
void allgather_merge(cudaStream_t stream, const float* record, float* gathered, int world, int batch, int nq, int hd,
                     const bf16* gate, bf16* out, void* nccl_comm);

}  // namespace arcaine
