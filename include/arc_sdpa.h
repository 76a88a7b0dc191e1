/*
 * C ABI of the B200 (sm_100a) scaled-dot-product-attention library.
 *
 * These entry points are what a foreign-function binding of Arcaine's attention
 * path would bind: plain pointers, sizes and a CUDA stream handle, `int` status
 * returned, nothing thrown, nothing allocated and no synchronisation on the hot
 * path (the reference's operators are enqueue-only too, src/common/gpu/ops.hpp:96
 * "caller owns synchronization").
 *
 * Conventions shared by every call
 *   - bf16 tensors are raw 16-bit patterns (the reference's `bf16 = uint16_t`,
 *     src/common/gpu/buffer.hpp:8); all pointers are device pointers unless a
 *     comment says otherwise, 16-byte aligned.
 *   - token-major layouts of the reference: Q / O / gate (tokens, nq, hd),
 *     K / V (positions, nkv, hd); strides below are in ELEMENTS and must be
 *     multiples of 8.  The head stride is always `hd`.
 *   - GQA: kv_head = q_head / (nq / nkv)
 *     (src/common/layers/attention_layout.hpp:37-52, src/modeling/qwen3_5/kernels.hpp:637).
 *   - score = (q . k) * scale + mask, softmax in fp32
 *     (src/common/layers/attention_batched.hpp:28-44).
 *   - `stream` is a cudaStream_t passed as void*.
 */
#ifndef ARC_SDPA_H_
#define ARC_SDPA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define ARC_OK 0
#define ARC_ERR_BAD_SHAPE 1            /* non-positive size, nq % nkv != 0, ... */
#define ARC_ERR_ALIGNMENT 2            /* pointer or stride not 16-byte aligned */
#define ARC_ERR_UNSUPPORTED_HEAD_DIM 3 /* hd not in {128, 256} (attention) / {128, 256, 512} (qkv_prepare) */
#define ARC_ERR_WORKSPACE_TOO_SMALL 4
#define ARC_ERR_CUDA 5                 /* a CUDA runtime / driver call failed */
#define ARC_ERR_COLLECTIVE 6           /* NCCL missing or a collective failed (arc_sdpa_allgather_merge) */
#define ARC_ERR_DEVICE_WAIT_TIMEOUT 7  /* a bounded device-side wait gave up */
#define ARC_ERR_NULL_POINTER 8
#define ARC_ERR_UNSUPPORTED_GQA 9      /* decode: more than 16 query heads per KV head */
#define ARC_ERR_TOO_LARGE 10           /* size beyond a documented fixed limit */
#define ARC_ERR_DEVICE_BAD_RANGE 11    /* a device-side kv_len / kv_row_offset reaches past the cache (see
                                          arc_sdpa_device_status) */

/* ---- mask types: the values the reference hands to oneDNN's sdpa
 * (src/modeling/diffusion_gemma/attention.cpp:1032,1040,1099) -------------- */
#define ARC_MASK_NONE 0     /* bidirectional: canvas queries over prompt + canvas */
#define ARC_MASK_EXPLICIT 1 /* additive f32 buffer (seq, kv_len), shared by heads */
#define ARC_MASK_CAUSAL 3   /* causal, aligned bottom-right; K may be longer than Q */
#define ARC_NO_WINDOW 2147483647

const char* arc_sdpa_status_string(int status);
/* Text of the last failing CUDA call made by this thread inside the library
 * (which call, and the CUDA error string); empty if none. */
const char* arc_sdpa_last_error(void);

/* -------------------------------------------------------------------------
 * Prefill / canvas attention.  Replaces gqa_attention_sdpa
 * (src/modeling/diffusion_gemma/attention.cpp:930-995), its matmul fallback
 * gqa_attention (:706-821), batched_attention
 * (src/common/layers/attention_batched.hpp:71-136) and the seq > 1 use of
 * qwen35_xmx_attention (src/modeling/qwen3_5/kernels.hpp:761-905).
 *
 * With ARC_MASK_CAUSAL, `window` (ARC_NO_WINDOW = off) keeps only the `window`
 * most recent keys, self included — the rule of fill_causal_mask
 * (src/common/kernels/attention_mask.hpp:12-38) evaluated inline.
 * `out` may alias `q` (the reference calls the Qwen kernel that way,
 * src/modeling/qwen3_5/operators.hpp:143-147).
 * `gate` (optional): out = bf16(attn) * sigmoid(gate), the fused form of
 * mul_sigmoid_inplace (src/modeling/qwen3_5_moe/kernels.hpp:80-88).
 * `num_splits` > 1 splits the key range over several CTAs per query tile and
 * needs `workspace` of arc_sdpa_prefill_workspace_bytes(); 0 picks a value
 * (ask the size function: a non-zero answer means a workspace is required).
 * ------------------------------------------------------------------------- */
typedef struct arc_sdpa_prefill_params {
    const void* q;     /* (batch, seq, nq, hd) bf16 */
    const void* k;     /* (batch, kv_len, nkv, hd) bf16 */
    const void* v;     /* (batch, kv_len, nkv, hd) bf16 */
    void* out;         /* (batch, seq, nq, hd) bf16 */
    const void* gate;  /* optional, laid out like out */
    const float* mask; /* optional, (seq, kv_len) f32, ARC_MASK_EXPLICIT only */
    float* out_lse;    /* optional, (batch, seq, nq) f32 natural-log softmax denominator */
    int32_t batch, seq, kv_len, nq, nkv, hd;
    int64_t q_stride_b, q_stride_t; /* elements */
    int64_t k_stride_b, k_stride_t;
    int64_t v_stride_b, v_stride_t;
    int64_t o_stride_b, o_stride_t; /* also used for gate */
    float scale;
    int32_t mask_type;
    int32_t window;
    int32_t num_splits;
    void* workspace;
    size_t workspace_bytes;
    /* Gemma4's bidirectional vision blocks, evaluated inside the kernel (optional, ARC_MASK_CAUSAL only;
     * fill_causal_mask_with_block_ids, src/common/kernels/attention_mask.hpp:44-73, without the
     * (seq, kv_len) f32 buffer).  block_ids: device int32 per absolute position, -1 = text token, a
     * non-negative id for each contiguous image / video block; a query inside a block also sees the
     * block's later keys.  block_ids[block_ids_offset + j] belongs to key j, so the array must reach
     * block_ids_offset + kv_len entries; the same ids serve every sequence of the batch.  Needs
     * workspace (arc_sdpa_prefill_workspace_bytes()); head dim 128 then runs the one-tile kernel. */
    const int32_t* block_ids;
    int32_t block_ids_offset;
    /* Copies of the output (optional; no counterpart in the reference, which is single-device).
     * out_copies: DEVICE array of out_copy_count (<= 15) addresses; every output element is stored to
     * `out` and, at the same element offset, to each of them by the kernel's own epilogue.  With a
     * head-sharded prefill over several GPUs the entries are the other ranks' mapped output buffers
     * (peer access / symmetric memory), offset to this rank's head slice: the output gather then rides
     * on the kernel's stores over NVLink while it computes, instead of a collective after it.  The
     * copies are complete when the call has completed on its stream; telling the other ranks is the
     * caller's business (a barrier, a flag).  Entries must be 16-byte aligned; lse is not copied. */
    const uint64_t* out_copies;
    int32_t out_copy_count;
} arc_sdpa_prefill_params;

size_t arc_sdpa_prefill_workspace_bytes(const arc_sdpa_prefill_params* p);
int arc_sdpa_prefill(const arc_sdpa_prefill_params* p, void* stream);

/* -------------------------------------------------------------------------
 * Split-KV decode: one new query token per sequence against a contiguous
 * per-sequence KV cache (Qwen35KvLayerCache, src/modeling/qwen3_5/cache.hpp:9-14).
 * Replaces the seq == 1 use of qwen35_xmx_attention / qwen35_online_attention
 * (src/modeling/qwen3_5/kernels.hpp:621-679,761-905), the bench-only
 * qwen35_xmx_attention_decode_gqa (:910-1054) and, with `gate`, the separate
 * mul_sigmoid_inplace launch (src/modeling/qwen3_5/operators.hpp:160).
 *
 * The whole key range of the batch is cut into equal shares, one per CTA;
 * partial (out, lse) records go through `workspace` and a merge kernel.
 * Sequence b owns cache rows [row0_b, row0_b + kv_len_b) where row0_b is
 * kv_row_offset[b] if given, else b * kv_stride_b.
 * `out_f32` / `out_lse` (optional): unrounded, ungated attention output and
 * natural-log LSE per (sequence, head), the record a sequence-sharded caller
 * exchanges between GPUs before arc_sdpa_merge.
 * ------------------------------------------------------------------------- */
typedef struct arc_sdpa_decode_params {
    const void* q;    /* (batch, nq, hd) bf16, batch stride q_stride_b */
    const void* k;    /* rows of (nkv, hd) bf16 */
    const void* v;
    void* out;        /* (batch, nq, hd) bf16, batch stride o_stride_b; may be NULL */
    const void* gate; /* optional, laid out like out */
    const int32_t* kv_len;        /* device [batch]; NULL -> kv_len_uniform */
    const int64_t* kv_row_offset; /* device [batch]; NULL -> b * kv_stride_b */
    float* out_f32;               /* optional (batch, nq, hd) */
    float* out_lse;               /* optional (batch, nq) */
    int32_t batch, nq, nkv, hd;
    int32_t kv_len_uniform;
    int32_t max_kv_len; /* > 0: upper bound of any kv_len[b].  kv_len_uniform above it is refused at once; a
                           device-side kv_len[b] above it, or a sequence whose rows [row0_b, row0_b +
                           kv_len_b) reach past kv_rows_total, stops the launch's work and shows as
                           ARC_ERR_DEVICE_BAD_RANGE in arc_sdpa_device_status().  0: only the
                           kv_rows_total check */
    int64_t q_stride_b, o_stride_b; /* elements */
    int64_t kv_stride_b;            /* rows between sequences (when kv_row_offset == NULL) */
    int64_t kv_stride_t;            /* elements between consecutive rows (>= nkv*hd) */
    int64_t kv_rows_total;          /* rows addressable from k and v (extent of the cache
                                       buffers); loads never reach beyond it */
    float scale;
    int32_t num_ctas; /* 0 -> one per SM */
    void* workspace;
    size_t workspace_bytes;
    /* Sequence-sharded decode over NVLink peer memory (optional; xchg_world <= 1: off; at most 16 ranks).
     * Each of xchg_world ranks (one process per GPU) holds a slice of every sequence's keys and
     * calls this function with the same batch / heads and the same xchg_step, which starts at 1 and
     * must grow by one per call.  A rank whose slice is empty still takes part: kv_rows_total 0 with
     * kv_len NULL and kv_len_uniform 0 sends records with lse = -inf.  xchg_peers: DEVICE array of
     * xchg_world addresses, entry r = base of rank r's exchange buffer of arc_sdpa_exchange_bytes()
     * bytes, mapped into this process (peer access / symmetric memory), zero-filled before the first
     * step.  The merge kernel stores this rank's (out, lse) record into every rank's buffer as 8-byte
     * (value, step) words — a receiver recognises each word by its step, so no flag or fence follows
     * the data — then waits, bounded (about a second, after which ARC_ERR_DEVICE_WAIT_TIMEOUT shows in
     * arc_sdpa_device_status()), for the words of all ranks and writes the merged (and gated) result
     * to `out`.  `out_f32` / `out_lse`, if given, still receive this rank's own partial. */
    const uint64_t* xchg_peers;
    int32_t xchg_world, xchg_rank;
    uint32_t xchg_step;
    int64_t xchg_wait_cycles; /* SM clocks the merge waits for the other ranks' records; 0 = about a second */
} arc_sdpa_decode_params;

/* Bytes of one rank's exchange buffer for sequence-sharded decode. */
size_t arc_sdpa_exchange_bytes(int32_t world, int32_t batch, int32_t nq, int32_t hd);

size_t arc_sdpa_decode_workspace_bytes(const arc_sdpa_decode_params* p);
int arc_sdpa_decode(const arc_sdpa_decode_params* p, void* stream);

/* -------------------------------------------------------------------------
 * arc_sdpa_decode without a workspace.  No counterpart in the reference: it
 * exists for callers that cannot obtain device scratch themselves — a server
 * whose planner has already given all GPU memory to its own arena, or a thin
 * foreign-language binding with no device allocator — and for loops where a
 * cudaMalloc (which stalls the device) is not acceptable.
 *
 * Same parameters and results as arc_sdpa_decode; `workspace` and
 * `workspace_bytes` are ignored.  The partial records go to an array of
 * ARC_STATIC_SCRATCH_BYTES built into the library image (each GPU that loads
 * the library holds it until the process exits).  The call allocates nothing:
 * no cudaMalloc / cudaFree, no allocating library routine.
 *   - Shapes whose arc_sdpa_decode_workspace_bytes() exceeds
 *     ARC_STATIC_SCRATCH_BYTES are refused with ARC_ERR_TOO_LARGE
 *     (arc_sdpa_last_error() gives both sizes).
 *   - The first call on each device resolves the array's device address; make
 *     that first call before starting any stream capture on that device.
 *   - All calls on a device share the one array, which keeps whatever the last
 *     call left in it.  Nothing needs clearing between calls — a call writes
 *     every record it later reads — but two calls that overlap on the GPU
 *     (different streams, no ordering between them) race on it: keep them on one
 *     stream or order them with events.
 * ------------------------------------------------------------------------- */
#define ARC_STATIC_SCRATCH_BYTES (8u << 20)
int arc_sdpa_decode_static(const arc_sdpa_decode_params* p, void* stream);

/* -------------------------------------------------------------------------
 * Log-sum-exp merge of `num_parts` partial results over disjoint key ranges
 * (no counterpart in the reference, which never splits the key range):
 *   lse = log sum_c exp(lse_c),  out = sum_c exp(lse_c - lse) * o_c.
 * part_out (num_parts, rows, hd) f32, part_lse (num_parts, rows) f32; part c
 * starts part_out_stride / part_lse_stride ELEMENTS after part c-1 (0 = dense:
 * rows*hd and rows), so a packed per-rank record [out | lse] can be merged in
 * place after an all-gather.
 * Outputs (each optional): out_bf16 (rows, hd) with the optional sigmoid gate
 * (rows, hd) bf16 applied, out_f32 (rows, hd) ungated, out_lse (rows).
 * ------------------------------------------------------------------------- */
int arc_sdpa_merge(const float* part_out, const float* part_lse, int32_t num_parts, int64_t rows,
                   int32_t hd, int64_t part_out_stride, int64_t part_lse_stride, const void* gate,
                   void* out_bf16, float* out_f32, float* out_lse, void* stream);

/* a[i] = bf16(f32(a[i]) * sigmoid(f32(gate[i]))): mul_sigmoid_inplace,
 * src/modeling/qwen3_5_moe/kernels.hpp:80-88. */
int arc_mul_sigmoid_inplace(void* a, const void* gate, int64_t n, void* stream);

/* Additive causal / sliding-window mask buffer: fill_causal_mask,
 * src/common/kernels/attention_mask.hpp:12-38.  mask is (q_len, kv_len) f32. */
int arc_fill_causal_mask(float* mask, int32_t q_len, int32_t kv_len, int32_t past_offset,
                         int32_t sliding_window, void* stream);

/* The same plus Gemma4's bidirectional vision blocks: fill_causal_mask_with_block_ids,
 * src/common/kernels/attention_mask.hpp:44-73.  block_ids is a device int32 array
 * indexed by absolute position (-1 = text token); tokens with the same
 * non-negative id see each other in both directions.  NULL = plain causal.
 * Pass the result to arc_sdpa_prefill with mask_type 1. */
int arc_fill_causal_mask_with_block_ids(float* mask, const int32_t* block_ids, int32_t q_len, int32_t kv_len,
                                        int32_t past_offset, int32_t sliding_window, void* stream);

/* ---------------------------------------------------------------------------
 * Pre-processing of the projected Q / K / V rows and the KV-cache append, one
 * launch.  Replaces, for one layer call: rms_norm / rms_norm_no_scale
 * (src/common/kernels/rms_norm.hpp:9-56), fused_norm_rope_inplace and
 * apply_rope (src/modeling/diffusion_gemma/attention_kernels.hpp:99-153,
 * attention.cpp:529-610) and the two cache memcpys (attention.cpp:1017-1020;
 * src/modeling/qwen3_5/operators.hpp:136-140).
 *
 * Per (token, head) row of hd bf16 values v:
 *   y = bf16(v * rsqrt(mean(v^2) + eps) * weight)        (weight NULL: unit scale)
 *   Q and K rows, pairs p < n_active_pairs:  y[p]        = bf16(y0 c - y1 s)
 *                                            y[p + hd/2] = bf16(y0 s + y1 c)
 *   with (c, s) = rope_cos/rope_sin[token * n_active_pairs + p], or, tables NULL,
 *   cos/sin((pos + token) / theta^(2p/hd)) in fp32.
 * Q is rewritten in place; K rows go to k_dst, V rows (unit scale, no rotation)
 * to v_dst — pass the cache address of the first appended position, with the
 * cache's row stride, and the append costs no copy.  v_src NULL with v_dst set:
 * V is taken from k_src before its norm (the full-attention layers' shared K/V
 * projection, attention.cpp:587-595); k_dst must then differ from k_src
 * (ARC_ERR_BAD_SHAPE otherwise: an in-place K would be normalised under V's
 * feet).  q NULL, or k_src NULL, skips that part.  Token strides must hold a
 * token's heads (>= heads * hd); negative strides are refused.
 * hd in {128, 256, 512}; strides in elements, multiples of 8; all pointers
 * 16-byte aligned.
 * ------------------------------------------------------------------------- */
typedef struct arc_qkv_prepare_params {
    void* q;              /* (batch, seq, nq, hd) bf16, in place; or NULL */
    const void* k_src;    /* (batch, seq, nkv, hd) bf16; or NULL */
    const void* v_src;    /* (batch, seq, nkv, hd) bf16; or NULL */
    void* k_dst;          /* first destination row of K (cache + past_len * row) */
    void* v_dst;          /* first destination row of V; or NULL */
    const void* q_weight; /* [hd] bf16 or NULL */
    const void* k_weight; /* [hd] bf16 or NULL */
    const float* rope_cos;    /* (seq, n_active_pairs) f32, or NULL: computed from theta */
    const float* rope_sin;
    const int32_t* pos_offset; /* device int32[batch]: position of each sequence's first token; or NULL */
    int32_t batch, seq, nq, nkv, hd;
    int32_t n_active_pairs;   /* int(partial_rotary_factor * hd / 2); 0: no rotation */
    int64_t q_stride_b, q_stride_t;
    int64_t k_src_stride_b, k_src_stride_t;
    int64_t v_src_stride_b, v_src_stride_t;
    int64_t k_dst_stride_b, k_dst_stride_t;
    int64_t v_dst_stride_b, v_dst_stride_t;
    int64_t rope_stride_b;    /* elements between two sequences' tables; 0: one table for all */
    int32_t pos0;             /* position of the first token when pos_offset is NULL */
    float theta;
    float eps;
    /* Qwen3.5 form (qwen35_apply_mrope, src/modeling/qwen3_5/kernels.hpp:576-617; call site
     * src/modeling/qwen3_5/operators.hpp:127-140).  All zero / NULL = the form described above. */
    int32_t rot_half;         /* distance between the two values of a rotation pair; 0 = hd / 2.  Otherwise
                               * a power of two, >= 8 and <= hd / 4 (pairs (f, f + rotary_dim / 2)) */
    int32_t freq_denom;       /* denominator of the frequency exponent 2 f / denom; 0 = hd (Qwen3.5: rotary_dim) */
    const int32_t* mrope_positions; /* device int32 (batch, 3, seq): position of every token on the temporal /
                               * height / width axis; NULL = one position per token (pos_offset / pos0) */
    int32_t mrope_section[3]; /* frequency f takes axis a in {1, 2} when a <= f < 3 * section[a] and f % 3 == a,
                               * else axis 0 */
    int32_t v_copy;           /* 1: V rows are appended as they are (no unit-RMS norm) */
} arc_qkv_prepare_params;

int arc_qkv_prepare(const arc_qkv_prepare_params* p, void* stream);

/* ---------------------------------------------------------------------------
 * Multi-GPU helpers (one process per GPU).  No counterpart in the reference, whose two GPUs split
 * layers and copy activations through host memory (src/modeling/diffusion_gemma/model.cpp:33-46);
 * these give a C or C++ host the partitions and the record exchange without Python.
 * ------------------------------------------------------------------------- */

/* Prefill / canvas: KV heads first (with their nq / nkv query heads), then whole sequences, dealt to
 * `world` ranks: world = head_ways x batch_ways with head_ways the largest divisor of world that
 * divides nkv.  Rank `rank` owns KV heads [kv_head_begin, kv_head_end), query heads
 * [q_head_begin, q_head_end) and sequences [batch_begin, batch_end) (possibly none). */
typedef struct arc_head_shard {
    int32_t kv_head_begin, kv_head_end;
    int32_t q_head_begin, q_head_end;
    int32_t batch_begin, batch_end;
} arc_head_shard;
int arc_plan_head_shards(int32_t nq, int32_t nkv, int32_t batch, int32_t world, int32_t rank, arc_head_shard* out);

/* Long-context decode: contiguous key range [*begin, *end) of rank `rank`, boundaries on multiples of
 * `align` keys (0 = 64).  Short sequences leave the last ranks an empty range (kv_len, kv_len). */
int arc_plan_seq_shards(int64_t kv_len, int32_t world, int32_t rank, int32_t align, int64_t* begin, int64_t* end);

/* Batched decode: whole sequences dealt to ranks longest first, each to the rank with the fewest keys so
 * far, so that the ranks read about the same number of keys.  kv_len: HOST array [batch];
 * owner: HOST array [batch], owner[b] = rank of sequence b. */
int arc_plan_batch_shards(const int32_t* kv_len, int32_t batch, int32_t world, int32_t* owner);

/* Exchange buffer of the in-kernel record exchange (arc_sdpa_decode_params.xchg_*): clears this rank's
 * buffer (its flags must be zero before the first step; every rank must have done this, and the ranks
 * must have met on the host, before anyone's first step) and copies the `world` peer addresses the caller
 * mapped (peer access, IPC or symmetric memory; peers[rank] = this rank's own buffer) into the device
 * array `peers_dev` [world] that xchg_peers points to.  Enqueued on `stream`. */
int arc_sdpa_exchange_init(void* buffer, int32_t world, int32_t batch, int32_t nq, int32_t hd, const uint64_t* peers,
                           uint64_t* peers_dev, void* stream);

/* The collective form of the same exchange: ncclAllGather of this rank's packed record
 * [out f32 (batch, nq, hd) | lse f32 (batch, nq) | padding to a multiple of 4 floats]
 * (arc_sdpa_record_floats() floats, as arc_sdpa_decode writes it through out_f32 / out_lse when they point
 * into one buffer) into `gathered` (world records), then the log-sum-exp merge with the optional gate
 * into out_bf16 (batch, nq, hd).  `comm` is an ncclComm_t; the NCCL library already loaded in the process
 * is used (else libnccl.so.2 is loaded).  ARC_ERR_COLLECTIVE if NCCL is missing or reports an error. */
size_t arc_sdpa_record_floats(int32_t batch, int32_t nq, int32_t hd);
int arc_sdpa_allgather_merge(const float* record, float* gathered, int32_t world, int32_t batch, int32_t nq, int32_t hd,
                             const void* gate, void* out_bf16, void* comm, void* stream);

/* Device-side status of the current device: ARC_OK, ARC_ERR_DEVICE_WAIT_TIMEOUT (the first bounded
 * wait that gave up since the last clear; fault_code says which kind, fault_detail where) or
 * ARC_ERR_DEVICE_BAD_RANGE (fault_detail = the sequence).  While a status is set, launches
 * return at once without doing their work.  Synchronises the device. */
int arc_sdpa_device_status(uint32_t* fault_code, uint32_t* fault_detail);
int arc_sdpa_clear_device_status(void);

/* Number of kernels this library has launched in this process (all devices). */
uint64_t arc_sdpa_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* ARC_SDPA_H_ */
