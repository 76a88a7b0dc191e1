/*
 * CPU restatement of Arcaine's attention hot path.  TEST INFRASTRUCTURE ONLY:
 * this file is the checker for the CUDA kernels (tests, the smoke run and the
 * CPU-baseline leg of the benchmark); the product never calls it.
 *
 * PARITY UNPINNED: the reference ships no attention test, golden vector or
 * known-answer fixture, and its own implementation (SYCL + oneDNN) cannot be
 * built without a DPC++ toolchain.  The functions below restate the
 * reference's arithmetic from its sources and are cross-checked only against
 * each other and against independent fp32 formulations.
 *
 * Every function cites the reference source it follows (path inside the
 * Arcaine project, file:line).  bf16 values travel as raw uint16_t bits, the
 * reference's own convention (src/common/gpu/buffer.hpp:8).
 *
 * Layouts (all contiguous, row-major):
 *   Q, O, gate : (seq, nq, hd)      K, V : (kv_len, nkv, hd)
 * Batched variants add a leading batch dimension with explicit strides.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <limits.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---- bf16 <-> f32 : src/common/gpu/buffer.hpp:10-23 ---------------------- */
ORACLE_API float oracle_bf16_to_float(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* Round to nearest even by bias add; like the reference, no NaN special case. */
ORACLE_API uint16_t oracle_float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t bias = ((u >> 16) & 1u) + 0x7FFFu;
    return (uint16_t)((u + bias) >> 16);
}

static inline float b2f(uint16_t v) { return oracle_bf16_to_float(v); }
static inline uint16_t f2b(float f) { return oracle_float_to_bf16(f); }

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* The launcher of a multi-process run pins OMP_NUM_THREADS to 1; the timed CPU baseline asks for
 * the host's cores explicitly. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ---- bench input recipe : src/bench/qwen35_attention_bench.cpp:86-94 ----- */
/* LCG state*1664525+1013904223; x = (((state>>16)&1023) - 512)/1024 -> bf16.
 * `state` is carried across calls so Q, K, V can be filled in that order. */
ORACLE_API void oracle_lcg_fill(uint16_t* dst, size_t n, uint32_t* state) {
    uint32_t s = *state;
    for (size_t i = 0; i < n; ++i) {
        s = s * 1664525u + 1013904223u;
        float x = (float)((int)((s >> 16) & 1023u) - 512) / 1024.0f;
        dst[i] = f2b(x);
    }
    *state = s;
}

/* ---- additive mask : src/common/kernels/attention_mask.hpp:12-38 --------- */
/* mask[qi][kvj] = -inf if the key is in the future of the query or falls
 * out of the `sliding_window` most recent positions (self included), else 0.
 * sliding_window == INT_MAX disables the window. */
ORACLE_API void oracle_fill_causal_mask(float* mask, int q_len, int kv_len,
                                        int past_offset, int sliding_window) {
    for (int qi = 0; qi < q_len; ++qi) {
        for (int kvj = 0; kvj < kv_len; ++kvj) {
            int q_global = past_offset + qi;
            int kv_global = past_offset - (kv_len - q_len) + kvj;
            int causal = kv_global > q_global;
            int too_far = (sliding_window != INT_MAX) &&
                          (kv_global < q_global - sliding_window + 1);
            mask[(size_t)qi * kv_len + kvj] = (causal || too_far) ? -INFINITY : 0.0f;
        }
    }
}

/* The same with Gemma4's vision blocks: src/common/kernels/attention_mask.hpp:44-73.
 * block_ids[pos] is -1 for text and a non-negative id per image / video block; tokens
 * of one block see each other in both directions. */
ORACLE_API void oracle_fill_causal_mask_with_block_ids(float* mask, const int32_t* block_ids, int q_len,
                                                       int kv_len, int past_offset, int sliding_window) {
    for (int qi = 0; qi < q_len; ++qi) {
        for (int kvj = 0; kvj < kv_len; ++kvj) {
            int q_global = past_offset + qi;
            int kv_global = past_offset - (kv_len - q_len) + kvj;
            int q_block = block_ids ? block_ids[q_global] : -1;
            int kv_block = block_ids ? block_ids[kv_global] : -1;
            int same = q_block >= 0 && q_block == kv_block;
            int causal = !same && kv_global > q_global;
            int too_far = (sliding_window != INT_MAX) &&
                          (kv_global < q_global - sliding_window + 1);
            mask[(size_t)qi * kv_len + kvj] = (causal || too_far) ? -INFINITY : 0.0f;
        }
    }
}

/* Visible key span [lo, hi) of one query row.  mask_type follows the values
 * the reference passes to oneDNN (src/modeling/diffusion_gemma/attention.cpp:
 * 1032,1040,1099): 0 = none, 1 = explicit additive buffer, 3 = causal aligned
 * bottom-right (K may be longer than Q).  `window` (INT_MAX or <= 0 = off)
 * narrows the causal span to the `window` most recent keys, self included,
 * exactly as oracle_fill_causal_mask does. */
static inline void row_span(int mask_type, int window, int seq, int kv_len, int qi,
                            int* lo, int* hi) {
    *lo = 0;
    *hi = kv_len;
    if (mask_type == 3) {
        int diag = qi + (kv_len - seq); /* last visible key */
        int h = diag + 1;
        if (h < 0) h = 0;
        *hi = h < kv_len ? h : kv_len;
        if (window != INT_MAX && window > 0) {
            int l = diag - window + 1;
            *lo = l > 0 ? l : 0;
        }
        if (*lo > *hi) *lo = *hi;
    }
}

/* ---- gate : src/modeling/qwen3_5_moe/kernels.hpp:80-88 ------------------- */
ORACLE_API void oracle_mul_sigmoid_inplace(uint16_t* a, const uint16_t* gate, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float g = b2f(gate[i]);
        float sig = 1.0f / (1.0f + expf(-g));
        a[i] = f2b(b2f(a[i]) * sig);
    }
}

/* ---- RMSNorm (+ RoPE) of one tensor of (tokens, heads, hd) rows -----------
 * rms_norm: src/common/kernels/rms_norm.hpp:9-49 (weight NULL = rms_norm_no_scale);
 * rotation and rounding order: fused_norm_rope_inplace,
 * src/modeling/diffusion_gemma/attention_kernels.hpp:99-153 — the normalised value is
 * rounded to bf16, then pairs (p, p + hd/2), p < n_active_pairs, are rotated by the
 * table entry [token * n_active_pairs + p] or, table NULL, by
 * angle = (offset + token) / theta^(2p/hd) evaluated in fp32.  The sum of squares is
 * taken in double here (the reference reduces in fp32 in work-group order): the
 * result can differ from any fp32 evaluation by one bf16 step in rare elements.
 * src and dst may alias; strides are in elements between tokens. */
ORACLE_API void oracle_norm_rope(const uint16_t* src, long long src_stride_t, uint16_t* dst,
                                 long long dst_stride_t, const uint16_t* weight, int tokens, int heads,
                                 int hd, int n_active_pairs, int offset, float theta, float eps,
                                 const float* rope_cos, const float* rope_sin) {
    const int half = hd / 2;
    for (int t = 0; t < tokens; ++t) {
        for (int h = 0; h < heads; ++h) {
            const uint16_t* x = src + (long long)t * src_stride_t + (long long)h * hd;
            uint16_t* y = dst + (long long)t * dst_stride_t + (long long)h * hd;
            double ss = 0.0;
            for (int d = 0; d < hd; ++d) {
                double v = b2f(x[d]);
                ss += v * v;
            }
            const float rms_inv = (float)(1.0 / sqrt(ss / (double)hd + (double)eps));
            float row[1024];
            for (int d = 0; d < hd; ++d) {
                float v = b2f(x[d]) * rms_inv;
                if (weight) v *= b2f(weight[d]);
                row[d] = b2f(f2b(v));
            }
            for (int p = 0; p < n_active_pairs; ++p) {
                float c, sn;
                if (rope_cos) {
                    c = rope_cos[(long long)t * n_active_pairs + p];
                    sn = rope_sin[(long long)t * n_active_pairs + p];
                } else {
                    float inv_freq = 1.0f / powf(theta, 2.0f * (float)p / (float)hd);
                    float angle = (float)(offset + t) * inv_freq;
                    c = cosf(angle);
                    sn = sinf(angle);
                }
                const float x0 = row[p], x1 = row[p + half];
                row[p] = x0 * c - x1 * sn;
                row[p + half] = x0 * sn + x1 * c;
            }
            for (int d = 0; d < hd; ++d) y[d] = f2b(row[d]);
        }
    }
}

/* ---- Qwen3.5 multi-axis RoPE : src/modeling/qwen3_5/kernels.hpp:576-617 ----
 * In place on (tokens, heads, head_dim) rows: pairs (f, f + rotary_dim/2), f < rotary_dim/2,
 * angle = positions[axis(f)][token] / theta^(2 f / rotary_dim), where a frequency takes axis
 * a in {1, 2} when a <= f < 3 * sections[a] and f % 3 == a, else axis 0.  positions is
 * (3, tokens). */
static int mrope_axis(int frequency, const int* sections) {
    for (int axis = 1; axis <= 2; ++axis) {
        int limit = sections[axis] * 3;
        if (frequency >= axis && frequency < limit && frequency % 3 == axis) return axis;
    }
    return 0;
}

ORACLE_API void oracle_mrope(uint16_t* x, const int32_t* positions, int tokens, int heads, int head_dim,
                             int rotary_dim, float theta, const int* sections) {
    const int half = rotary_dim / 2;
    for (int t = 0; t < tokens; ++t)
        for (int h = 0; h < heads; ++h) {
            uint16_t* row = x + ((size_t)t * heads + h) * head_dim;
            for (int f = 0; f < half; ++f) {
                int axis = mrope_axis(f, sections);
                int position = positions[(size_t)axis * tokens + t];
                float inv = 1.0f / powf(theta, 2.0f * (float)f / (float)rotary_dim);
                float angle = (float)position * inv;
                float c = cosf(angle), sn = sinf(angle);
                float x0 = b2f(row[f]), x1 = b2f(row[f + half]);
                row[f] = f2b(x0 * c - x1 * sn);
                row[f + half] = f2b(x0 * sn + x1 * c);
            }
        }
}

/* ---- grading oracle: fp32-softmax SDPA ------------------------------------
 * O = softmax(scale * Q K^T + mask) V on the bf16-valued inputs, with GQA
 * kv_head = q_head / (nq / nkv) (src/common/layers/attention_layout.hpp:37-52,
 * src/modeling/qwen3_5/kernels.hpp:637), scale placed as in
 * src/common/layers/attention_batched.hpp:28-44 (score*scale + mask).
 * Products of two bf16 values are exact in fp32; sums run in double so the
 * result is the reference point, not one more rounding of it.
 * Optional outputs: out_f32 (unrounded), out_bf16 (RNE), lse (natural log of
 * the softmax denominator, including the row maximum).  When `gate` is given,
 * the bf16 output is multiplied as oracle_mul_sigmoid_inplace does (attention
 * result rounded to bf16 first, src/modeling/qwen3_5/operators.hpp:143-160)
 * and out_f32 holds attention * sigmoid(gate) without the intermediate
 * rounding.
 * rows == NULL: every (token, head) row; else `n_rows` flat row indices
 * token*nq + head, outputs packed in that order. */
ORACLE_API int oracle_sdpa_f32(const uint16_t* Q, const uint16_t* K, const uint16_t* V,
                               const uint16_t* gate, const float* mask, int mask_type,
                               int window, int seq, int kv_len, int nq, int nkv, int hd,
                               float scale, const int64_t* rows, int64_t n_rows,
                               float* out_f32, uint16_t* out_bf16, float* lse) {
    if (nkv <= 0 || nq % nkv != 0 || hd <= 0 || hd > 1024) return -1;
    if (mask_type == 1 && mask == NULL) return -2;
    int64_t total = rows ? n_rows : (int64_t)seq * nq;
    int g = nq / nkv;
    int err = 0;
#pragma omp parallel
    {
        double* p = (double*)malloc(sizeof(double) * (size_t)(kv_len > 0 ? kv_len : 1));
        double* acc = (double*)malloc(sizeof(double) * (size_t)hd);
        float* qf = (float*)malloc(sizeof(float) * (size_t)hd);
        if (!p || !acc || !qf) {
#pragma omp atomic write
            err = -3;
        } else {
#pragma omp for schedule(dynamic, 4)
            for (int64_t r = 0; r < total; ++r) {
                int64_t flat = rows ? rows[r] : r;
                int t = (int)(flat / nq);
                int h = (int)(flat % nq);
                int kh = h / g;
                const uint16_t* qrow = Q + ((size_t)t * nq + h) * hd;
                for (int d = 0; d < hd; ++d) qf[d] = b2f(qrow[d]);
                int lo, hi;
                row_span(mask_type, window, seq, kv_len, t, &lo, &hi);
                double m = -INFINITY;
                for (int j = lo; j < hi; ++j) {
                    const uint16_t* krow = K + ((size_t)j * nkv + kh) * hd;
                    double dot = 0.0;
#pragma omp simd reduction(+ : dot)
                    for (int d = 0; d < hd; ++d) dot += (double)(qf[d] * b2f(krow[d]));
                    double s = dot * (double)scale;
                    if (mask_type == 1) s += (double)mask[(size_t)t * kv_len + j];
                    p[j] = s;
                    if (s > m) m = s;
                }
                for (int d = 0; d < hd; ++d) acc[d] = 0.0;
                double z = 0.0;
                if (m > -INFINITY) {
                    for (int j = lo; j < hi; ++j) {
                        double e = exp(p[j] - m);
                        if (e == 0.0) continue;
                        z += e;
                        const uint16_t* vrow = V + ((size_t)j * nkv + kh) * hd;
#pragma omp simd
                        for (int d = 0; d < hd; ++d) acc[d] += e * (double)b2f(vrow[d]);
                    }
                }
                double inv = z > 0.0 ? 1.0 / z : 0.0;
                if (lse) lse[r] = z > 0.0 ? (float)(m + log(z)) : -INFINITY;
                for (int d = 0; d < hd; ++d) {
                    float o = (float)(acc[d] * inv);
                    if (gate) {
                        float gv = b2f(gate[((size_t)t * nq + h) * hd + d]);
                        float sig = 1.0f / (1.0f + expf(-gv));
                        if (out_f32) out_f32[(size_t)r * hd + d] = o * sig;
                        if (out_bf16) out_bf16[(size_t)r * hd + d] = f2b(b2f(f2b(o)) * sig);
                    } else {
                        if (out_f32) out_f32[(size_t)r * hd + d] = o;
                        if (out_bf16) out_bf16[(size_t)r * hd + d] = f2b(o);
                    }
                }
            }
        }
        free(p);
        free(acc);
        free(qf);
    }
    return err;
}

/* ---- scalar online-softmax kernel : src/modeling/qwen3_5/kernels.hpp:621-679
 * Causal GQA attention, one key at a time: query token t sees keys
 * 0 .. past+t; fp32 running max / sum / accumulator, expf, score = dot*scale,
 * final acc/sum rounded to bf16.  The reference reduces the dot product with
 * a 256-wide binary tree in local memory; the same tree order is kept here so
 * the fp32 sums round identically (head_dim <= 256, zero padded). */
ORACLE_API int oracle_qwen35_online_attention(const uint16_t* query, const uint16_t* key,
                                              const uint16_t* value, uint16_t* output,
                                              int seq, int past, int query_heads,
                                              int key_heads, int head_dim, float scale) {
    if (head_dim > 256) return -1;
    if (key_heads <= 0 || query_heads % key_heads != 0) return -2;
    int64_t total = (int64_t)seq * query_heads;
#pragma omp parallel for schedule(dynamic, 2)
    for (int64_t grp = 0; grp < total; ++grp) {
        int token = (int)(grp / query_heads);
        int qh = (int)(grp % query_heads);
        int kh = qh / (query_heads / key_heads);
        float reduce[256];
        float out_acc[256];
        for (int d = 0; d < 256; ++d) out_acc[d] = 0.0f;
        float running_max = -INFINITY, running_sum = 0.0f;
        const uint16_t* qrow = query + ((size_t)token * query_heads + qh) * head_dim;
        int visible = past + token + 1;
        for (int pos = 0; pos < visible; ++pos) {
            const uint16_t* krow = key + ((size_t)pos * key_heads + kh) * head_dim;
            for (int d = 0; d < 256; ++d)
                reduce[d] = d < head_dim ? b2f(qrow[d]) * b2f(krow[d]) : 0.0f;
            for (int stride = 128; stride > 0; stride >>= 1)
                for (int d = 0; d < stride; ++d) reduce[d] += reduce[d + stride];
            float score = reduce[0] * scale;
            float next_max = fmaxf(running_max, score);
            float alpha = expf(running_max - next_max);
            float pw = expf(score - next_max);
            running_sum = running_sum * alpha + pw;
            running_max = next_max;
            const uint16_t* vrow = value + ((size_t)pos * key_heads + kh) * head_dim;
            for (int d = 0; d < head_dim; ++d)
                out_acc[d] = out_acc[d] * alpha + b2f(vrow[d]) * pw;
        }
        uint16_t* orow = output + ((size_t)token * query_heads + qh) * head_dim;
        for (int d = 0; d < head_dim; ++d) orow[d] = f2b(out_acc[d] / running_sum);
    }
    return 0;
}

/* ---- matmul + fused softmax + matmul path ---------------------------------
 * src/modeling/diffusion_gemma/attention.cpp:706-821 (gqa_attention) with
 * src/modeling/diffusion_gemma/attention_kernels.hpp:234-293
 * (fused_masked_softmax): scores are stored in bf16 after the first matmul,
 * softmax runs in fp32 over the valid span [lo,hi) of each row and its
 * probabilities are stored in bf16 (zero outside the span), the second matmul
 * accumulates in fp32 and stores bf16.  There is no scale on this path.
 * Query tiling / band slicing of the reference only bounds scratch size and
 * does not change any value, so one full-width pass is taken here.
 * Deviation: the reference's work-group tree reductions (256 lanes strided
 * over the row) are replaced by a left-to-right fp32 pass. */
ORACLE_API int oracle_gqa_attention(const uint16_t* Q, int seq, int nq, int hd,
                                    const uint16_t* Kc, const uint16_t* Vc, int kv_len,
                                    int nkv, int past_offset, int sliding_window,
                                    int causal, uint16_t* out) {
    if (nkv <= 0 || nq % nkv != 0) return -1;
    int g = nq / nkv;
    int kv0 = past_offset - (kv_len - seq);
    int64_t total = (int64_t)seq * nq;
    int err = 0;
#pragma omp parallel
    {
        uint16_t* x = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(kv_len > 0 ? kv_len : 1));
        float* acc = (float*)malloc(sizeof(float) * (size_t)hd);
        if (!x || !acc) {
#pragma omp atomic write
            err = -3;
        } else {
#pragma omp for schedule(dynamic, 4)
            for (int64_t r = 0; r < total; ++r) {
                int t = (int)(r / nq), h = (int)(r % nq), kh = h / g;
                const uint16_t* qrow = Q + ((size_t)t * nq + h) * hd;
                int q_global = past_offset + t;
                int lo = 0, hi = kv_len;
                if (causal) {
                    int hh = q_global - kv0 + 1;
                    hi = hh < kv_len ? hh : kv_len;
                    if (sliding_window != INT_MAX) {
                        int l = q_global - kv0 - sliding_window + 1;
                        lo = l > 0 ? l : 0;
                    }
                }
                /* Scores only inside the visible band (the reference slices the
                 * same band per query tile, attention.cpp:721-769). */
                for (int j = lo; j < hi; ++j) {
                    const uint16_t* krow = Kc + ((size_t)j * nkv + kh) * hd;
                    float dot = 0.0f;
#pragma omp simd reduction(+ : dot)
                    for (int d = 0; d < hd; ++d) dot += b2f(qrow[d]) * b2f(krow[d]);
                    x[j] = f2b(dot);
                }
                float m = -3.4028235e38f;
                for (int c = lo; c < hi; ++c) m = fmaxf(m, b2f(x[c]));
                float z = 0.0f;
                for (int c = lo; c < hi; ++c) z += expf(b2f(x[c]) - m);
                float inv_z = 1.0f / z;
                for (int c = lo; c < hi; ++c) x[c] = f2b(expf(b2f(x[c]) - m) * inv_z);
                for (int d = 0; d < hd; ++d) acc[d] = 0.0f;
                for (int c = lo; c < hi; ++c) {
                    float p = b2f(x[c]);
                    if (p == 0.0f) continue;
                    const uint16_t* vrow = Vc + ((size_t)c * nkv + kh) * hd;
#pragma omp simd
                    for (int d = 0; d < hd; ++d) acc[d] += p * b2f(vrow[d]);
                }
                uint16_t* orow = out + ((size_t)t * nq + h) * hd;
                for (int d = 0; d < hd; ++d) orow[d] = f2b(acc[d]);
            }
        }
        free(x);
        free(acc);
    }
    return err;
}

/* ---- nine-step batched path : src/common/layers/attention_batched.hpp:71-136
 * bf16 scores -> f32 (score*scale + mask, :28-44) -> accurate softmax in f32
 * -> bf16 probabilities -> second matmul -> bf16.  The mask is the buffer of
 * oracle_fill_causal_mask unless skip_mask is set. */
ORACLE_API int oracle_batched_attention(const uint16_t* Q, int seq, int nq, int hd,
                                        const uint16_t* K, const uint16_t* V, int kv_len,
                                        int nkv, int past_offset, int sliding_window,
                                        float scale, int skip_mask, uint16_t* out) {
    if (nkv <= 0 || nq % nkv != 0) return -1;
    int g = nq / nkv;
    float* mask = NULL;
    if (!skip_mask) {
        mask = (float*)malloc(sizeof(float) * (size_t)seq * (size_t)kv_len);
        if (!mask) return -3;
        oracle_fill_causal_mask(mask, seq, kv_len, past_offset, sliding_window);
    }
    int64_t total = (int64_t)seq * nq;
    int err = 0;
#pragma omp parallel
    {
        float* s = (float*)malloc(sizeof(float) * (size_t)(kv_len > 0 ? kv_len : 1));
        float* acc = (float*)malloc(sizeof(float) * (size_t)hd);
        if (!s || !acc) {
#pragma omp atomic write
            err = -3;
        } else {
#pragma omp for schedule(dynamic, 4)
            for (int64_t r = 0; r < total; ++r) {
                int t = (int)(r / nq), h = (int)(r % nq), kh = h / g;
                const uint16_t* qrow = Q + ((size_t)t * nq + h) * hd;
                float m = -INFINITY;
                for (int j = 0; j < kv_len; ++j) {
                    const uint16_t* krow = K + ((size_t)j * nkv + kh) * hd;
                    float dot = 0.0f;
#pragma omp simd reduction(+ : dot)
                    for (int d = 0; d < hd; ++d) dot += b2f(qrow[d]) * b2f(krow[d]);
                    float v = b2f(f2b(dot)) * scale;
                    if (mask) v += mask[(size_t)t * kv_len + j];
                    s[j] = v;
                    m = fmaxf(m, v);
                }
                float z = 0.0f;
                for (int j = 0; j < kv_len; ++j) {
                    s[j] = expf(s[j] - m);
                    z += s[j];
                }
                for (int d = 0; d < hd; ++d) acc[d] = 0.0f;
                for (int j = 0; j < kv_len; ++j) {
                    float p = b2f(f2b(s[j] / z));
                    if (p == 0.0f) continue;
                    const uint16_t* vrow = V + ((size_t)j * nkv + kh) * hd;
#pragma omp simd
                    for (int d = 0; d < hd; ++d) acc[d] += p * b2f(vrow[d]);
                }
                uint16_t* orow = out + ((size_t)t * nq + h) * hd;
                for (int d = 0; d < hd; ++d) orow[d] = f2b(acc[d]);
            }
        }
        free(s);
        free(acc);
    }
    free(mask);
    return err;
}

/* ---- split-KV merge identity ----------------------------------------------
 * Not in the reference (it never splits the key range).  For partials
 * (o_c, lse_c) computed over disjoint key ranges,
 *   lse = log sum_c exp(lse_c),  out = sum_c exp(lse_c - lse) * o_c,
 * which equals the unsplit softmax.  o: (n_parts, rows, hd) f32, lse:
 * (n_parts, rows) f32; a part with lse = -inf contributes nothing. */
ORACLE_API void oracle_merge_partials(const float* o, const float* lse, int n_parts,
                                      int64_t rows, int hd, float* out, float* out_lse) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double m = -INFINITY;
        for (int c = 0; c < n_parts; ++c) {
            double l = lse[(size_t)c * rows + r];
            if (l > m) m = l;
        }
        double z = 0.0;
        for (int c = 0; c < n_parts; ++c) {
            double l = lse[(size_t)c * rows + r];
            if (l > -INFINITY) z += exp(l - m);
        }
        for (int d = 0; d < hd; ++d) {
            double acc = 0.0;
            if (z > 0.0) {
                for (int c = 0; c < n_parts; ++c) {
                    double l = lse[(size_t)c * rows + r];
                    if (l > -INFINITY)
                        acc += exp(l - m) / z * (double)o[((size_t)c * rows + r) * hd + d];
                }
            }
            out[(size_t)r * hd + d] = (float)acc;
        }
        if (out_lse) out_lse[r] = z > 0.0 ? (float)(m + log(z)) : -INFINITY;
    }
}
