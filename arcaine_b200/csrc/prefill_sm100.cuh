// GQA flash-attention prefill / canvas kernel for sm_100a.
//
// One CTA owns a tile of 128 query tokens of one query head and walks the key
// blocks (128 keys) that tile can see.  Q, K and V tiles are staged in shared
// memory by TMA (128-byte swizzle, one 64-element column chunk per copy);
// S = Q K^T and O += P V run on the tcgen05 tensor cores with both accumulators
// in tensor memory; P is written back to tensor memory as bf16 over the S
// columns and fed to the second MMA from there, so probabilities never touch
// shared or global memory.  Softmax is online, fp32, one query row per thread.
//
// Warp roles (192 threads): warps 0-3 softmax + correction + epilogue (their
// warp index selects the 32 TMEM lanes each may touch), warp 4 TMA producer and
// TMEM owner, warp 5 MMA issuer.
//
// Masking follows the reference's rules evaluated inline instead of through a
// (q_len, kv_len) f32 buffer: causal aligned bottom-right with an optional
// window of the W most recent keys, self included
// (src/common/kernels/attention_mask.hpp:12-38); no mask for the bidirectional
// canvas-over-prompt call (src/modeling/diffusion_gemma/attention.cpp:1093-1103);
// an explicit additive buffer is still accepted.  Key blocks wholly outside a
// tile's visible band are never loaded (the band idea of gqa_attention,
// src/modeling/diffusion_gemma/attention.cpp:721-769, per CTA).
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include "ptx.cuh"

namespace arc {

struct PrefillParams {
    uint16_t* out;
    const uint16_t* gate;
    const float* mask;
    float* out_lse;
    float* part_o;
    float* part_lse;
    uint32_t* fault;
    int batch, seq, kv_len, nq, nkv;
    long long o_stride_b, o_stride_t;
    float scale_log2;  // scale * log2(e)
    int mask_type, window;
    int num_splits;
#ifdef ARC_PREFILL_TRACE
    long long* trace;  // debug builds only: per-block timestamps of CTA 0
#endif
};

template <int HD>
struct PrefillCfg {
    static constexpr int BM = 128;  // query rows per CTA
    static constexpr int BN = 128;  // keys per block
    static constexpr int CH = HD / 64;
    static constexpr int CHUNK_BYTES = 128 * 128;  // 128 rows x 64 bf16
    static constexpr int TILE_BYTES = CH * CHUNK_BYTES;
    static constexpr int TMEM_COLS = (HD == 128) ? 256 : 512;
    static constexpr int COL_S = 0;    // 128 fp32 columns; P (bf16) aliases the first 64
    static constexpr int COL_O = 128;  // HD fp32 columns
    static constexpr int NUM_BARS = 9;
    static constexpr int XCH_BYTES = (2 * 2 * 128 + 2 * 128) * 4;  // row-max exchange (2 phases) + row-sum exchange
    static constexpr int SMEM_BYTES = 3 * TILE_BYTES + NUM_BARS * 8 + 16 + XCH_BYTES + 1024;
    static constexpr int THREADS = 384;  // 3 warpgroups: softmax A, softmax B, {TMA, MMA, 2 idle warps}
    static constexpr int MIN_CTAS = (HD == 128) ? 2 : 1;
    // Register re-split between warpgroups (hd128, two CTAs per SM: 80 registers per thread at launch).
    static constexpr bool RESPLIT = (HD == 128);
    static constexpr int REGS_SOFTMAX = 104;
    static constexpr int REGS_OTHER = 24;
};

// Per-row visibility for blocks that need element masking.
struct RowMask {
    int lo, hi;            // visible keys [lo, hi)
    int kv_len;
    const float* mask_row;  // optional additive mask row (natural-log domain)
};

__device__ __forceinline__ float max3f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Element masking mode of a key block: 0 = every key visible, 1 = per-row span
// [lo, hi), 2 = span plus an additive f32 mask row.
// Scaled (log2-domain) and masked score of one key.
template <int MODE>
__device__ __forceinline__ float masked_score(uint32_t raw, float sl, int key, const RowMask& rm) {
    float x = __uint_as_float(raw) * sl;
    if (MODE == 2) {
        if (rm.mask_row && key < rm.kv_len) x += rm.mask_row[key] * 1.4426950408889634f;
    }
    return (key >= rm.lo && key < rm.hi) ? x : -CUDART_INF_F;
}

// Maximum of one 32-column chunk, folded into four independent running maxima.
template <int MODE>
__device__ __forceinline__ void chunk_max(const uint32_t (&v)[32], float (&mx)[4], float sl, int key0,
                                          const RowMask& rm) {
#pragma unroll
    for (int e = 0; e < 32; e += 8) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float a, b;
            if (MODE != 0) {
                a = masked_score<MODE>(v[e + 2 * u], sl, key0 + e + 2 * u, rm);
                b = masked_score<MODE>(v[e + 2 * u + 1], sl, key0 + e + 2 * u + 1, rm);
            } else {
                a = __uint_as_float(v[e + 2 * u]);
                b = __uint_as_float(v[e + 2 * u + 1]);
            }
            mx[u] = max3f(mx[u], a, b);
        }
    }
}

// exp2 of one chunk against the running max, packed to bf16x2; four independent partial sums.
template <int MODE>
__device__ __forceinline__ void chunk_exp(const uint32_t (&v)[32], uint32_t (&pk)[16], float (&ls)[4], float sl,
                                          float m_eff, int key0, const RowMask& rm) {
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        float p0, p1;
        if (MODE != 0) {
            p0 = fast_exp2(masked_score<MODE>(v[e], sl, key0 + e, rm) - m_eff);
            p1 = fast_exp2(masked_score<MODE>(v[e + 1], sl, key0 + e + 1, rm) - m_eff);
        } else {
            p0 = fast_exp2(fmaf(__uint_as_float(v[e]), sl, -m_eff));
            p1 = fast_exp2(fmaf(__uint_as_float(v[e + 1]), sl, -m_eff));
        }
        ls[(e >> 1) & 3] += p0 + p1;
        pk[e >> 1] = pack_bf16x2(p0, p1);
    }
}

// How a 32-key chunk relates to the rows of this warp (warp-uniform, so the
// warp-collective TMEM instructions stay converged): 0 = every key visible to all
// 32 rows (no element test needed), 1 = mixed, 2 = no key visible to any row.
// With a causal diagonal crossing a 128 x 128 block, each warp meets at most one
// or two mixed chunks; the rest is either plain or skipped.
__device__ __forceinline__ int chunk_class(int kc, const RowMask& rm) {
    const bool all = rm.lo <= kc && kc + 32 <= rm.hi;
    const bool none = rm.hi <= kc || rm.lo >= kc + 32;
    if (__all_sync(0xffffffffu, all)) return 0;
    if (__all_sync(0xffffffffu, none)) return 2;
    return 1;
}

template <bool ADD_MASK>
__device__ __forceinline__ void chunk_max_any(const uint32_t (&v)[32], float (&mx_raw)[4], float (&mx_scaled)[4],
                                              float sl, int kc, const RowMask& rm) {
    const int cls = ADD_MASK ? 1 : chunk_class(kc, rm);
    if (cls == 0) chunk_max<0>(v, mx_raw, sl, kc, rm);
    else if (cls == 1) chunk_max<ADD_MASK ? 2 : 1>(v, mx_scaled, sl, kc, rm);
}

template <bool ADD_MASK>
__device__ __forceinline__ void chunk_exp_any(const uint32_t (&v)[32], uint32_t (&pk)[16], float (&ls)[4], float sl,
                                              float m_eff, int kc, const RowMask& rm) {
    const int cls = ADD_MASK ? 1 : chunk_class(kc, rm);
    if (cls == 0) {
        chunk_exp<0>(v, pk, ls, sl, m_eff, kc, rm);
    } else if (cls == 1) {
        chunk_exp<ADD_MASK ? 2 : 1>(v, pk, ls, sl, m_eff, kc, rm);
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = 0u;
    }
}


// Barrier between the two warps that share a set of 32 query rows (warp w and w + 4):
// hardware barrier 1 + w, 64 threads.  Every softmax warp executes exactly one pair_sync per
// key block and one after the loop, whatever happened to its waits, so neither can hang here.
__device__ __forceinline__ void pair_sync(int pair) {
    asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
}

template <int R>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R));
}
template <int R>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R));
}

template <int HD>
__global__ void __launch_bounds__(PrefillCfg<HD>::THREADS, PrefillCfg<HD>::MIN_CTAS)
    sdpa_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    using C = PrefillCfg<HD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = smem + C::TILE_BYTES;
    uint8_t* sV = smem + 2 * C::TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * C::TILE_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = bars + 2;
    uint64_t* v_full = bars + 3;
    uint64_t* v_empty = bars + 4;
    uint64_t* s_full = bars + 5;
    uint64_t* p_full = bars + 6;
    uint64_t* o_full = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NUM_BARS);
    uint32_t* abort_slot = tmem_slot + 1;
    float* xch_max = reinterpret_cast<float*>(tmem_slot + 4);  // [phase 2][half 2][row 128]
    float* xch_sum = xch_max + 2 * 2 * 128;                    // [half 2][row 128]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int qt = blockIdx.x;
    const int h = blockIdx.y;
    const int b = blockIdx.z / p.num_splits;
    const int split = blockIdx.z % p.num_splits;
    const int kvh = h / (p.nq / p.nkv);
    const int q0 = qt * C::BM;
    const int off = p.kv_len - p.seq;
    const bool causal = (p.mask_type == 3);
    const bool windowed = causal && p.window > 0 && p.window != 0x7fffffff;
    const int q_last = min(q0 + C::BM - 1, p.seq - 1);

    // Key blocks [blk_lo, blk_hi) this tile can see, then this split's share.
    int blk_lo = 0, blk_hi = (p.kv_len + C::BN - 1) / C::BN;
    if (causal) {
        int last_key = min(p.kv_len - 1, q_last + off);
        blk_hi = last_key >= 0 ? last_key / C::BN + 1 : 0;
        if (windowed) blk_lo = max(0, q0 + off - p.window + 1) / C::BN;
    }
    const int nblk = max(0, blk_hi - blk_lo);
    const int per = (nblk + p.num_splits - 1) / p.num_splits;
    const int my_lo = blk_lo + split * per;
    const int my_hi = min(blk_hi, my_lo + per);
    const int n_my = max(0, my_hi - my_lo);

    const long long rows_total = (long long)p.batch * p.seq * p.nq;

    if (threadIdx.x == 0) *abort_slot = (*reinterpret_cast<volatile uint32_t*>(p.fault) != 0u) ? 1u : 0u;
    __syncthreads();
    if (*abort_slot) return;

    if (n_my == 0) {
        // Nothing visible: zero output (or an empty partial) for this tile.
        if (warp < 4) {
            const int t = q0 + threadIdx.x;
            if (t < p.seq) {
                const long long row = ((long long)b * p.seq + t) * p.nq + h;
                if (p.num_splits > 1) {
                    float4* dst = reinterpret_cast<float4*>(p.part_o + ((long long)split * rows_total + row) * HD);
                    for (int i = 0; i < HD / 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    p.part_lse[(long long)split * rows_total + row] = -CUDART_INF_F;
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(p.out + b * p.o_stride_b + t * p.o_stride_t + (long long)h * HD);
                    for (int i = 0; i < HD / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                    if (p.out_lse) p.out_lse[row] = -CUDART_INF_F;
                }
            }
        }
        return;
    }

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(k_full, 1);
        mbar_init(k_empty, 1);
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(p_full, 256);
        mbar_init(o_full, 1);
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp >= 8) {
        if (C::RESPLIT) setmaxnreg_dec<C::REGS_OTHER>();
        if (warp == 8 && lane == 0) {
            // -------------------------------------------------------------- TMA producer
            prefetch_tensormap(&tm_q);
            prefetch_tensormap(&tm_k);
            prefetch_tensormap(&tm_v);
            mbar_arrive_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < C::CH; ++c) tma_load_4d(sQ + c * C::CHUNK_BYTES, &tm_q, q_full, c * 64, h, q0, b);
            for (int i = 0; i < n_my; ++i) {
                const int key0 = (my_lo + i) * C::BN;
                if (i > 0 && !mbar_wait(k_empty, (i - 1) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_EMPTY, 0x100u + i);
                    break;
                }
                mbar_arrive_expect_tx(k_full, C::TILE_BYTES);
#pragma unroll
                for (int c = 0; c < C::CH; ++c)
                    tma_load_4d(sK + c * C::CHUNK_BYTES, &tm_k, k_full, c * 64, kvh, key0, b);
                if (i > 0 && !mbar_wait(v_empty, (i - 1) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_EMPTY, 0x200u + i);
                    break;
                }
                mbar_arrive_expect_tx(v_full, C::TILE_BYTES);
#pragma unroll
                for (int c = 0; c < C::CH; ++c)
                    tma_load_4d(sV + c * C::CHUNK_BYTES, &tm_v, v_full, c * 64, kvh, key0, b);
            }
        } else if (warp == 9 && lane == 0) {
            // -------------------------------------------------------------- MMA issuer
            constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, false);
            constexpr uint32_t IDESC_PV = make_idesc_bf16(128, HD, true);
            const uint32_t tS = tmem_base + C::COL_S;
            const uint32_t tO = tmem_base + C::COL_O;
            const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) report_fault(p.fault, FAULT_WAIT_Q, 0);
            for (int i = 0; ok && i < n_my; ++i) {
                if (!mbar_wait(k_full, i & 1)) {
                    report_fault(p.fault, FAULT_WAIT_K, i);
                    break;
                }
                tc_fence_after_sync();
                // S = Q K^T : both operands K-major, 8-row groups 1024 bytes apart.
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t o = (kk >> 2) * C::CHUNK_BYTES + (kk & 3) * 32;
                    umma_ss(tS, make_smem_desc_sw128(aQ + o, 16, 1024), make_smem_desc_sw128(aK + o, 16, 1024),
                            IDESC_QK, kk > 0 ? 1u : 0u);
                }
                umma_commit(k_empty);
                umma_commit(s_full);
#ifdef ARC_PREFILL_TRACE
                if (p.trace && blockIdx.x == 20 && blockIdx.y == 0 && blockIdx.z == 0 && i < 16) p.trace[i * 8 + 7] = clock64();
#endif
                if (!mbar_wait(p_full, i & 1)) {
                    report_fault(p.fault, FAULT_WAIT_P, i);
                    break;
                }
#ifdef ARC_PREFILL_TRACE
                if (p.trace && blockIdx.x == 20 && blockIdx.y == 0 && blockIdx.z == 0 && i < 16) p.trace[i * 8 + 5] = clock64();
#endif
                if (!mbar_wait(v_full, i & 1)) {
                    report_fault(p.fault, FAULT_WAIT_V, i);
                    break;
                }
                tc_fence_after_sync();
                // O += P V : P from tensor memory, 8 columns per 16 keys; the two key
                // halves of a block keep their P at the start of their own S columns
                // (keys 0-63 at columns 0-31, keys 64-127 at columns 64-95).  V is
                // MN-major: 64-element head-dim chunks 16 KB apart (leading offset),
                // 8-key groups 1024 bytes apart (stride offset).
#pragma unroll
                for (int ks = 0; ks < C::BN / 16; ++ks) {
                    const uint32_t pcol = (ks < 4) ? ks * 8 : 64 + (ks - 4) * 8;
                    umma_ts(tO, tS + pcol, make_smem_desc_sw128(aV + ks * 2048, C::CHUNK_BYTES, 1024), IDESC_PV,
                            (i > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(v_empty);
#ifdef ARC_PREFILL_TRACE
                if (p.trace && blockIdx.x == 20 && blockIdx.y == 0 && blockIdx.z == 0 && i < 16) p.trace[i * 8 + 6] = clock64();
#endif
            }
            umma_commit(o_full);
        }
    } else {
        // ------------------------------------------------------------------ softmax / epilogue
        // Two threads per query row: warps 0-3 own keys 0-63 of every block (S columns
        // 0-63), warps 4-7 keys 64-127; both halves of a row sit in the same TMEM lane.
        if (C::RESPLIT) setmaxnreg_inc<C::REGS_SOFTMAX>();
        const int half = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const int t = q0 + r;
        constexpr int OC = HD / 2;  // output columns per thread
        const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + lane_sel + C::COL_S + half * 64;
        const uint32_t tO = tmem_base + lane_sel + C::COL_O + half * OC;
        const float sl = p.scale_log2;

        int row_lo = 0, row_hi = p.kv_len;  // visible keys [row_lo, row_hi)
        if (causal) {
            const int diag = t + off;
            row_hi = min(max(diag + 1, 0), p.kv_len);
            if (windowed) row_lo = max(0, diag - p.window + 1);
            if (row_lo > row_hi) row_lo = row_hi;
        }
        const bool has_mask = (p.mask_type == 1) && p.mask != nullptr;
        const float* mask_row = has_mask && t < p.seq ? p.mask + (long long)t * p.kv_len : nullptr;
        const RowMask rm{row_lo, row_hi, p.kv_len, mask_row};

        float m = -CUDART_INF_F;  // running max, log2 domain, possibly stale by <= 8
        float l = 0.f;            // this thread's share of the row sum
        bool ok = true;
        uint32_t va[32], vb[32];  // this thread's 64 scores of the current block

        for (int i = 0; i < n_my; ++i) {
            const int kc = (my_lo + i) * C::BN + half * 64;
#ifdef ARC_PREFILL_TRACE
            const bool tr = p.trace && blockIdx.x == 20 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0 && i < 16;
            if (tr) p.trace[i * 8 + 0] = clock64();
#endif
            if (ok && !mbar_wait_warp(s_full, i & 1)) {
                report_fault(p.fault, FAULT_WAIT_S, i);
                ok = false;
            }
            if (!ok) {
                // Gave up on a wait: keep meeting the partner warp at the pair barrier so it can
                // never be left waiting there, but touch nothing else.
                pair_sync(warp & 3);
                continue;
            }
            tc_fence_after_sync();
#ifdef ARC_PREFILL_TRACE
            if (tr) p.trace[i * 8 + 1] = clock64();
#endif
            tmem_ld32(tS, va);
            tmem_ld32(tS + 32, vb);
            tmem_wait_ld();

            // Maximum of this thread's 64 scores, then of the whole row via shared memory.
            float mr[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            float ms[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            if (has_mask) {
                chunk_max_any<true>(va, mr, ms, sl, kc, rm);
                chunk_max_any<true>(vb, mr, ms, sl, kc + 32, rm);
            } else {
                chunk_max_any<false>(va, mr, ms, sl, kc, rm);
                chunk_max_any<false>(vb, mr, ms, sl, kc + 32, rm);
            }
            const float m_half = fmaxf(fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * sl,
                                       fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3])));
            xch_max[((i & 1) * 2 + half) * 128 + r] = m_half;
            pair_sync(warp & 3);
            const float m_blk = fmaxf(m_half, xch_max[((i & 1) * 2 + (half ^ 1)) * 128 + r]);
#ifdef ARC_PREFILL_TRACE
            if (tr) p.trace[i * 8 + 2] = clock64();
#endif
            const float m_new = fmaxf(m, m_blk);
            if (i == 0) {
                m = m_new;
            } else {
                const bool need = m_new > m + 8.0f;
                if (__any_sync(0xffffffffu, need)) {
                    // Rare: the row maximum grew by more than 2^8; rescale this thread's half of
                    // O in tensor memory (its partner takes the same decision from the same values),
                    // then fetch the scores again.
                    const float alpha = (m_new == -CUDART_INF_F) ? 1.0f : fast_exp2(m - m_new);
#pragma unroll 1
                    for (int c = 0; c < OC / 32; ++c) {
                        tmem_ld32(tO + c * 32, va);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) va[e] = __float_as_uint(__uint_as_float(va[e]) * alpha);
                        tmem_st32(tO + c * 32, va);
                    }
                    l *= alpha;
                    m = m_new;
                    tmem_ld32(tS, va);
                    tmem_wait_ld();
                }
            }
            const float m_eff = (m == -CUDART_INF_F) ? 0.f : m;

            // Probabilities as bf16 over the first 32 of this thread's S columns (all 64 scores
            // are already in registers), row-sum share in fp32.
            float ls4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[16];
            if (has_mask) {
                chunk_exp_any<true>(va, pk, ls4, sl, m_eff, kc, rm);
                tmem_st16(tS, pk);
                chunk_exp_any<true>(vb, pk, ls4, sl, m_eff, kc + 32, rm);
                tmem_st16(tS + 16, pk);
            } else {
                chunk_exp_any<false>(va, pk, ls4, sl, m_eff, kc, rm);
                tmem_st16(tS, pk);
                chunk_exp_any<false>(vb, pk, ls4, sl, m_eff, kc + 32, rm);
                tmem_st16(tS + 16, pk);
            }
            l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
#ifdef ARC_PREFILL_TRACE
            if (tr) p.trace[i * 8 + 3] = clock64();
#endif
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(p_full);
#ifdef ARC_PREFILL_TRACE
            if (tr) p.trace[i * 8 + 4] = clock64();
#endif
        }

        // Row sum = both halves' shares.
        xch_sum[half * 128 + r] = l;
        pair_sync(warp & 3);
        l += xch_sum[(half ^ 1) * 128 + r];
        if (ok && !mbar_wait_warp(o_full, 0)) {
            report_fault(p.fault, FAULT_WAIT_O, 0);
            ok = false;
        }
        tc_fence_after_sync();
        if (ok) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const float lse = l > 0.f ? (m + fast_log2(l)) * 0.6931471805599453f : -CUDART_INF_F;
            const long long row = ((long long)b * p.seq + t) * p.nq + h;
            const bool store = t < p.seq;
            if (p.num_splits > 1) {
                float* dst = p.part_o + ((long long)split * rows_total + row) * HD + half * OC;
#pragma unroll 1
                for (int c = 0; c < OC / 32; ++c) {
                    tmem_ld32(tO + c * 32, va);
                    tmem_wait_ld();
                    if (store) {
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            *reinterpret_cast<float4*>(dst + c * 32 + e) =
                                make_float4(__uint_as_float(va[e]) * inv, __uint_as_float(va[e + 1]) * inv,
                                            __uint_as_float(va[e + 2]) * inv, __uint_as_float(va[e + 3]) * inv);
                    }
                }
                if (store && half == 0) p.part_lse[(long long)split * rows_total + row] = lse;
            } else {
                const long long eoff = b * p.o_stride_b + t * p.o_stride_t + (long long)h * HD + half * OC;
                uint16_t* dst = p.out + eoff;
                const uint16_t* g = p.gate ? p.gate + eoff : nullptr;
#pragma unroll 1
                for (int c = 0; c < OC / 32; ++c) {
                    tmem_ld32(tO + c * 32, va);
                    tmem_wait_ld();
                    if (store) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            float o[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) o[u] = __uint_as_float(va[e + u]) * inv;
                            if (g) {
                                const uint4 gv = *reinterpret_cast<const uint4*>(g + c * 32 + e);
                                const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                                for (int u = 0; u < 8; ++u) {
                                    const float gf = bf16_bits_to_f32(static_cast<uint16_t>(gw[u >> 1] >> ((u & 1) * 16)));
                                    const float sig = 1.0f / (1.0f + __expf(-gf));
                                    o[u] = bf16_round(o[u]) * sig;
                                }
                            }
                            uint4 ov;
                            ov.x = pack_bf16x2(o[0], o[1]);
                            ov.y = pack_bf16x2(o[2], o[3]);
                            ov.z = pack_bf16x2(o[4], o[5]);
                            ov.w = pack_bf16x2(o[6], o[7]);
                            *reinterpret_cast<uint4*>(dst + c * 32 + e) = ov;
                        }
                    }
                }
                if (store && half == 0 && p.out_lse) p.out_lse[row] = lse;
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace arc
