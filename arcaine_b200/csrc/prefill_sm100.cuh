// GQA flash-attention prefill / canvas kernel for sm_100a, one query tile at a time per CTA: the
// kernel for head dim 256, additive masks, key-range splits and small problems (head dim 128
// with enough tiles runs two tiles per CTA, prefill_pair_sm100.cuh).
//
// One CTA owns a tile of 128 query tokens of one query head and walks the key
// blocks (128 keys) that tile can see.  Q, K and V tiles are staged in shared
// memory by TMA (128-byte swizzle, one 64-element column chunk per copy);
// S = Q K^T and O += P V run on the tcgen05 tensor cores with both accumulators
// in tensor memory; P is written back to tensor memory as bf16 over the S
// columns and fed to the second MMA from there, so probabilities never touch
// shared or global memory.  Softmax is online, fp32.
//
// Warp roles: eight softmax / correction / epilogue warps, two threads per query row
// (warp index mod 4 selects the 32 TMEM lanes, warp index / 4 the 64-key half of each
// block), then one TMA producer warp (also the TMEM owner) and one MMA issuing warp.
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
#include <type_traits>
#include <cuda.h>
#include <math_constants.h>

#include "ptx.cuh"

namespace arc {

struct PrefillParams {
    uint16_t* out;
    const unsigned long long* out_copies;  // n_copies more output buffers (other GPUs' over NVLink), same offsets
    int n_copies;
    const uint16_t* gate;
    const float* mask;
    float* out_lse;
    float* part_o;
    float* part_lse;
    const int* vis_hi;  // optional [seq]: first key row t can no longer see (causal rule extended by vision blocks)
    uint32_t* fault;
    int batch, seq, kv_len, nq, nkv;
    long long o_stride_b, o_stride_t;
    float scale_log2;  // scale * log2(e)
    int mask_type, window;
    int num_splits;
    int q_tiles;      // ceil(seq / 128)
    int total_tiles;  // q_tiles * cur_heads * batch * num_splits, dealt round-robin to the persistent CTAs
    int cur_heads;    // head units the tile list walks: nq, or nq / 2 when a CTA takes two query heads at a time
    int head_pair;    // prefill_pair_sm100.cuh: 1 = the CTA's two tiles are the same tokens of two heads of one KV group
    int group;        // nq / nkv
    int group_shift;  // log2(group) if it is a power of two, else -1
    // >= 0 (one-tile kernel): the launch covers the tail of a two-tile launch's unit list — tile w is head (w & 1)
    // of the head pair with unit index tail_base + (w >> 1), one tile per CTA; -1: the plain tile list
    int tail_base;
};

// One CTA per SM, persistent: it takes tiles (128 query tokens of one query head) round-robin
// and keeps its pipelines running across tile boundaries — the next tile's Q, K and V stream in
// and its first score blocks are computed while the softmax warps still write the previous
// tile's output.  The score accumulator is
// multi-buffered in tensor memory (S0, S1[, S2], then O), so S = Q K^T runs one or two key
// blocks ahead of the softmax; eight softmax warps (two threads per query row, 64 keys
// each).  With three score buffers (head dim 128) they look at the next block's maximum
// before they exponentiate the current one, which hides the exchange of row maxima; with
// two (head dim 256) every block is taken on its own, because the next block's scores
// cannot be computed before this block's probabilities have been consumed.
// Eight rather than sixteen softmax warps on purpose: the
// single MMA-issuing thread shares an instruction scheduler with them, and with four busy
// warps per scheduler it could not issue MMAs fast enough to keep the tensor pipe fed.
template <int HD>
struct PrefillCfg {
    static constexpr int BM = 128;  // query rows per tile
    static constexpr int BN = 128;  // keys per block
    static constexpr int CH = HD / 64;
    static constexpr int CHUNK_BYTES = 128 * 128;  // 128 rows x 64 bf16
    static constexpr int TILE_BYTES = CH * CHUNK_BYTES;
    static constexpr int K_STAGES = (HD == 128) ? 3 : 1;
    static constexpr int V_STAGES = (HD == 128) ? 2 : 1;
    static constexpr int TMEM_COLS = 512;
    static constexpr int NSB = (HD == 128) ? 3 : 2;  // score buffers: S = Q K^T runs NSB-1 blocks ahead of the softmax
    static constexpr int COL_S = 0;                  // NSB buffers of 128 fp32 columns; P (bf16) is written over them
    static constexpr int COL_O = NSB * 128;          // HD fp32 columns
    static constexpr int NUM_BARS = 2 + 2 * K_STAGES + 2 * V_STAGES + 2 * NSB + 1 + 2 + 2;  // the last two: cluster merge
    static constexpr int XCH_FLOATS = 2 * 2 * 128 + 2 * 128 + 2 * 128;  // row-max exchange (2 phases), row-sum exchange, (max, sum) per row for the cluster merge
    static constexpr int SMEM_BYTES = (1 + K_STAGES + V_STAGES) * TILE_BYTES + NUM_BARS * 8 + 16 + XCH_FLOATS * 4 + 1024;
    static constexpr int SOFTMAX_WARPS = 8;
    static constexpr int THREADS = 32 * (SOFTMAX_WARPS + 2);
    static constexpr int MAX_REGS = 168;  // ten warps put three on some scheduler: 3 x 32 x 168 fits its 16384 registers, 176 does not
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

// 32 bytes (16 bf16) to q: one 256-bit store where q is 32-byte aligned (a whole DRAM sector), else two
// 128-bit stores.
__device__ __forceinline__ void store_bf16x16(uint16_t* q, const uint32_t (&w)[8]) {
    if ((reinterpret_cast<uintptr_t>(q) & 31u) == 0) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(q), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                     "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                     : "memory");
    } else {
        *reinterpret_cast<uint4*>(q) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(q + 8) = make_uint4(w[4], w[5], w[6], w[7]);
    }
}

// The same 32 bytes at element offset `off` of every copy of the output (plain stores; a copy in another
// GPU's memory travels over NVLink while the kernel computes on).
__device__ __forceinline__ void store_copies_bf16x16(const unsigned long long* copies, int n, long long off,
                                                     const uint32_t (&w)[8]) {
    for (int c = 0; c < n; ++c) store_bf16x16(reinterpret_cast<uint16_t*>(copies[c]) + off, w);
}

// bf16(attention) * sigmoid(gate), the rounding order of mul_sigmoid_inplace after a bf16 attention
// output (src/modeling/qwen3_5_moe/kernels.hpp:80-88).
__device__ __forceinline__ float sigmoid_gate_bits(float attn, uint16_t gate_bits) {
    const float g = bf16_bits_to_f32(gate_bits);
    return bf16_round(attn) * (1.0f / (1.0f + __expf(-g)));
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
    if constexpr (MODE == 0) {
        // Every key visible.  Plain fp32 instructions on purpose: measured on B200, a warp issues an
        // fma.f32x2 / add.f32x2 only every ~8 clocks (the scalar forms every clock), about as often as
        // an ex2.approx; both the packed forms and a polynomial 2^x on the FMA pipe for a share of
        // the scores made the kernel slower.
        const float nm = -m_eff;
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(v[e]), sl, nm));
            const float p1 = fast_exp2(fmaf(__uint_as_float(v[e + 1]), sl, nm));
            ls[e & 3] += p0;
            ls[(e + 1) & 3] += p1;
            pk[e >> 1] = pack_bf16x2(p0, p1);
        }
    } else if constexpr (MODE == 1) {
        // Per-row span: one select per score (exp2(-inf) = 0).
        const float nm = -m_eff;
        const int lo_rel = rm.lo - key0, hi_rel = rm.hi - key0;  // visible: lo_rel <= e < hi_rel
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
            const float x0 = fmaf(__uint_as_float(v[e]), sl, nm), x1 = fmaf(__uint_as_float(v[e + 1]), sl, nm);
            const float p0 = fast_exp2((e >= lo_rel && e < hi_rel) ? x0 : -CUDART_INF_F);
            const float p1 = fast_exp2((e + 1 >= lo_rel && e + 1 < hi_rel) ? x1 : -CUDART_INF_F);
            ls[e & 3] += p0;
            ls[(e + 1) & 3] += p1;
            pk[e >> 1] = pack_bf16x2(p0, p1);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
            const float p0 = fast_exp2(masked_score<MODE>(v[e], sl, key0 + e, rm) - m_eff);
            const float p1 = fast_exp2(masked_score<MODE>(v[e + 1], sl, key0 + e + 1, rm) - m_eff);
            ls[(e >> 1) & 3] += p0 + p1;
            pk[e >> 1] = pack_bf16x2(p0, p1);
        }
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



// Barrier between the two warps that share a set of 32 query rows (warps q and q + 4):
// hardware barrier 1 + q, 64 threads.  Every softmax warp executes the same number of
// pair_syncs per tile, whatever happened to its waits, so neither warp of a pair can be left
// waiting here.
__device__ __forceinline__ void pair_sync(int quarter) {
    asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory");
}

// All eight softmax warps (named barrier 5; barriers 1-4 belong to pair_sync).
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 5, 256;" ::: "memory"); }

// One unit of work of the persistent kernel.
struct TileWork {
    int q0, h, b, split, kvh;
    int my_lo, n_my;  // key blocks [my_lo, my_lo + n_my) of this tile and split
};

// Position of a persistent CTA in the launch's tile list: tile w = ((z * cur_heads) + h) * q_tiles + qt,
// token tiles fastest (neighbouring CTAs share K/V blocks in L2), then query heads, then
// z = batch * num_splits + split.  The cursor moves by gridDim.x tiles per step with carries
// instead of dividing again.
struct TileCursor {
    int w, qt, h, z;
    int dqt, dh, dz, step;
    __device__ __forceinline__ void init(const PrefillParams& p) { init(p, blockIdx.x, gridDim.x); }
    // first tile and stride given explicitly (a cluster of CTAs walks the list together)
    __device__ __forceinline__ void init(const PrefillParams& p, int first, int step_) {
        w = first;
        step = step_;
        if (p.tail_base >= 0) {  // (the grid holds one CTA per tile: the strides below are never used)
            const int idx = p.tail_base + (w >> 1);
            qt = idx % p.q_tiles;
            const int prest = idx / p.q_tiles, pairs = p.cur_heads >> 1;
            h = (prest % pairs) * 2 + (w & 1);
            z = prest / pairs;
            dqt = dh = dz = 0;
            return;
        }
        qt = w % p.q_tiles;
        const int rest = w / p.q_tiles;
        h = rest % p.cur_heads;
        z = rest / p.cur_heads;
        dqt = step % p.q_tiles;
        const int srest = step / p.q_tiles;
        dh = srest % p.cur_heads;
        dz = srest / p.cur_heads;
    }
    __device__ __forceinline__ void advance(const PrefillParams& p) {
        w += step;
        qt += dqt;
        int carry = qt >= p.q_tiles ? 1 : 0;
        qt -= carry * p.q_tiles;
        h += dh + carry;
        carry = h >= p.cur_heads ? 1 : 0;
        h -= carry * p.cur_heads;
        z += dz + carry;
    }
};

// nsplit > 0: the key range is split over the CTAs of a cluster (split = the CTA's rank) and the
// tile list holds whole tiles; else the split is part of the tile index (z = batch * num_splits + split).
template <int HD>
__device__ __forceinline__ TileWork decode_tile(const PrefillParams& p, const TileCursor& cur, int nsplit = 0, int split = 0) {
    using C = PrefillCfg<HD>;
    TileWork t;
    t.h = cur.h;
    if (nsplit > 0) {
        t.b = cur.z;
        t.split = split;
    } else if (p.num_splits == 1) {
        t.b = cur.z;
        t.split = 0;
        nsplit = 1;
    } else {
        t.b = cur.z / p.num_splits;
        t.split = cur.z % p.num_splits;
        nsplit = p.num_splits;
    }
    t.kvh = p.group_shift >= 0 ? (t.h >> p.group_shift) : t.h / p.group;
    t.q0 = cur.qt * C::BM;
    const int off = p.kv_len - p.seq;
    const bool causal = (p.mask_type == 3);
    const bool windowed = causal && p.window > 0 && p.window != 0x7fffffff;
    const int q_last = min(t.q0 + C::BM - 1, p.seq - 1);
    int blk_lo = 0, blk_hi = (p.kv_len + C::BN - 1) / C::BN;
    if (causal) {
        // the span ends are monotone in the row, so the tile's last row decides
        const int last_key = p.vis_hi ? p.vis_hi[q_last] - 1 : min(p.kv_len - 1, q_last + off);
        blk_hi = last_key >= 0 ? last_key / C::BN + 1 : 0;
        if (windowed) blk_lo = max(0, t.q0 + off - p.window + 1) / C::BN;
    }
    const int nblk = max(0, blk_hi - blk_lo);
    const int per = (nblk + nsplit - 1) / nsplit;
    t.my_lo = blk_lo + t.split * per;
    t.n_my = max(0, min(blk_hi, t.my_lo + per) - t.my_lo);
    return t;
}

// ADD_MASK and GATE select code that most calls do not need (an additive mask row per query, the
// sigmoid-gated epilogue); the common instance carries neither and stays small.
// CLUSTER: the kernel is launched in thread-block clusters; the CTAs of a cluster share a tile and
// split its key range, then fold their accumulators through distributed shared memory — each CTA
// writes its unnormalised O and (max, sum) per row into its own shared memory (the K / V buffers are
// free by then), and merges a share of the rows reading all of them.  One launch, no partial records
// in global memory, no merge kernel.
template <int HD, bool ADD_MASK, bool GATE, bool CLUSTER = false>
__global__ void __maxnreg__(PrefillCfg<HD>::MAX_REGS)
    sdpa_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    using C = PrefillCfg<HD>;
    constexpr int KS = C::K_STAGES;
    constexpr int VS = C::V_STAGES;
    constexpr int NSB = C::NSB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = smem + C::TILE_BYTES;       // [KS] stages
    uint8_t* sV = sK + KS * C::TILE_BYTES;    // [VS] stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + VS * C::TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* q_empty = bars + 1;       // the tile's last S = Q K^T has completed: Q may be replaced
    uint64_t* k_full = bars + 2;
    uint64_t* k_empty = k_full + KS;
    uint64_t* v_full = k_empty + KS;
    uint64_t* v_empty = v_full + VS;
    uint64_t* s_full = v_empty + VS;    // [NSB] score buffers
    uint64_t* p_full = s_full + NSB;    // [NSB]
    uint64_t* pv_done = p_full + NSB;   // one phase per key block: O += P V of that block has completed
    uint64_t* o_full = pv_done + 1;     // one phase per tile: the tile's last O += P V has completed
    uint64_t* o_empty = o_full + 1;     // one phase per tile: the softmax warps have read O out
    uint64_t* part_ready = o_empty + 1;  // cluster merge, one phase per tile: every CTA's share of the tile is in its shared memory
    uint64_t* read_done = part_ready + 1; // cluster merge, one phase per tile: every CTA has finished reading this CTA's share
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NUM_BARS);
    uint32_t* abort_slot = tmem_slot + 1;
    float* xch_max = reinterpret_cast<float*>(tmem_slot + 4);  // [phase 2][key half 2][row 128]
    float* xch_sum = xch_max + 2 * 2 * 128;                    // [key half 2][row 128]
    float2* cl_stat = reinterpret_cast<float2*>(xch_sum + 2 * 128);  // [row 128] (max, sum) of this CTA's key range
    const int csize = CLUSTER ? (int)cluster_nctarank() : 1;
    const int crank = CLUSTER ? (int)cluster_ctarank() : 0;
    const int cfirst = CLUSTER ? (int)(blockIdx.x / csize) : (int)blockIdx.x;  // this CTA's (cluster's) first tile
    const int cstep = CLUSTER ? (int)(gridDim.x / csize) : (int)gridDim.x;
    auto tile_of = [&](const TileCursor& c) { return CLUSTER ? decode_tile<HD>(p, c, csize, crank) : decode_tile<HD>(p, c); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long rows_total = (long long)p.batch * p.seq * p.nq;
    const bool causal = (p.mask_type == 3);
    const bool windowed = causal && p.window > 0 && p.window != 0x7fffffff;
    const int off = p.kv_len - p.seq;

    grid_launch_dependents();  // with key-range splits the merge kernel follows: it may be scheduled already
    constexpr int PRODUCER_WARP = C::SOFTMAX_WARPS;
    constexpr int MMA_WARP = C::SOFTMAX_WARPS + 1;
    if (threadIdx.x == 0) {
        const uint32_t fault_word = *reinterpret_cast<volatile uint32_t*>(p.fault);
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < KS; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
        }
        for (int s = 0; s < VS; ++s) {
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < NSB; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 32 * C::SOFTMAX_WARPS);
        }
        mbar_init(pv_done, 1);
        mbar_init(o_full, 1);
        mbar_init(o_empty, 32 * C::SOFTMAX_WARPS);
        mbar_init(part_ready, csize);  // one arrival per CTA of the cluster
        mbar_init(read_done, csize);
        fence_mbar_init();
        *abort_slot = fault_word != 0u ? 1u : 0u;
    }
    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            prefetch_tensormap(&tm_q);
            prefetch_tensormap(&tm_k);
            prefetch_tensormap(&tm_v);
        }
        __syncwarp();
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if constexpr (CLUSTER) cluster_sync_all();  // every CTA's barriers exist before anyone arrives on them
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    // A call that finds a status word set does no work: every role walks an empty tile list and meets
    // the others at the end (in a cluster nobody may leave early anyway).
    const int total_tiles = *abort_slot ? 0 : p.total_tiles;

    if (warp == PRODUCER_WARP) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int gk = 0, gv = 0, tc = 0;  // K blocks, V blocks and non-empty tiles loaded so far
            int tn = 0;                  // tiles seen (cluster merge: one phase of read_done each)
            bool ok = true;
            TileCursor cur;
            for (cur.init(p, cfirst, cstep); ok && cur.w < total_tiles; cur.advance(p), ++tn) {
                const TileWork tw = tile_of(cur);
                if (tw.n_my == 0) continue;
                if constexpr (CLUSTER) {
                    // the K / V buffers held this CTA's share of the previous tile: wait until the whole
                    // cluster has read it
                    if (tn > 0 && !mbar_wait_cluster(read_done, (tn - 1) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_EMPTY, 0x400u);
                        break;
                    }
                }
                if (tc > 0 && !mbar_wait(q_empty, (tc - 1) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_EMPTY, 0x300u);
                    break;
                }
                mbar_arrive_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
                for (int c = 0; c < C::CH; ++c) tma_load_4d(sQ + c * C::CHUNK_BYTES, &tm_q, q_full, c * 64, tw.h, tw.q0, tw.b);
                int uk = 0, uv = 0;
                // K runs up to K_STAGES blocks ahead of the MMAs, V up to V_STAGES; the two rings
                // are filled in the order the MMAs will need them.
                while (uk < tw.n_my || uv < tw.n_my) {
                    if (uk < tw.n_my && (uk <= uv + 1 || uv >= tw.n_my)) {
                        const int st = gk % KS;
                        if (gk >= KS && !mbar_wait(&k_empty[st], ((gk / KS) - 1) & 1)) {
                            report_fault(p.fault, FAULT_WAIT_EMPTY, 0x100u);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(&k_full[st], C::TILE_BYTES);
#pragma unroll
                        for (int c = 0; c < C::CH; ++c)
                            tma_load_4d(sK + st * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_k, &k_full[st], c * 64, tw.kvh,
                                        (tw.my_lo + uk) * C::BN, tw.b);
                        ++uk;
                        ++gk;
                    } else {
                        const int st = gv % VS;
                        if (gv >= VS && !mbar_wait(&v_empty[st], ((gv / VS) - 1) & 1)) {
                            report_fault(p.fault, FAULT_WAIT_EMPTY, 0x200u);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(&v_full[st], C::TILE_BYTES);
#pragma unroll
                        for (int c = 0; c < C::CH; ++c)
                            tma_load_4d(sV + st * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_v, &v_full[st], c * 64, tw.kvh,
                                        (tw.my_lo + uv) * C::BN, tw.b);
                        ++uv;
                        ++gv;
                    }
                }
                ++tc;
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        // Per tile: the first NSB-1 score blocks; then for every block u:  S(u+NSB-1) into the
        // buffer P(u-1) just left (runs while the softmax warps work on S(u)), then
        // O += P(u) V(u) once P(u) is in tensor memory.  Counters run across tiles, so buffers,
        // stages and barrier phases simply keep rotating.
        if (lane == 0) {
            constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, false);
            constexpr uint32_t IDESC_PV = make_idesc_bf16(128, HD, true);
            const uint32_t tO = tmem_base + C::COL_O;
            const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
            // Descriptors are built once; per MMA only the start-address field (bytes >> 4, low
            // word) moves, so the issuing thread needs a handful of instructions per MMA.
            const uint64_t dQ = make_smem_desc_sw128(aQ, 16, 1024);
            const uint64_t dK = make_smem_desc_sw128(aK, 16, 1024);
            const uint64_t dV = make_smem_desc_sw128(aV, C::CHUNK_BYTES, 1024);
            int gs = 0, gp = 0, tc = 0;  // score blocks issued, P V blocks issued, non-empty tiles started
            auto issue_qk = [&]() -> bool {
                if (!mbar_wait(&k_full[gs % KS], (gs / KS) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_K, gs);
                    return false;
                }
                tc_fence_after_sync();
                const uint32_t tS = tmem_base + C::COL_S + (gs % NSB) * 128;
                const uint64_t dKu = dK + (uint64_t)(((gs % KS) * C::TILE_BYTES) >> 4);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t o = ((kk >> 2) * C::CHUNK_BYTES + (kk & 3) * 32) >> 4;
                    umma_ss(tS, dQ + o, dKu + o, IDESC_QK, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[gs % NSB]);
                umma_commit(&k_empty[gs % KS]);
                ++gs;
                return true;
            };
            bool ok = true;
            TileCursor cur;
            for (cur.init(p, cfirst, cstep); ok && cur.w < total_tiles; cur.advance(p)) {
                const TileWork tw = tile_of(cur);
                if (tw.n_my == 0) continue;
                if (!mbar_wait(q_full, tc & 1)) {
                    report_fault(p.fault, FAULT_WAIT_Q, tc);
                    break;
                }
                int issued = 0;  // score blocks of this tile issued so far
                for (; ok && issued < NSB - 1 && issued < tw.n_my; ++issued) ok = issue_qk();
                if (ok && issued == tw.n_my) umma_commit(q_empty);
                for (int u = 0; ok && u < tw.n_my; ++u) {
                    if (issued < tw.n_my) {
                        ok = issue_qk();
                        if (!ok) break;
                        if (++issued == tw.n_my) umma_commit(q_empty);
                    }
                    if (!mbar_wait(&p_full[gp % NSB], (gp / NSB) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_P, gp);
                        ok = false;
                        break;
                    }
                    if (!mbar_wait(&v_full[gp % VS], (gp / VS) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_V, gp);
                        ok = false;
                        break;
                    }
                    if (u == 0 && tc > 0 && !mbar_wait(o_empty, (tc - 1) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_O, 0x100u + tc);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    // P from tensor memory: each 32-key chunk keeps its 16 bf16x2 columns at the start
                    // of its own 32 score columns, so 16 keys = 8 columns at 32*(ks/2) + 8*(ks%2).  V is
                    // MN-major: 64-element head-dim chunks 16 KB apart (leading offset), 8-key groups
                    // 1024 bytes apart (stride offset).
                    const uint32_t tS = tmem_base + C::COL_S + (gp % NSB) * 128;
                    const uint64_t dVu = dV + (uint64_t)(((gp % VS) * C::TILE_BYTES) >> 4);
#pragma unroll
                    for (int ks = 0; ks < C::BN / 16; ++ks) {
                        umma_ts(tO, tS + (ks >> 1) * 32 + (ks & 1) * 8, dVu + (uint64_t)((ks * 2048) >> 4), IDESC_PV,
                                (u > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(&v_empty[gp % VS]);
                    umma_commit(pv_done);
                    ++gp;
                }
                if (ok) umma_commit(o_full);
                ++tc;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / epilogue
        // Two threads per query row: warps 0-3 own keys 0-63 of every block (score columns
        // 0-63), warps 4-7 keys 64-127; both threads of a row sit in the same TMEM lane.
        const int kh = warp >> 2;       // 64-key half of each block
        const int quarter = warp & 3;   // TMEM lane quarter
        const int r = quarter * 32 + lane;
        constexpr int OC = HD / 2;  // output columns per thread
        const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t tS0 = tmem_base + lane_sel + C::COL_S + kh * 64;
        const uint32_t tO = tmem_base + lane_sel + C::COL_O + kh * OC;
        const float sl = p.scale_log2;
        constexpr bool has_mask = ADD_MASK;  // the additive-mask form is a kernel of its own: the common one stays small

        int gb = 0, tc = 0;  // key blocks and non-empty tiles processed so far
        int tn = 0;          // tiles seen (cluster merge: one phase of part_ready / read_done each)
        bool ok = true;
        uint32_t va[32], vb[32];  // this thread's 64 scores of the current block

        // Cluster merge at the end of a tile.  has_blocks: this CTA's key range of the tile is not empty
        // (m, l_share are then its row maximum and this thread's share of the row sum).
        //
        // Every CTA writes its unnormalised accumulator and (max, sum) per row into its own shared memory,
        // tells the cluster with one arrival per CTA, and folds rows [crank * 128 / CS, +128 / CS): a warp
        // takes an eighth of them, a lane 4 consecutive columns (twice for head dim 256) of every CTA's
        // share.  A lane's 16 (32) remote 16-byte loads are issued eight at a time before any is used — the
        // fold is bound by the latency of distributed shared memory, not by arithmetic.
        auto fold_rows = [&](const TileWork& tw, auto cs_tag) {
            constexpr int CS = decltype(cs_tag)::value;
            constexpr int WROWS = 128 / CS / C::SOFTMAX_WARPS;  // rows per warp
            constexpr int PIECES = HD / 128;                    // 16-byte pieces of a row per lane
            constexpr int ITEMS = WROWS * PIECES;               // (row, piece) items per lane
            constexpr int IB = CS >= 8 ? 1 : 8 / CS;            // items per batch: eight 16-byte loads in flight
            float* opart = reinterpret_cast<float*>(sK);
            const int row0 = crank * (128 / CS) + warp * WROWS;
            uint2 gv[IB];
            auto load_gates = [&](int it0) {
                if (!p.gate) return;
#pragma unroll
                for (int b = 0; b < IB; ++b) {
                    const int i = (it0 + b) / PIECES, j = (it0 + b) % PIECES;
                    const int tt = tw.q0 + row0 + i;
                    const long long eoff = tw.b * p.o_stride_b + tt * p.o_stride_t + (long long)tw.h * HD;
                    gv[b] = tt < p.seq ? *reinterpret_cast<const uint2*>(p.gate + eoff + (lane + 32 * j) * 4) : make_uint2(0u, 0u);
                }
            };
            // The gate values of the first batch depend on nothing here: request them before waiting for
            // the cluster (those of a later batch go out together with its loads).
            load_gates(0);
            if (!__all_sync(0xffffffffu, mbar_wait_cluster(part_ready, tn & 1))) {
                report_fault(p.fault, FAULT_WAIT_FULL, 0x700u);
                ok = false;
            }
            if (!ok) return;
            const uint32_t st_base = smem_u32(cl_stat), op_base = smem_u32(opart);
#pragma unroll 1
            for (int it0 = 0; it0 < ITEMS; it0 += IB) {
                float4 o[IB][CS];
                float2 st[IB][CS];
                if (it0 > 0) load_gates(it0);
#pragma unroll
                for (int b = 0; b < IB; ++b) {
                    const int i = (it0 + b) / PIECES, j = (it0 + b) % PIECES;
                    const int rr = row0 + i;
                    const uint32_t off = (uint32_t)(rr * HD + (((lane + 32 * j) ^ (rr & 7)) << 2)) * 4u;
#pragma unroll
                    for (int c = 0; c < CS; ++c) {
                        st[b][c] = ld_cluster_f32x2(map_to_cta(st_base + rr * 8, c));
                        o[b][c] = ld_cluster_f32x4(map_to_cta(op_base + off, c));
                    }
                }
#pragma unroll
                for (int b = 0; b < IB; ++b) {
                    const int i = (it0 + b) / PIECES, j = (it0 + b) % PIECES;
                    const int rr = row0 + i;
                    float mx = -CUDART_INF_F, ltot = 0.f;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int c = 0; c < CS; ++c) mx = fmaxf(mx, st[b][c].x);
#pragma unroll
                    for (int c = 0; c < CS; ++c) {
                        // a CTA without key blocks wrote no rows: whatever was read from it is not used
                        const float w = st[b][c].x != -CUDART_INF_F ? fast_exp2(st[b][c].x - mx) : 0.f;
                        ltot = fmaf(w, st[b][c].y, ltot);
                        if (w != 0.f) {
                            acc.x = fmaf(w, o[b][c].x, acc.x);
                            acc.y = fmaf(w, o[b][c].y, acc.y);
                            acc.z = fmaf(w, o[b][c].z, acc.z);
                            acc.w = fmaf(w, o[b][c].w, acc.w);
                        }
                    }
                    const float inv = ltot > 0.f ? 1.0f / ltot : 0.f;
                    const int tt = tw.q0 + rr;
                    if (tt >= p.seq) continue;
                    const long long eoff = tw.b * p.o_stride_b + tt * p.o_stride_t + (long long)tw.h * HD;
                    float o4[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
                    if (p.gate) {
                        o4[0] = sigmoid_gate_bits(o4[0], (uint16_t)(gv[b].x & 0xffffu));
                        o4[1] = sigmoid_gate_bits(o4[1], (uint16_t)(gv[b].x >> 16));
                        o4[2] = sigmoid_gate_bits(o4[2], (uint16_t)(gv[b].y & 0xffffu));
                        o4[3] = sigmoid_gate_bits(o4[3], (uint16_t)(gv[b].y >> 16));
                    }
                    const uint2 packed = make_uint2(pack_bf16x2(o4[0], o4[1]), pack_bf16x2(o4[2], o4[3]));
                    *reinterpret_cast<uint2*>(p.out + eoff + (lane + 32 * j) * 4) = packed;
                    for (int c = 0; c < p.n_copies; ++c)
                        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.out_copies[c]) + eoff + (lane + 32 * j) * 4) = packed;
                    if (j == 0 && lane == 0 && p.out_lse)
                        p.out_lse[((long long)tw.b * p.seq + tt) * p.nq + tw.h] =
                            ltot > 0.f ? (mx + fast_log2(ltot)) * 0.6931471805599453f : -CUDART_INF_F;
                }
            }
        };
        auto cluster_tile_end = [&](const TileWork& tw, float m, float l_share, bool has_blocks) {
            float* opart = reinterpret_cast<float*>(sK);  // [128 rows][HD] fp32, 16-byte pieces swizzled by row & 7
            float l = 0.f;
            // the previous tile's share (rows and statistics) must have been read by the whole cluster before
            // this one overwrites it
            if (tn > 0 && !__all_sync(0xffffffffu, mbar_wait_cluster(read_done, (tn - 1) & 1))) {
                report_fault(p.fault, FAULT_WAIT_EMPTY, 0x500u);
                ok = false;
            }
            if (has_blocks) {
                xch_sum[kh * 128 + r] = l_share;
                pair_sync(quarter);
                l = xch_sum[r] + xch_sum[128 + r];
                if (ok && !mbar_wait_warp(o_full, tc & 1)) {
                    report_fault(p.fault, FAULT_WAIT_O, tc);
                    ok = false;
                }
                ++tc;
                if (ok) {
                    tc_fence_after_sync();
                    // this thread's half of the row, unnormalised, into this CTA's shared memory (every MMA
                    // that read the K / V buffers has completed: o_full follows them)
#pragma unroll 1
                    for (int c = 0; c < OC / 32; c += 2) {
                        tmem_ld32(tO + c * 32, va);
                        tmem_ld32(tO + c * 32 + 32, vb);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 64; e += 4) {
                            const uint32_t* src = e < 32 ? va + e : vb + (e - 32);
                            const int piece = (kh * OC + c * 32 + e) >> 2;
                            *reinterpret_cast<float4*>(opart + r * HD + ((piece ^ (r & 7)) << 2)) =
                                make_float4(__uint_as_float(src[0]), __uint_as_float(src[1]), __uint_as_float(src[2]),
                                            __uint_as_float(src[3]));
                        }
                    }
                    tc_fence_before_sync();
                    mbar_arrive(o_empty);  // the accumulator is out: the next tile may overwrite it
                }
            }
            if (kh == 0) cl_stat[r] = make_float2(has_blocks ? m : -CUDART_INF_F, l);
            // my CTA's share is written once all 256 softmax threads are here: one thread tells every CTA of
            // the cluster (release at cluster scope, cumulative over what the barrier ordered before it)
            const uint32_t pr = smem_u32(part_ready), rd = smem_u32(read_done);
            softmax_sync();
            if (threadIdx.x == 0) {
                fence_acq_rel_cluster();
                for (int c = 0; c < csize; ++c) mbar_arrive_cluster(map_to_cta(pr, c));
            }
            if (csize == 2) fold_rows(tw, std::integral_constant<int, 2>{});  // the host launches clusters of 2 or 4
            else fold_rows(tw, std::integral_constant<int, 4>{});
            // every softmax thread of this CTA is done reading the cluster's shared memory
            softmax_sync();
            if (threadIdx.x == 0) {
                for (int c = 0; c < csize; ++c) mbar_arrive_cluster(map_to_cta(rd, c));
            }
            ++tn;
        };

        TileCursor cur;
        for (cur.init(p, cfirst, cstep); cur.w < total_tiles; cur.advance(p)) {
            const TileWork tw = tile_of(cur);
            const int t = tw.q0 + r;
            const long long row = ((long long)tw.b * p.seq + t) * p.nq + tw.h;
            if (CLUSTER && tw.n_my == 0) {
                cluster_tile_end(tw, -CUDART_INF_F, 0.f, false);  // the other CTAs of the cluster may have key blocks
                continue;
            }
            if (tw.n_my == 0) {
                // Nothing visible: zero output (or an empty partial) for this tile.
                if (t < p.seq) {
                    if (p.num_splits > 1) {
                        float4* dst = reinterpret_cast<float4*>(p.part_o + ((long long)tw.split * rows_total + row) * HD + kh * OC);
                        for (int i = 0; i < OC / 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (kh == 0) p.part_lse[(long long)tw.split * rows_total + row] = -CUDART_INF_F;
                    } else {
                        const long long zoff = tw.b * p.o_stride_b + t * p.o_stride_t + (long long)tw.h * HD + kh * OC;
                        for (int c = -1; c < p.n_copies; ++c) {
                            uint4* dst = reinterpret_cast<uint4*>((c < 0 ? p.out : reinterpret_cast<uint16_t*>(p.out_copies[c])) + zoff);
                            for (int i = 0; i < OC / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                        }
                        if (kh == 0 && p.out_lse) p.out_lse[row] = -CUDART_INF_F;
                    }
                }
                continue;
            }

            int row_lo = 0, row_hi = p.kv_len;  // visible keys [row_lo, row_hi)
            if (causal) {
                const int diag = t + off;
                row_hi = min(max(diag + 1, 0), p.kv_len);
                if (p.vis_hi && t < p.seq) row_hi = p.vis_hi[t];  // a vision block's later keys are visible too
                if (windowed) row_lo = max(0, diag - p.window + 1);
                if (row_lo > row_hi) row_lo = row_hi;
            }
            const float* mask_row = has_mask && t < p.seq ? p.mask + (long long)t * p.kv_len : nullptr;
            const RowMask rm{row_lo, row_hi, p.kv_len, mask_row};

            float m = -CUDART_INF_F;  // running max, log2 domain, possibly stale by <= 8
            float l = 0.f;            // this thread's share of the row sum

            // Partial maximum of the tile's block u (global block g = gb + u) over this thread's
            // 64 keys, published for the row's other thread.  False if the scores never arrived.
            // (The scores are fetched again for the exponentials: holding both blocks' 128 values
            // in registers at once does not fit next to the working set.)
            auto publish_max = [&](int u) -> bool {
                const int g = gb + u;
                if (!mbar_wait_warp(&s_full[g % NSB], (g / NSB) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_S, g);
                    return false;
                }
                tc_fence_after_sync();
                uint32_t wa[32], wb[32];
                tmem_ld32(tS0 + (g % NSB) * 128, wa);
                tmem_ld32(tS0 + (g % NSB) * 128 + 32, wb);
                tmem_wait_ld();
                const int kc = (tw.my_lo + u) * C::BN + kh * 64;
                float mr[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                float ms[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                if (has_mask) {
                    chunk_max_any<true>(wa, mr, ms, sl, kc, rm);
                    chunk_max_any<true>(wb, mr, ms, sl, kc + 32, rm);
                } else {
                    chunk_max_any<false>(wa, mr, ms, sl, kc, rm);
                    chunk_max_any<false>(wb, mr, ms, sl, kc + 32, rm);
                }
                xch_max[(g & 1) * 256 + kh * 128 + r] = fmaxf(fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * sl,
                                                             fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3])));
                return true;
            };

            if constexpr (NSB >= 3) {
                // Block 0: publish, meet, adopt the row maximum, fetch the scores.
                if (ok) ok = publish_max(0);
                pair_sync(quarter);
                if (ok) {
                    const float* xm = xch_max + (gb & 1) * 256;
                    m = fmaxf(xm[r], xm[128 + r]);
                    tmem_ld32(tS0 + (gb % NSB) * 128, va);
                    tmem_ld32(tS0 + (gb % NSB) * 128 + 32, vb);
                    tmem_wait_ld();
                }

                for (int i = 0; i < tw.n_my; ++i) {
                    const int g = gb + i;
                    const int kc = (tw.my_lo + i) * C::BN + kh * 64;
                    const uint32_t tS = tS0 + (g % NSB) * 128;
                    const bool have_next = i + 1 < tw.n_my;
                    // The next block's scores were computed one or two blocks ago: take their maximum
                    // now, so that the exchange through shared memory is hidden behind this block's
                    // exponentials.
                    if (ok && have_next) ok = publish_max(i + 1);
                    if (ok) {
                        // Probabilities of block i as bf16: each 32-key chunk over the first 16 of its
                        // own 32 score columns; row-sum share in fp32.
                        const float m_eff = (m == -CUDART_INF_F) ? 0.f : m;
                        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
                        uint32_t pk[16];
                        if (has_mask) {
                            chunk_exp_any<true>(va, pk, ls4, sl, m_eff, kc, rm);
                            tmem_st16(tS, pk);
                            chunk_exp_any<true>(vb, pk, ls4, sl, m_eff, kc + 32, rm);
                            tmem_st16(tS + 32, pk);
                        } else {
                            chunk_exp_any<false>(va, pk, ls4, sl, m_eff, kc, rm);
                            tmem_st16(tS, pk);
                            chunk_exp_any<false>(vb, pk, ls4, sl, m_eff, kc + 32, rm);
                            tmem_st16(tS + 32, pk);
                        }
                        l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
                        tmem_wait_st();
                        tc_fence_before_sync();
                        mbar_arrive(&p_full[g % NSB]);
                        if (have_next) {  // lands during the barrier below
                            tmem_ld32(tS0 + ((g + 1) % NSB) * 128, va);
                            tmem_ld32(tS0 + ((g + 1) % NSB) * 128 + 32, vb);
                        }
                    }
                    if (!have_next) break;
                    pair_sync(quarter);
                    if (!ok) continue;
                    const float* xm = xch_max + ((g + 1) & 1) * 256;
                    const float m_new = fmaxf(m, fmaxf(xm[r], xm[128 + r]));
                    const bool need = m_new > m + 8.0f;
                    if (__any_sync(0xffffffffu, need)) {
                        // Rare: the row maximum grows by more than 2^8 with the next block.  Once
                        // O += P V of block i has landed, rescale this thread's half of O in tensor
                        // memory (the row's other thread takes the same decision from the same values).
                        const float alpha = (m_new == -CUDART_INF_F) ? 1.0f : fast_exp2(m - m_new);
                        tmem_wait_ld();
                        if (!mbar_wait_warp(pv_done, g & 1)) {
                            report_fault(p.fault, FAULT_WAIT_O, g);
                            ok = false;
                            continue;
                        }
                        tc_fence_after_sync();
                        uint32_t ww[32];
    #pragma unroll 1
                        for (int c = 0; c < OC / 32; ++c) {
                            tmem_ld32(tO + c * 32, ww);
                            tmem_wait_ld();
    #pragma unroll
                            for (int e = 0; e < 32; ++e) ww[e] = __float_as_uint(__uint_as_float(ww[e]) * alpha);
                            tmem_st32(tO + c * 32, ww);
                        }
                        tmem_wait_st();
                        l *= alpha;
                        m = m_new;
                    }
                    tmem_wait_ld();
                }
            } else {
                // Two score buffers leave no room to look ahead: S(i+1) can only be computed once P(i-1) has
                // been consumed, so waiting for it before the exponentials of block i would put the tensor
                // pipe and the softmax in series.  Here every block is taken on its own: maximum, exchange,
                // exponentials; meanwhile the tensor pipe runs O += P(i-1) V(i-1) and S(i+1).
                for (int i = 0; i < tw.n_my; ++i) {
                    const int g = gb + i;
                    const int kc = (tw.my_lo + i) * C::BN + kh * 64;
                    const uint32_t tS = tS0 + (g % NSB) * 128;
                    if (ok && !mbar_wait_warp(&s_full[g % NSB], (g / NSB) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_S, g);
                        ok = false;
                    }
                    if (ok) {
                        tc_fence_after_sync();
                        tmem_ld32(tS, va);
                        tmem_ld32(tS + 32, vb);
                        tmem_wait_ld();
                        float mr[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                        float ms[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                        chunk_max_any<has_mask>(va, mr, ms, sl, kc, rm);
                        chunk_max_any<has_mask>(vb, mr, ms, sl, kc + 32, rm);
                        xch_max[(g & 1) * 256 + kh * 128 + r] = fmaxf(fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * sl,
                                                                     fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3])));
                    }
                    pair_sync(quarter);
                    if (!ok) continue;
                    const float* xm = xch_max + (g & 1) * 256;
                    const float m_new = fmaxf(m, fmaxf(xm[r], xm[128 + r]));
                    if (i == 0) {
                        m = m_new;  // nothing accumulated yet
                    } else if (__any_sync(0xffffffffu, m_new > m + 8.0f)) {
                        // Rare: the row maximum grows by more than 2^8.  Once O += P V of the previous block has
                        // landed, rescale this thread's half of O in tensor memory (the row's other thread takes
                        // the same decision from the same values).
                        const float alpha = (m_new == -CUDART_INF_F) ? 1.0f : fast_exp2(m - m_new);
                        if (!mbar_wait_warp(pv_done, (g - 1) & 1)) {
                            report_fault(p.fault, FAULT_WAIT_O, g);
                            ok = false;
                            continue;
                        }
                        tc_fence_after_sync();
                        uint32_t ww[32];
#pragma unroll 1
                        for (int c = 0; c < OC / 32; ++c) {
                            tmem_ld32(tO + c * 32, ww);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 32; ++e) ww[e] = __float_as_uint(__uint_as_float(ww[e]) * alpha);
                            tmem_st32(tO + c * 32, ww);
                        }
                        tmem_wait_st();
                        l *= alpha;
                        m = m_new;
                    }
                    const float m_eff = (m == -CUDART_INF_F) ? 0.f : m;
                    float ls4[4] = {0.f, 0.f, 0.f, 0.f};
                    uint32_t pk[16];
                    chunk_exp_any<has_mask>(va, pk, ls4, sl, m_eff, kc, rm);
                    tmem_st16(tS, pk);
                    chunk_exp_any<has_mask>(vb, pk, ls4, sl, m_eff, kc + 32, rm);
                    tmem_st16(tS + 32, pk);
                    l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(&p_full[g % NSB]);
                }
            }
            gb += tw.n_my;
            if constexpr (CLUSTER) {
                cluster_tile_end(tw, m, l, true);
                continue;
            }

            // Row sum = the two threads' shares.
            xch_sum[kh * 128 + r] = l;
            pair_sync(quarter);
            l = xch_sum[r] + xch_sum[128 + r];
            if (ok && !mbar_wait_warp(o_full, tc & 1)) {
                report_fault(p.fault, FAULT_WAIT_O, tc);
                ok = false;
            }
            ++tc;
            if (!ok) continue;
            tc_fence_after_sync();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const float lse = l > 0.f ? (m + fast_log2(l)) * 0.6931471805599453f : -CUDART_INF_F;
            const bool store = t < p.seq;
            if (p.num_splits > 1) {
                float* dst = p.part_o + ((long long)tw.split * rows_total + row) * HD + kh * OC;
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
                // O is in registers / on its way out: the next tile may overwrite the accumulator.
                tc_fence_before_sync();
                mbar_arrive(o_empty);
                if (store && kh == 0) p.part_lse[(long long)tw.split * rows_total + row] = lse;
            } else {
                const long long eoff = tw.b * p.o_stride_b + t * p.o_stride_t + (long long)tw.h * HD + kh * OC;
                uint16_t* dst = p.out + eoff;
                const uint16_t* gp = (GATE && p.gate) ? p.gate + eoff : nullptr;
                // One thread writes 128 (or 256) contiguous bytes of its row.
#pragma unroll 1
                for (int c = 0; c < OC / 32; ++c) {
                    tmem_ld32(tO + c * 32, va);
                    tmem_wait_ld();
                    if (c == OC / 32 - 1) {
                        tc_fence_before_sync();
                        mbar_arrive(o_empty);
                    }
                    if (store) {
#pragma unroll
                        for (int e = 0; e < 32; e += 16) {
                            uint32_t ov[8];
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                float o[8];
#pragma unroll
                                for (int u = 0; u < 8; ++u) o[u] = __uint_as_float(va[e + hh * 8 + u]) * inv;
                                if (gp) {
                                    const uint4 gv = *reinterpret_cast<const uint4*>(gp + c * 32 + e + hh * 8);
                                    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                                    for (int u = 0; u < 8; ++u) {
                                        const float gf = bf16_bits_to_f32(static_cast<uint16_t>(gw[u >> 1] >> ((u & 1) * 16)));
                                        const float sig = 1.0f / (1.0f + __expf(-gf));
                                        o[u] = bf16_round(o[u]) * sig;
                                    }
                                }
#pragma unroll
                                for (int u = 0; u < 4; ++u) ov[hh * 4 + u] = pack_bf16x2(o[2 * u], o[2 * u + 1]);
                            }
                            store_bf16x16(dst + c * 32 + e, ov);
                            if (p.n_copies) store_copies_bf16x16(p.out_copies, p.n_copies, eoff + c * 32 + e, ov);
                        }
                    }
                }
                if (store && kh == 0 && p.out_lse) p.out_lse[row] = lse;
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == PRODUCER_WARP) tmem_dealloc(tmem_base, C::TMEM_COLS);
    // A launch that covers the tail of a two-tile launch's unit list runs beside that launch (programmatic
    // stream serialization) and reads nothing it writes — but whatever follows in the stream waits for this
    // grid only, so this grid does not complete before the one in front of it has: every CTA ends on the
    // grid-dependency wait (a no-op for launches without the attribute).
    if (p.tail_base >= 0) grid_dependency_wait();
    // A CTA's shared memory may be read by the others only while it is alive: nobody leaves before the
    // whole cluster is through (all threads are still running here).
    if constexpr (CLUSTER) cluster_sync_all();
}

}  // namespace arc
