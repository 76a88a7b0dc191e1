// GQA flash-attention prefill / canvas kernel for sm_100a.
//
// One CTA owns one or two tiles of 128 query tokens of one query head each and
// walks the key blocks (128 keys) those tiles can see.  Q, K and V tiles are staged in shared
// memory by TMA (128-byte swizzle, one 64-element column chunk per copy);
// S = Q K^T and O += P V run on the tcgen05 tensor cores with both accumulators
// in tensor memory; P is written back to tensor memory as bf16 over the S
// columns and fed to the second MMA from there, so probabilities never touch
// shared or global memory.  Softmax is online, fp32, one query row per thread.
//
// Warp roles: per tile eight softmax / correction / epilogue warps, two threads per
// query row (warp index mod 4 selects the 32 TMEM lanes, the next bit the key half
// of each block), then one TMA producer warp (also the TMEM owner) and one MMA
// issuing warp.
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
    int pair_heads;  // NT == 2: 1 = the CTA's tiles are query heads 2y, 2y+1; 0 = token tiles 2x, 2x+1
#ifdef ARC_PREFILL_TRACE
    long long* trace;  // debug builds only: per-block timestamps of CTA 0
#endif
};

// NT = query tiles (128 rows each) one CTA works on.  hd128 pairs two tiles that
// share every K/V block (two query heads of one KV head, or two consecutive token
// tiles) on one SM: both S/O accumulator sets fill the 512 TMEM columns, and a
// single MMA-issuing thread alternates between the tiles, so one tile's softmax
// always runs under the other tile's MMAs.  hd256 has room for one tile.
template <int HD>
struct PrefillCfg {
    static constexpr int NT = (HD == 128) ? 2 : 1;
    static constexpr int BM = 128;  // query rows per tile
    static constexpr int BN = 128;  // keys per block
    static constexpr int CH = HD / 64;
    static constexpr int CHUNK_BYTES = 128 * 128;  // 128 rows x 64 bf16
    static constexpr int TILE_BYTES = CH * CHUNK_BYTES;
    static constexpr int STAGES = (HD == 128) ? 2 : 1;  // K and V ring depth
    static constexpr int TMEM_COLS = 512;
    static constexpr int TILE_COLS = 128 + HD;  // per tile: S (128 fp32 columns, P aliases them) then O
    static constexpr int NUM_BARS = 1 + 4 * STAGES + 3 * NT;
    static constexpr int XCH_FLOATS = 2 * 2 * 128 + 2 * 128;  // per tile: row-max exchange (2 phases) + row-sum exchange
    static constexpr int SMEM_BYTES = (NT + 2 * STAGES) * TILE_BYTES + NUM_BARS * 8 + 16 + NT * XCH_FLOATS * 4 + 1024;
    static constexpr int SOFTMAX_WARPS = 8 * NT;  // two threads per query row
    static constexpr int THREADS = 32 * (SOFTMAX_WARPS + 2);
    static constexpr int MAX_REGS = (NT == 2) ? 96 : 168;  // 65536 registers over the warps of a CTA, allocated four warps at a time
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


// Barrier between the two warps that share a set of 32 query rows of one tile: hardware
// barrier `id`, 64 threads.  Every softmax warp of an active tile executes exactly one
// pair_sync per key block and one after the loop, whatever happened to its waits, so
// neither warp of a pair can be left waiting here.
__device__ __forceinline__ void pair_sync(int id) {
    asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

// Geometry of one query tile of a CTA.
struct TileGeom {
    int q0;     // first query token
    int head;   // query head
    int lo, n;  // key blocks [lo, lo + n) this tile (and split) walks; n == 0: nothing to do
    bool valid; // tile exists (token tiles: the last CTA of an odd count has one tile only)
};

template <int HD>
__device__ __forceinline__ TileGeom tile_geometry(const PrefillParams& p, int x, int split) {
    using C = PrefillCfg<HD>;
    TileGeom g;
    if (C::NT == 2 && p.pair_heads) {
        g.q0 = blockIdx.x * C::BM;
        g.head = blockIdx.y * 2 + x;
    } else {
        g.q0 = (blockIdx.x * C::NT + x) * C::BM;
        g.head = blockIdx.y;
    }
    g.valid = g.q0 < p.seq;
    g.lo = 0;
    g.n = 0;
    if (!g.valid) return g;
    const int off = p.kv_len - p.seq;
    const bool causal = (p.mask_type == 3);
    const bool windowed = causal && p.window > 0 && p.window != 0x7fffffff;
    const int q_last = min(g.q0 + C::BM - 1, p.seq - 1);
    int blk_lo = 0, blk_hi = (p.kv_len + C::BN - 1) / C::BN;
    if (causal) {
        const int last_key = min(p.kv_len - 1, q_last + off);
        blk_hi = last_key >= 0 ? last_key / C::BN + 1 : 0;
        if (windowed) blk_lo = max(0, g.q0 + off - p.window + 1) / C::BN;
    }
    const int nblk = max(0, blk_hi - blk_lo);
    const int per = (nblk + p.num_splits - 1) / p.num_splits;
    g.lo = blk_lo + split * per;
    g.n = max(0, min(blk_hi, g.lo + per) - g.lo);
    return g;
}

template <int HD>
__global__ void __maxnreg__(PrefillCfg<HD>::MAX_REGS)
    sdpa_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    using C = PrefillCfg<HD>;
    constexpr int NT = C::NT;
    constexpr int ST = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                              // [NT] tiles
    uint8_t* sK = smem + NT * C::TILE_BYTES;         // [ST] stages
    uint8_t* sV = sK + ST * C::TILE_BYTES;           // [ST] stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + ST * C::TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = k_full + ST;
    uint64_t* v_full = k_empty + ST;
    uint64_t* v_empty = v_full + ST;
    uint64_t* s_full = v_empty + ST;  // [NT]
    uint64_t* p_full = s_full + NT;   // [NT]
    uint64_t* o_full = p_full + NT;   // [NT]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NUM_BARS);
    uint32_t* abort_slot = tmem_slot + 1;
    float* xch = reinterpret_cast<float*>(tmem_slot + 4);  // per tile: max [2][2][128], sum [2][128]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.z / p.num_splits;
    const int split = blockIdx.z % p.num_splits;
    const long long rows_total = (long long)p.batch * p.seq * p.nq;

    TileGeom tg[NT];
    int u_lo = 0x7fffffff, u_hi = 0;  // union of the tiles' block ranges
#pragma unroll
    for (int x = 0; x < NT; ++x) {
        tg[x] = tile_geometry<HD>(p, x, split);
        if (tg[x].n > 0) {
            u_lo = min(u_lo, tg[x].lo);
            u_hi = max(u_hi, tg[x].lo + tg[x].n);
        }
    }
    const int n_u = max(0, u_hi - u_lo);
    const int kvh = tg[0].head / (p.nq / p.nkv);  // both tiles share the KV head

    if (threadIdx.x == 0) *abort_slot = (*reinterpret_cast<volatile uint32_t*>(p.fault) != 0u) ? 1u : 0u;
    __syncthreads();
    if (*abort_slot) return;

    // Tiles with nothing visible: zero output (or an empty partial), written by the first
    // four warps of the tile's softmax group.
#pragma unroll
    for (int x = 0; x < NT; ++x) {
        if (tg[x].valid && tg[x].n == 0 && warp >= 8 * x && warp < 8 * x + 4) {
            const int t = tg[x].q0 + (warp & 3) * 32 + lane;
            if (t < p.seq) {
                const long long row = ((long long)b * p.seq + t) * p.nq + tg[x].head;
                if (p.num_splits > 1) {
                    float4* dst = reinterpret_cast<float4*>(p.part_o + ((long long)split * rows_total + row) * HD);
                    for (int i = 0; i < HD / 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    p.part_lse[(long long)split * rows_total + row] = -CUDART_INF_F;
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(p.out + b * p.o_stride_b + t * p.o_stride_t +
                                                          (long long)tg[x].head * HD);
                    for (int i = 0; i < HD / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                    if (p.out_lse) p.out_lse[row] = -CUDART_INF_F;
                }
            }
        }
    }
    if (n_u == 0) return;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < ST; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int x = 0; x < NT; ++x) {
            mbar_init(&s_full[x], 1);
            mbar_init(&p_full[x], 256);
            mbar_init(&o_full[x], 1);
        }
        fence_mbar_init();
    }
    constexpr int PRODUCER_WARP = C::SOFTMAX_WARPS;
    constexpr int MMA_WARP = C::SOFTMAX_WARPS + 1;
    if (warp == PRODUCER_WARP) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == PRODUCER_WARP) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&tm_q);
            prefetch_tensormap(&tm_k);
            prefetch_tensormap(&tm_v);
            int n_q = 0;
#pragma unroll
            for (int x = 0; x < NT; ++x) n_q += (tg[x].n > 0) ? 1 : 0;
            mbar_arrive_expect_tx(q_full, n_q * C::TILE_BYTES);
#pragma unroll
            for (int x = 0; x < NT; ++x) {
                if (tg[x].n > 0) {
#pragma unroll
                    for (int c = 0; c < C::CH; ++c)
                        tma_load_4d(sQ + x * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_q, q_full, c * 64, tg[x].head,
                                    tg[x].q0, b);
                }
            }
            for (int u = 0; u < n_u; ++u) {
                const int st = u % ST;
                const int key0 = (u_lo + u) * C::BN;
                if (u >= ST && !mbar_wait(&k_empty[st], ((u / ST) - 1) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_EMPTY, 0x100u + u);
                    break;
                }
                mbar_arrive_expect_tx(&k_full[st], C::TILE_BYTES);
#pragma unroll
                for (int c = 0; c < C::CH; ++c)
                    tma_load_4d(sK + st * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_k, &k_full[st], c * 64, kvh, key0, b);
                if (u >= ST && !mbar_wait(&v_empty[st], ((u / ST) - 1) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_EMPTY, 0x200u + u);
                    break;
                }
                mbar_arrive_expect_tx(&v_full[st], C::TILE_BYTES);
#pragma unroll
                for (int c = 0; c < C::CH; ++c)
                    tma_load_4d(sV + st * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_v, &v_full[st], c * 64, kvh, key0, b);
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        // One thread issues, for every key block u of the union range and every tile x that
        // sees it:  O_x += P_x(u) V(u)  followed at once by  S_x = Q_x K(u+1)^T.  With two
        // tiles the tensor pipe therefore runs tile A's pair of MMAs, then tile B's, and so
        // on, and each tile's softmax has the other tile's MMA time to finish.
        if (lane == 0) {
            constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, false);
            constexpr uint32_t IDESC_PV = make_idesc_bf16(128, HD, true);
            const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
            int done[NT];  // blocks of tile x whose PV has been issued
#pragma unroll
            for (int x = 0; x < NT; ++x) done[x] = 0;
            auto sees = [&](int x, int u) {
                return tg[x].n > 0 && u_lo + u >= tg[x].lo && u_lo + u < tg[x].lo + tg[x].n;
            };
            auto issue_qk = [&](int x, int st) {
                const uint32_t tS = tmem_base + x * C::TILE_COLS;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t o = (kk >> 2) * C::CHUNK_BYTES + (kk & 3) * 32;
                    umma_ss(tS, make_smem_desc_sw128(aQ + x * C::TILE_BYTES + o, 16, 1024),
                            make_smem_desc_sw128(aK + st * C::TILE_BYTES + o, 16, 1024), IDESC_QK, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[x]);
            };
            bool ok = mbar_wait(q_full, 0);
            if (!ok) report_fault(p.fault, FAULT_WAIT_Q, 0);
            if (ok && !mbar_wait(&k_full[0], 0)) {
                report_fault(p.fault, FAULT_WAIT_K, 0);
                ok = false;
            }
            if (ok) {
                tc_fence_after_sync();
#pragma unroll
                for (int x = 0; x < NT; ++x)
                    if (sees(x, 0)) issue_qk(x, 0);
                umma_commit(&k_empty[0]);
            }
            for (int u = 0; ok && u < n_u; ++u) {
                const int st = u % ST;
                const int st1 = (u + 1) % ST;
                bool v_ready = false, k_ready = false;
#pragma unroll
                for (int x = 0; x < NT; ++x) {
                    if (ok && sees(x, u)) {
                        if (!mbar_wait(&p_full[x], done[x] & 1)) {
                            report_fault(p.fault, FAULT_WAIT_P, u);
                            ok = false;
                        }
#ifdef ARC_PREFILL_TRACE
                        if (p.trace && blockIdx.x == 20 && blockIdx.y == 0 && blockIdx.z == 0 && u < 16)
                            p.trace[u * 16 + 11 + 2 * x] = clock64();
#endif
                        if (ok && !v_ready) {
                            if (!mbar_wait(&v_full[st], (u / ST) & 1)) {
                                report_fault(p.fault, FAULT_WAIT_V, u);
                                ok = false;
                            }
                            v_ready = true;
                        }
                        if (ok) {
                            tc_fence_after_sync();
                            // P from tensor memory, 8 columns per 16 keys; the two key halves of a
                            // block keep their P at the start of their own S columns (keys 0-63 at
                            // columns 0-31, keys 64-127 at columns 64-95).  V is MN-major: 64-element
                            // head-dim chunks 16 KB apart (leading offset), 8-key groups 1024 bytes
                            // apart (stride offset).
                            const uint32_t tS = tmem_base + x * C::TILE_COLS;
                            const uint32_t tO = tS + 128;
#pragma unroll
                            for (int ks = 0; ks < C::BN / 16; ++ks) {
                                const uint32_t pcol = (ks < 4) ? ks * 8 : 64 + (ks - 4) * 8;
                                umma_ts(tO, tS + pcol,
                                        make_smem_desc_sw128(aV + st * C::TILE_BYTES + ks * 2048, C::CHUNK_BYTES, 1024),
                                        IDESC_PV, (done[x] > 0 || ks > 0) ? 1u : 0u);
                            }
                            ++done[x];
                            if (done[x] == tg[x].n) umma_commit(&o_full[x]);
                        }
                    }
                    if (ok && u + 1 < n_u && sees(x, u + 1)) {
                        if (!k_ready) {
                            if (!mbar_wait(&k_full[st1], ((u + 1) / ST) & 1)) {
                                report_fault(p.fault, FAULT_WAIT_K, u + 1);
                                ok = false;
                            }
                            k_ready = true;
                        }
                        if (ok) {
                            tc_fence_after_sync();
                            issue_qk(x, st1);
#ifdef ARC_PREFILL_TRACE
                            if (p.trace && blockIdx.x == 20 && blockIdx.y == 0 && blockIdx.z == 0 && u < 16)
                                p.trace[u * 16 + 12 + 2 * x] = clock64();
#endif
                        }
                    }
                }
                if (ok) {
                    umma_commit(&v_empty[st]);
                    if (u + 1 < n_u) umma_commit(&k_empty[st1]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / epilogue
        // Two threads per query row: warps 0-3 of a tile's group own keys 0-63 of every block
        // (S columns 0-63), warps 4-7 keys 64-127; both halves of a row sit in the same TMEM lane.
        const int x = warp >> 3;            // tile of this warp
        const int half = (warp >> 2) & 1;   // key half
        const int quarter = warp & 3;       // TMEM lane quarter
        const TileGeom g = tg[x < NT ? x : 0];
        if (g.n > 0) {
            const int pair_id = 1 + x * 4 + quarter;
            const int r = quarter * 32 + lane;
            const int t = g.q0 + r;
            constexpr int OC = HD / 2;  // output columns per thread
            const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
            const uint32_t tS = tmem_base + lane_sel + x * C::TILE_COLS + half * 64;
            const uint32_t tO = tmem_base + lane_sel + x * C::TILE_COLS + 128 + half * OC;
            float* xch_max = xch + x * C::XCH_FLOATS;  // [phase 2][half 2][row 128]
            float* xch_sum = xch_max + 2 * 2 * 128;    // [half 2][row 128]
            const float sl = p.scale_log2;
            const int off = p.kv_len - p.seq;
            const bool causal = (p.mask_type == 3);
            const bool windowed = causal && p.window > 0 && p.window != 0x7fffffff;

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

            for (int i = 0; i < g.n; ++i) {
                const int kc = (g.lo + i) * C::BN + half * 64;
#ifdef ARC_PREFILL_TRACE
                const bool tr = p.trace && blockIdx.x == 20 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0 && i < 16;
                if (tr) p.trace[i * 16 + 0] = clock64();
#endif
                if (ok && !mbar_wait_warp(&s_full[x], i & 1)) {
                    report_fault(p.fault, FAULT_WAIT_S, i);
                    ok = false;
                }
                if (!ok) {
                    // Gave up on a wait: keep meeting the partner warp at the pair barrier so it
                    // can never be left waiting there, but touch nothing else.
                    pair_sync(pair_id);
                    continue;
                }
                tc_fence_after_sync();
#ifdef ARC_PREFILL_TRACE
                if (tr) p.trace[i * 16 + 1] = clock64();
#endif
#ifdef ARC_PREFILL_SKIP_SOFTMAX
                // Experiment only: no softmax work at all, to time the TMA + MMA pipeline alone.
                tc_fence_before_sync();
                mbar_arrive(&p_full[x]);
                pair_sync(pair_id);
                continue;
#endif
                tmem_ld32(tS, va);
                tmem_ld32(tS + 32, vb);
                tmem_wait_ld();
#ifdef ARC_PREFILL_TRACE
                if (tr) p.trace[i * 16 + 8] = clock64();
#endif

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
#ifdef ARC_PREFILL_TRACE
                if (tr) p.trace[i * 16 + 9] = clock64();
#endif
                xch_max[((i & 1) * 2 + half) * 128 + r] = m_half;
                pair_sync(pair_id);
                const float m_blk = fmaxf(m_half, xch_max[((i & 1) * 2 + (half ^ 1)) * 128 + r]);
#ifdef ARC_PREFILL_TRACE
                if (tr) p.trace[i * 16 + 2] = clock64();
#endif
                const float m_new = fmaxf(m, m_blk);
                if (i == 0) {
                    m = m_new;
                } else {
                    const bool need = m_new > m + 8.0f;
                    if (__any_sync(0xffffffffu, need)) {
                        // Rare: the row maximum grew by more than 2^8; rescale this thread's half
                        // of O in tensor memory (its partner takes the same decision from the same
                        // values), then fetch the scores again.
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

                // Probabilities as bf16 over the first 32 of this thread's S columns (all 64
                // scores are already in registers), row-sum share in fp32.
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
#ifdef ARC_PREFILL_TRACE
                    if (tr) p.trace[i * 16 + 10] = clock64();
#endif
                    chunk_exp_any<false>(vb, pk, ls4, sl, m_eff, kc + 32, rm);
                    tmem_st16(tS + 16, pk);
                }
                l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
#ifdef ARC_PREFILL_TRACE
                if (tr) p.trace[i * 16 + 3] = clock64();
#endif
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&p_full[x]);
#ifdef ARC_PREFILL_TRACE
                if (tr) p.trace[i * 16 + 4] = clock64();
#endif
            }

            // Row sum = both halves' shares.
            xch_sum[half * 128 + r] = l;
            pair_sync(pair_id);
            l += xch_sum[(half ^ 1) * 128 + r];
            if (ok && !mbar_wait_warp(&o_full[x], 0)) {
                report_fault(p.fault, FAULT_WAIT_O, 0);
                ok = false;
            }
            tc_fence_after_sync();
            if (ok) {
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                const float lse = l > 0.f ? (m + fast_log2(l)) * 0.6931471805599453f : -CUDART_INF_F;
                const long long row = ((long long)b * p.seq + t) * p.nq + g.head;
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
                    const long long eoff = b * p.o_stride_b + t * p.o_stride_t + (long long)g.head * HD + half * OC;
                    uint16_t* dst = p.out + eoff;
                    const uint16_t* gp = p.gate ? p.gate + eoff : nullptr;
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
                                if (gp) {
                                    const uint4 gv = *reinterpret_cast<const uint4*>(gp + c * 32 + e);
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
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == PRODUCER_WARP) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace arc
