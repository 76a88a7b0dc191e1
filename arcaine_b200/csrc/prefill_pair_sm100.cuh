// GQA flash-attention prefill kernel for sm_100a, head dim 128: two query tiles per CTA.
//
// A CTA owns 256 query tokens of one query head as two 128-row tiles, A and B, that walk the
// same key blocks.  Each tile is a pipeline of its own: four softmax warps (one query row per
// thread, TMEM lane = row, so row maxima and sums never leave the thread), one MMA-issuing
// thread, one score buffer S and one accumulator O in tensor memory (S_A S_B O_A O_B = 512
// columns), one Q buffer in shared memory.  The two pipelines share the K and V rings, which
// one producer thread fills by TMA, so every key block is fetched once for 256 rows.
//
// Sixteen warps in four groups with register budgets of their own (setmaxnreg):
//   warps 0-3 / 4-7   softmax of tile A / B: a thread takes its row's 128 scores out of tensor
//                     memory ONCE, masks them in registers where the block needs it, takes the
//                     maximum, exponentiates and writes P (bf16) back over the scores;
//   warps 8-11        epilogue: once a tile's last O += P V has landed they read the accumulator
//                     out, normalise, gate and store it, while the softmax warps are already
//                     working on the next tile's first key block;
//   warps 12-15       TMA producer of K / V, MMA issuer of A, MMA issuer of B, TMA producer of Q
//                     (one thread each).
//
// The pipelines run out of phase: while the softmax warps of A turn S_A(j) into P_A(j), the
// tensor pipe works for B (O_B += P_B V, S_B = Q_B K^T), and the other way round.  Left alone
// they fall into step (both wait for the tensor pipe, then both fight for the ex2 unit), so the
// phase is enforced: the softmax warps take turns at the exponentials, block by block, through
// a pair of mbarriers.  Per block and pipeline the issuer does
//   wait P(j);  O += P(j) V(j);  S(j+1) = Q K(j+1)^T     (P V in two halves of 64 keys, the first
//   one as soon as its probabilities are written)
// — P is written over S, so the next scores can only follow the P V that reads them, and both
// come from one thread, in order.
//
// Lazy rescaling, probabilities as bf16 over the score columns, bounded waits and the device
// status word are as in the single-tile kernel (prefill_sm100.cuh), which keeps head dim 256,
// additive masks and key-range splits.
#pragma once
#include "prefill_sm100.cuh"

namespace arc {

struct PairCfg {
    static constexpr int HD = 128;
    static constexpr int BM = 128;   // rows per tile; a CTA works on two
    static constexpr int BN = 128;   // keys per block
    static constexpr int CH = HD / 64;
    static constexpr int CHUNK_BYTES = 128 * 128;
    static constexpr int TILE_BYTES = CH * CHUNK_BYTES;
    static constexpr int K_STAGES = 2;
    static constexpr int V_STAGES = 2;
    static constexpr int TMEM_COLS = 512;
    static constexpr int COL_S = 0;    // + 128 * pipeline
    static constexpr int COL_O = 256;  // + 128 * pipeline
    // q_full[2] q_empty[2] k_full[KS] k_empty[KS] v_full[VS] v_empty[VS] then per pipeline:
    // s_full p_half[2] o_full o_empty turn fin[2]
    static constexpr int NUM_BARS = 4 + 2 * K_STAGES + 2 * V_STAGES + 16;
    static constexpr int FIN_FLOATS = 2 * 2 * 128 * 2;  // [tile parity][pipeline][row] (row sum, row maximum)
    static constexpr int SMEM_BYTES = (2 + K_STAGES + V_STAGES) * TILE_BYTES + NUM_BARS * 8 + 16 + FIN_FLOATS * 4 + 1024;
    static constexpr int SOFTMAX_WARPS = 8;   // four per pipeline
    static constexpr int EPILOGUE_WARP = 8;   // four warps
    static constexpr int PRODUCER_WARP = 12;
    static constexpr int ISSUER_WARP = 13;    // + pipeline
    static constexpr int Q_PRODUCER_WARP = 15;
    static constexpr int THREADS = 32 * 16;
    // The budgets may only redistribute what the CTA holds at launch (threads x the per-thread
    // count the launch bound gives, 128 for 512 threads): a group that asks for more waits for ever.
    static constexpr int REGS_SOFTMAX = 192;
    static constexpr int REGS_EPILOGUE = 80;
    static constexpr int REGS_CONTROL = 48;
    static constexpr int LAUNCH_REGS = (65536 / THREADS) & ~7;
    static_assert((SOFTMAX_WARPS * REGS_SOFTMAX + 4 * REGS_EPILOGUE + 4 * REGS_CONTROL) * 32 <= THREADS * LAUNCH_REGS,
                  "register budgets exceed what the CTA holds at launch");
};

// One unit of work: two 128-row tiles, and per tile the key blocks [lo, hi) it can see.  With an
// even number of query heads per KV head the tiles are the same 128 tokens of two heads of one KV
// group: both walk exactly the same key blocks, so neither pipeline ever idles while the other
// works on a block only it can see.  Otherwise they are 256 consecutive tokens of one head.
struct PairWork {
    int q0[2], h[2];
    int b, kvh;
    int lo[2], hi[2];
    int ulo, uhi;  // union of the two ranges (contiguous)
    bool live[2];  // the tile has rows below seq
    // Selected without dynamic indexing, so the struct stays in registers.
    __device__ __forceinline__ int q0_of(int s) const { return s ? q0[1] : q0[0]; }
    __device__ __forceinline__ int h_of(int s) const { return s ? h[1] : h[0]; }
    __device__ __forceinline__ int lo_of(int s) const { return s ? lo[1] : lo[0]; }
    __device__ __forceinline__ int hi_of(int s) const { return s ? hi[1] : hi[0]; }
    __device__ __forceinline__ bool live_of(int s) const { return s ? live[1] : live[0]; }
};

// Key blocks [lo, hi) a 128-row tile starting at token qs can see.
__device__ __forceinline__ void tile_blocks(const PrefillParams& p, int qs, int& blk_lo, int& blk_hi) {
    const int off = p.kv_len - p.seq;
    blk_lo = 0;
    blk_hi = (p.kv_len + PairCfg::BN - 1) / PairCfg::BN;
    if (p.mask_type == 3) {
        const int q_last = min(qs + PairCfg::BM - 1, p.seq - 1);
        const int last_key = min(p.kv_len - 1, q_last + off);
        blk_hi = last_key >= 0 ? last_key / PairCfg::BN + 1 : 0;
        if (p.window > 0 && p.window != 0x7fffffff) blk_lo = max(0, qs + off - p.window + 1) / PairCfg::BN;
    }
    if (blk_hi < blk_lo) blk_hi = blk_lo;
}

// Every role runs this once per unit, from code that has long left the instruction caches by
// then, so it is kept short: one division at most, and nothing computed twice.
__device__ __forceinline__ PairWork decode_pair(const PrefillParams& p, const TileCursor& cur) {
    PairWork t;
    t.b = cur.z;
    if (p.head_pair) {
        t.h[0] = cur.h * 2;
        t.h[1] = t.h[0] + 1;
        t.q0[0] = t.q0[1] = cur.qt * PairCfg::BM;
        t.kvh = p.group_shift >= 0 ? (t.h[0] >> p.group_shift) : t.h[0] / p.group;
        t.live[0] = t.live[1] = true;  // the tile list only holds tiles with rows
        tile_blocks(p, t.q0[0], t.lo[0], t.hi[0]);
        t.lo[1] = t.ulo = t.lo[0];
        t.hi[1] = t.uhi = t.hi[0];
    } else {
        t.h[0] = t.h[1] = cur.h;
        t.q0[0] = cur.qt * 2 * PairCfg::BM;
        t.q0[1] = t.q0[0] + PairCfg::BM;
        t.kvh = p.group_shift >= 0 ? (cur.h >> p.group_shift) : cur.h / p.group;
        t.live[0] = true;
        t.live[1] = t.q0[1] < p.seq;
        tile_blocks(p, t.q0[0], t.lo[0], t.hi[0]);
        t.lo[1] = t.hi[1] = 0;
        if (t.live[1]) tile_blocks(p, t.q0[1], t.lo[1], t.hi[1]);
        t.ulo = 0x7fffffff;
        t.uhi = 0;
#pragma unroll
        for (int s = 0; s < 2; ++s)
            if (t.hi[s] > t.lo[s]) {
                t.ulo = min(t.ulo, t.lo[s]);
                t.uhi = max(t.uhi, t.hi[s]);
            }
    }
    if (t.uhi == 0) t.ulo = 0;
    return t;
}

// Scores of keys outside the row's visible span [lo, hi) become -inf, in registers.
__device__ __forceinline__ void mask_chunk(uint32_t (&v)[32], int key0, const RowMask& rm) {
    const uint32_t lo_rel = static_cast<uint32_t>(rm.lo - key0), span = static_cast<uint32_t>(rm.hi - rm.lo);
#pragma unroll
    for (int e = 0; e < 32; ++e) v[e] = (static_cast<uint32_t>(e) - lo_rel < span) ? v[e] : 0xff800000u;  // lo <= key < hi
}

// The gated epilogue and the one that also stores copies of the output are instances of their own: code the
// common kernel does not carry.
template <bool GATE, bool COPIES>
__global__ void __launch_bounds__(PairCfg::THREADS, 1)
    sdpa_prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                             const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    using C = PairCfg;
    constexpr int HD = C::HD;
    constexpr int KS = C::K_STAGES;
    constexpr int VS = C::V_STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                       // [2] one per pipeline
    uint8_t* sK = smem + 2 * C::TILE_BYTES;   // [KS]
    uint8_t* sV = sK + KS * C::TILE_BYTES;    // [VS]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + VS * C::TILE_BYTES);
    uint64_t* q_full = bars;         // [2]
    uint64_t* q_empty = bars + 2;    // [2] the tile's last S = Q K^T has completed
    uint64_t* k_full = bars + 4;     // [KS]
    uint64_t* k_empty = k_full + KS; // [KS] two arrivals: one per issuer
    uint64_t* v_full = k_empty + KS;
    uint64_t* v_empty = v_full + VS; // [VS] two arrivals
    uint64_t* s_full = v_empty + VS; // [2] per pipeline from here on
    uint64_t* p_half = s_full + 2;   // [pipeline][half]: P of keys 0-63 / 64-127 of the block is in tensor memory
    uint64_t* o_full = p_half + 4;   // one phase per tile: the tile's last O += P V has completed
    uint64_t* o_empty = o_full + 2;  // one phase per tile: the epilogue warps have read O out
    uint64_t* turn = o_empty + 2;    // one phase per union key block: the pipeline's softmax warps are past it
    // fin[2 * s + (tile & 1)], one phase per second tile: the softmax warps have published the tile's row sums
    // and maxima.  Two barriers per pipeline, used in turn, because a tile of one key block needs no
    // O += P V to finish: with one barrier the softmax warps could complete it for tile n + 1 while a slow
    // epilogue (stores held up) still waits for tile n's completion — and a parity wait cannot tell "twice"
    // from "not yet".  They cannot reach tile n + 2 before the epilogue has taken tile n (the first O += P V
    // of tile n + 1 waits for that), so two are enough.
    uint64_t* fin = turn + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NUM_BARS);
    uint32_t* abort_slot = tmem_slot + 1;
    float2* fin_vals = reinterpret_cast<float2*>(tmem_slot + 4);  // [tile parity 2][pipeline 2][row 128] (row sum, row maximum)

    grid_launch_dependents();  // a launch behind this one (the single-head tail of the unit list) may be scheduled as SMs free up
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // After an L2 flush the status word, the three descriptors and the first tiles are an HBM round trip each:
    // the descriptors and the status word are requested at once, and the barriers are set up while they travel.
    if (threadIdx.x == 32) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    if (threadIdx.x == 0) {
        const uint32_t fault_word = *reinterpret_cast<volatile uint32_t*>(p.fault);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&q_full[s], 1);
            mbar_init(&q_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_half[2 * s], 128);
            mbar_init(&p_half[2 * s + 1], 128);
            mbar_init(&o_full[s], 1);
            mbar_init(&o_empty[s], 128);
            mbar_init(&turn[s], 128);
            mbar_init(&fin[2 * s], 128);
            mbar_init(&fin[2 * s + 1], 128);
        }
        for (int s = 0; s < KS; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 2);
        }
        for (int s = 0; s < VS; ++s) {
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 2);
        }
        fence_mbar_init();
        *abort_slot = fault_word != 0u ? 1u : 0u;
    }
    __syncthreads();
    if (*abort_slot) return;
    if (warp == C::PRODUCER_WARP) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp >= C::PRODUCER_WARP) {
        reg_dealloc<C::REGS_CONTROL>();
        if (warp == C::PRODUCER_WARP) {
            // -------------------------------------------------------------- TMA producer of K and V
            if (lane == 0) {
                prefetch_tensormap(&tm_k);
                prefetch_tensormap(&tm_v);
                int gk = 0, gv = 0;        // key blocks loaded into each ring so far
                bool ok = true;
                TileCursor cur;
                for (cur.init(p); ok && cur.w < p.total_tiles; cur.advance(p)) {
                    const PairWork pw = decode_pair(p, cur);
                    // K stays at most two blocks ahead of V; both rings fill in the order of use.
                    const int n = pw.uhi - pw.ulo;
                    int uk = 0, uv = 0;
                    while (ok && (uk < n || uv < n)) {
                        if (uk < n && (uk <= uv + 1 || uv >= n)) {
                            const int st = gk % KS;
                            if (gk >= KS && !mbar_wait<1>(&k_empty[st], ((gk / KS) - 1) & 1)) {
                                report_fault(p.fault, FAULT_WAIT_EMPTY, 0x100u);
                                ok = false;
                                break;
                            }
                            mbar_arrive_expect_tx(&k_full[st], C::TILE_BYTES);
#pragma unroll
                            for (int c = 0; c < C::CH; ++c)
                                tma_load_4d(sK + st * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_k, &k_full[st], c * 64, pw.kvh,
                                            (pw.ulo + uk) * C::BN, pw.b);
                            ++uk;
                            ++gk;
                        } else {
                            const int st = gv % VS;
                            if (gv >= VS && !mbar_wait<1>(&v_empty[st], ((gv / VS) - 1) & 1)) {
                                report_fault(p.fault, FAULT_WAIT_EMPTY, 0x200u);
                                ok = false;
                                break;
                            }
                            mbar_arrive_expect_tx(&v_full[st], C::TILE_BYTES);
#pragma unroll
                            for (int c = 0; c < C::CH; ++c)
                                tma_load_4d(sV + st * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_v, &v_full[st], c * 64, pw.kvh,
                                            (pw.ulo + uv) * C::BN, pw.b);
                            ++uv;
                            ++gv;
                        }
                    }
                }
            }
        } else if (warp == C::Q_PRODUCER_WARP) {
            // -------------------------------------------------------------- TMA producer of Q
            // A thread of its own: the next unit's Q tiles are requested the moment the current tiles'
            // last scores are out, whatever the K / V producer is waiting for at that time.
            if (lane == 0) {
                prefetch_tensormap(&tm_q);
                int tq0 = 0, tq1 = 0;  // tiles with key blocks loaded so far, per pipeline
                bool ok = true;
                TileCursor cur;
                for (cur.init(p); ok && cur.w < p.total_tiles; cur.advance(p)) {
                    const PairWork pw = decode_pair(p, cur);
#pragma unroll
                    for (int s = 0; s < 2; ++s) {
                        if (pw.hi[s] == pw.lo[s]) continue;
                        int& tq = s ? tq1 : tq0;
                        if (tq > 0 && !mbar_wait<1>(&q_empty[s], (tq - 1) & 1)) {
                            report_fault(p.fault, FAULT_WAIT_EMPTY, 0x300u + s);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(&q_full[s], C::TILE_BYTES);
#pragma unroll
                        for (int c = 0; c < C::CH; ++c)
                            tma_load_4d(sQ + s * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_q, &q_full[s], c * 64, pw.h[s],
                                        pw.q0[s], pw.b);
                        ++tq;
                    }
                    // The unit after this one: its Q rows (one 256-byte piece per token, far apart in
                    // memory) are asked into L2 now, a whole unit ahead of the load that needs them.
                    TileCursor nx = cur;
                    nx.advance(p);
                    if (ok && nx.w < p.total_tiles) {
                        const PairWork pn = decode_pair(p, nx);
#pragma unroll
                        for (int s = 0; s < 2; ++s) {
                            if (pn.hi[s] == pn.lo[s]) continue;
#pragma unroll
                            for (int c = 0; c < C::CH; ++c) tma_prefetch_4d(&tm_q, c * 64, pn.h[s], pn.q0[s], pn.b);
                        }
                    }
                }
            }
        } else if (warp <= C::ISSUER_WARP + 1) {
            // -------------------------------------------------------------- MMA issuer of one pipeline
            if (lane == 0) {
                const int s = warp - C::ISSUER_WARP;
                constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, false);
                constexpr uint32_t IDESC_PV = make_idesc_bf16(128, HD, true);
                const uint32_t tS = tmem_base + C::COL_S + s * 128;
                const uint32_t tO = tmem_base + C::COL_O + s * 128;
                // Descriptors are built once; per MMA only the start-address field (bytes >> 4, in
                // the low word) moves, by a compile-time constant.
                const uint64_t dQ = make_smem_desc_sw128(smem_u32(sQ + s * C::TILE_BYTES), 16, 1024);
                const uint64_t dK = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
                const uint64_t dV = make_smem_desc_sw128(smem_u32(sV), C::CHUNK_BYTES, 1024);
                static_assert(KS == 2 && VS == 2 && HD == 128, "ring arithmetic assumes two stages and head dim 128");
                int gu = 0;  // union key blocks passed so far (ring position, same in both issuers)
                int g = 0;   // key blocks of this pipeline issued so far
                int tq = 0;  // tiles of this pipeline with key blocks so far
                bool ok = true;
                // S = Q K(j)^T for ring position r; releases the K stage.  For a block this pipeline does
                // not use, only the release (once the stage has been filled, so arrivals stay in step).
                auto scores = [&](int r, bool active, bool last) -> bool {
                    if (!mbar_wait<1>(&k_full[r % KS], (r / KS) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_K, r);
                        return false;
                    }
                    if (!active) {
                        mbar_arrive(&k_empty[r % KS]);
                        return true;
                    }
                    tc_fence_after_sync();
                    const uint64_t dKs = dK + (uint64_t)((r & 1) * (C::TILE_BYTES >> 4));
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint32_t o = ((kk >> 2) * C::CHUNK_BYTES + (kk & 3) * 32) >> 4;  // 16 head-dim columns
                        umma_ss(tS, dQ + o, dKs + o, IDESC_QK, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(&s_full[s]);
                    umma_commit(&k_empty[r % KS]);
                    if (last) umma_commit(&q_empty[s]);
                    return true;
                };
                TileCursor cur;
                for (cur.init(p); ok && cur.w < p.total_tiles; cur.advance(p)) {
                    const PairWork pw = decode_pair(p, cur);
                    const int lo = pw.lo_of(s), hi = pw.hi_of(s);
                    if (pw.uhi == pw.ulo) continue;
                    if (hi > lo && !mbar_wait<1>(&q_full[s], tq & 1)) {
                        report_fault(p.fault, FAULT_WAIT_Q, tq);
                        break;
                    }
                    // Position j: O += P(j) V(j), then S(j+1).  The loop starts one position early, so that
                    // the tile's first scores come out of the same (single) place in the code.
                    for (int j = pw.ulo - 1; ok && j < pw.uhi; ++j) {
                        const bool act = j >= lo && j < hi;
                        if (j >= pw.ulo && !mbar_wait<1>(&v_full[gu % VS], (gu / VS) & 1)) {
                            report_fault(p.fault, FAULT_WAIT_V, gu);
                            ok = false;
                            break;
                        }
                        if (j < pw.ulo) {
                            // nothing to accumulate yet
                        } else if (act) {
                            if (!mbar_wait<1>(&p_half[2 * s], g & 1)) {
                                report_fault(p.fault, FAULT_WAIT_P, g);
                                ok = false;
                                break;
                            }
                            if (j == lo && tq > 0 && !mbar_wait<1>(&o_empty[s], (tq - 1) & 1)) {
                                report_fault(p.fault, FAULT_WAIT_O, 0x100u + tq);
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            // P from tensor memory: each 32-key chunk keeps its 16 bf16x2 columns at the
                            // start of its own 32 score columns.  V is MN-major: 64-element head-dim
                            // chunks 16 KB apart, 8-key groups 1024 bytes apart; 16 keys = 2048 bytes.
                            // The first 64 keys go to the tensor pipe while the softmax warps are still
                            // exponentiating the other 64.
                            const uint64_t dVs = dV + (uint64_t)((gu & 1) * (C::TILE_BYTES >> 4));
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk)
                                umma_ts(tO, tS + (kk >> 1) * 32 + (kk & 1) * 8, dVs + (uint64_t)((kk * 2048) >> 4), IDESC_PV,
                                        (j > lo || kk > 0) ? 1u : 0u);
                            if (!mbar_wait<1>(&p_half[2 * s + 1], g & 1)) {
                                report_fault(p.fault, FAULT_WAIT_P, 0x1000u + g);
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
#pragma unroll
                            for (int kk = 4; kk < 8; ++kk)
                                umma_ts(tO, tS + (kk >> 1) * 32 + (kk & 1) * 8, dVs + (uint64_t)((kk * 2048) >> 4), IDESC_PV, 1u);
                            umma_commit(&v_empty[gu % VS]);
                            if (j + 1 == hi) umma_commit(&o_full[s]);
                            ++g;
                        } else {
                            mbar_arrive(&v_empty[gu % VS]);
                        }
                        if (j >= pw.ulo) ++gu;  // ring position of block j + 1 from here on
                        // S(j+1): over the P just consumed, behind the MMAs that read it
                        if (j + 1 < pw.uhi) {
                            const bool act1 = j + 1 >= lo && j + 1 < hi;
                            ok = scores(gu, act1, act1 && j + 2 == hi);
                        }
                    }
                    if (hi > lo) ++tq;
                }
            }
        }
    } else if (warp >= C::EPILOGUE_WARP) {
        // ------------------------------------------------------------------ epilogue
        // Thread = query row (TMEM lane); tiles A and B of every unit in turn.  The accumulator is
        // released as soon as it is in registers, normally before the next tile's first P is ready.
        reg_dealloc<C::REGS_EPILOGUE>();
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
        int tq0 = 0, tq1 = 0;  // tiles with key blocks so far, per pipeline
        bool ok = true;
        uint32_t wa[32];
        TileCursor cur;
        for (cur.init(p); ok && cur.w < p.total_tiles; cur.advance(p)) {
            const PairWork pw = decode_pair(p, cur);
#pragma unroll 1
            for (int s = 0; s < 2 && ok; ++s) {
                const int t = pw.q0_of(s) + r;
                const bool store = pw.live_of(s) && t < p.seq;
                const long long row = ((long long)pw.b * p.seq + t) * p.nq + pw.h_of(s);
                const long long eoff = pw.b * p.o_stride_b + t * p.o_stride_t + (long long)pw.h_of(s) * HD;
                if (pw.hi_of(s) == pw.lo_of(s)) {
                    // Nothing visible for this tile: zero output.
                    if (store) {
                        for (int c = -1; c < (COPIES ? p.n_copies : 0); ++c) {
                            uint4* dst = reinterpret_cast<uint4*>((c < 0 ? p.out : reinterpret_cast<uint16_t*>(p.out_copies[c])) + eoff);
                            for (int i = 0; i < HD / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                        }
                        if (p.out_lse) p.out_lse[row] = -CUDART_INF_F;
                    }
                    continue;
                }
                const int tq = s ? tq1 : tq0;
                if (!mbar_wait_relaxed_warp<2>(&fin[2 * s + (tq & 1)], (tq >> 1) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_FULL, 0x500u + s);
                    ok = false;
                    break;
                }
                const float2 fv = fin_vals[((tq & 1) * 2 + s) * 128 + r];
                const float row_l = fv.x, row_m = fv.y;
                if (!mbar_wait_relaxed_warp<2>(&o_full[s], tq & 1)) {
                    report_fault(p.fault, FAULT_WAIT_O, tq);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                if (s) ++tq1; else ++tq0;
                const float inv = row_l > 0.f ? 1.0f / row_l : 0.f;
                const uint32_t tO = tmem_base + lane_sel + C::COL_O + s * 128;
                uint16_t* dst = p.out + eoff;
                const uint16_t* gp = GATE ? p.gate + eoff : nullptr;
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    tmem_ld32(tO + c * 32, wa);
                    tmem_wait_ld();
                    if (c + 1 == HD / 32) {
                        // O is in registers: the next tile may overwrite the accumulator.
                        tc_fence_before_sync();
                        mbar_arrive(&o_empty[s]);
                    }
                    if (store) {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {  // 16 values = 32 bytes per round
                            uint32_t w8[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                w8[u] = pack_bf16x2(__uint_as_float(wa[i * 16 + 2 * u]) * inv, __uint_as_float(wa[i * 16 + 2 * u + 1]) * inv);
                            if (GATE) {
                                // bf16(attention) * sigmoid(gate): the rounding order of the two-launch form
                                const uint4 g0 = *reinterpret_cast<const uint4*>(gp + c * 32 + i * 16);
                                const uint4 g1 = *reinterpret_cast<const uint4*>(gp + c * 32 + i * 16 + 8);
                                const uint32_t gw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                                for (int u = 0; u < 8; ++u) {
                                    const float a0 = __uint_as_float(w8[u] << 16), a1 = __uint_as_float(w8[u] & 0xffff0000u);
                                    const float g0f = __uint_as_float(gw[u] << 16), g1f = __uint_as_float(gw[u] & 0xffff0000u);
                                    w8[u] = pack_bf16x2(a0 * (1.0f / (1.0f + __expf(-g0f))), a1 * (1.0f / (1.0f + __expf(-g1f))));
                                }
                            }
                            store_bf16x16(dst + c * 32 + i * 16, w8);
                            if (COPIES) store_copies_bf16x16(p.out_copies, p.n_copies, eoff + c * 32 + i * 16, w8);
                        }
                    }
                }
                if (store && p.out_lse)
                    p.out_lse[row] = row_l > 0.f ? (row_m + fast_log2(row_l)) * 0.6931471805599453f : -CUDART_INF_F;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax
        // Warps 0-3 serve tile A, warps 4-7 tile B; a thread owns one query row and takes its 128
        // scores of a block out of tensor memory once.
        reg_alloc<C::REGS_SOFTMAX>();
        const int s = warp >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t tS = tmem_base + lane_sel + C::COL_S + s * 128;
        const uint32_t tO = tmem_base + lane_sel + C::COL_O + s * 128;
        const float sl = p.scale_log2;
        const bool causal = (p.mask_type == 3);
        const bool windowed = causal && p.window > 0 && p.window != 0x7fffffff;
        const int off = p.kv_len - p.seq;

        int g = 0, tq = 0;  // key blocks and tiles (with key blocks) of this pipeline so far
        int gu = 0;         // union key blocks of the CTA so far (the same count in both pipelines)
        bool ok = true;
        uint32_t s0[32], s1[32], s2[32], s3[32];  // the row's 128 scores of the current block

        TileCursor cur;
        for (cur.init(p); ok && cur.w < p.total_tiles; cur.advance(p)) {
            const PairWork pw = decode_pair(p, cur);
            if (pw.uhi == pw.ulo) continue;
            const int t = pw.q0_of(s) + r;
            const int lo = pw.lo_of(s), hi = pw.hi_of(s);
            int row_lo = 0, row_hi = p.kv_len;  // visible keys [row_lo, row_hi)
            if (causal) {
                const int diag = t + off;
                row_hi = min(max(diag + 1, 0), p.kv_len);
                if (windowed) row_lo = max(0, diag - p.window + 1);
                if (row_lo > row_hi) row_lo = row_hi;
            }
            const RowMask rm{row_lo, row_hi, p.kv_len, nullptr};

            float m = -CUDART_INF_F;  // running max, log2 domain, possibly stale by <= 8
            float l = 0.f;            // row sum
            // Both pipelines walk every key block of the pair, used or not, and take turns at the
            // exponentials: A's block u goes after B's block u - 1, B's block u after A's block u.
            // That keeps the pipelines half a period apart, so that one computes while the tensor
            // pipe works for the other.
            for (int j = pw.ulo; j < pw.uhi; ++j, ++gu) {
                const bool act = j >= lo && j < hi;
                const int kc = j * C::BN;
                float m_eff = 0.f;
                // 32-key chunks no row of the warp can see (bit c set) are neither reduced nor exponentiated
                uint32_t none = 0u;
                if (act) {
                    if (!mbar_wait_warp<3>(&s_full[s], g & 1)) {
                        report_fault(p.fault, FAULT_WAIT_S, g);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    // Every key of the block visible to every row of the warp (seven blocks in nine
                    // with a 1024-key window): no element tests at all.
                    const bool full = __all_sync(0xffffffffu, rm.lo <= kc && kc + C::BN <= rm.hi);
                    for (;;) {
                        tmem_ld32(tS, s0);
                        tmem_ld32(tS + 32, s1);
                        tmem_ld32(tS + 64, s2);
                        tmem_ld32(tS + 96, s3);
                        tmem_wait_ld();
                        float mr[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                        if (full) {
                            chunk_max<0>(s0, mr, sl, kc, rm);
                            chunk_max<0>(s1, mr, sl, kc, rm);
                            chunk_max<0>(s2, mr, sl, kc, rm);
                            chunk_max<0>(s3, mr, sl, kc, rm);
                        } else {
                            // window edge, diagonal, ragged end: per chunk either whole, mixed (scores of
                            // keys outside the row's span become -inf in registers) or out of sight
                            none = 0u;
                            int cls = chunk_class(kc, rm);
                            if (cls == 1) mask_chunk(s0, kc, rm);
                            if (cls == 2) none |= 1u; else chunk_max<0>(s0, mr, sl, kc, rm);
                            cls = chunk_class(kc + 32, rm);
                            if (cls == 1) mask_chunk(s1, kc + 32, rm);
                            if (cls == 2) none |= 2u; else chunk_max<0>(s1, mr, sl, kc, rm);
                            cls = chunk_class(kc + 64, rm);
                            if (cls == 1) mask_chunk(s2, kc + 64, rm);
                            if (cls == 2) none |= 4u; else chunk_max<0>(s2, mr, sl, kc, rm);
                            cls = chunk_class(kc + 96, rm);
                            if (cls == 1) mask_chunk(s3, kc + 96, rm);
                            if (cls == 2) none |= 8u; else chunk_max<0>(s3, mr, sl, kc, rm);
                        }
                        const float m_new = fmaxf(m, fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * sl);
                        if (j == lo) {
                            m = m_new;
                            break;
                        }
                        const bool need = m_new > m + 8.0f;
                        if (!__any_sync(0xffffffffu, need)) break;
                        // Rare: some row's maximum grows by more than 2^8.  O += P V of the previous block
                        // has landed (these scores were issued behind it): rescale those rows of O in
                        // tensor memory, then take the scores again (their registers were the scratch).
                        const float alpha = need ? fast_exp2(m - m_new) : 1.0f;
#pragma unroll 1
                        for (int c = 0; c < HD / 32; ++c) {
                            tmem_ld32(tO + c * 32, s0);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 32; ++e) s0[e] = __float_as_uint(__uint_as_float(s0[e]) * alpha);
                            tmem_st32(tO + c * 32, s0);
                        }
                        tmem_wait_st();
                        l *= alpha;
                        if (need) m = m_new;
                    }
                    m_eff = (m == -CUDART_INF_F) ? 0.f : m;
                }
                // my turn?
                {
                    uint64_t* other = &turn[s ^ 1];
                    const bool must = (s == 1) || gu > 0;
                    const uint32_t parity = (uint32_t)((s == 1) ? gu : gu - 1) & 1u;
                    if (must && !mbar_wait_warp<3>(other, parity)) {
                        report_fault(p.fault, FAULT_WAIT_FULL, 0x400u + s);
                        ok = false;
                        break;
                    }
                }
                if (act) {
                    // Probabilities as bf16, each 32-key chunk over the first 16 of its own 32 score
                    // columns; row sum in fp32.
                    float ls4[4] = {0.f, 0.f, 0.f, 0.f};
                    uint32_t pk[16];
                    auto zero_pk = [&]() {
#pragma unroll
                        for (int e = 0; e < 16; ++e) pk[e] = 0u;
                    };
                    if (none & 1u) zero_pk(); else chunk_exp<0>(s0, pk, ls4, sl, m_eff, kc, rm);
                    tmem_st16(tS, pk);
                    if (none & 2u) zero_pk(); else chunk_exp<0>(s1, pk, ls4, sl, m_eff, kc, rm);
                    tmem_st16(tS + 32, pk);
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(&p_half[2 * s]);  // keys 0-63: their share of O += P V may start
                    if (none & 4u) zero_pk(); else chunk_exp<0>(s2, pk, ls4, sl, m_eff, kc, rm);
                    tmem_st16(tS + 64, pk);
                    if (none & 8u) zero_pk(); else chunk_exp<0>(s3, pk, ls4, sl, m_eff, kc, rm);
                    tmem_st16(tS + 96, pk);
                    l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(&p_half[2 * s + 1]);
                    ++g;
                }
                mbar_arrive(&turn[s]);
                if (act && j + 1 == hi) {
                    // The tile's last key block is on its way: hand the row sum and maximum to the
                    // epilogue warps and go on with the next tile.
                    fin_vals[((tq & 1) * 2 + s) * 128 + r] = make_float2(l, m);
                    mbar_arrive(&fin[2 * s + (tq & 1)]);
                    ++tq;
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == C::PRODUCER_WARP) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace arc
