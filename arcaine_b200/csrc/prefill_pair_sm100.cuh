// GQA flash-attention prefill kernel for sm_100a, head dim 128: two query tiles per CTA.
//
// A CTA owns 256 query tokens of one query head as two 128-row tiles, A and B, that walk the
// same key blocks.  Each tile is a pipeline of its own: four softmax warps (one query row per
// thread, TMEM lane = row, so row maxima and sums never leave the thread), one MMA-issuing
// thread, one score buffer S and one accumulator O in tensor memory (S_A S_B O_A O_B = 512
// columns), one Q buffer in shared memory.  The two pipelines share the K and V rings, which
// one producer thread fills by TMA, so every key block is fetched once for 256 rows.
//
// The pipelines run out of phase: while the softmax warps of A turn S_A(j) into P_A(j), the
// tensor pipe works for B (O_B += P_B V, S_B = Q_B K^T), and the other way round.  Left alone
// they fall into step (both wait for the tensor pipe, then both fight for the ex2 unit), so the
// phase is enforced: the softmax warps take turns at the exponentials, block by block, through
// a pair of mbarriers.  Per block
// and pipeline the issuer does   wait P(j);  O += P(j) V(j);  S(j+1) = Q K(j+1)^T   — P is
// written over S, so the next scores can only follow the P V that reads them, and both come
// from one thread, in order.  The two issuers sit on different instruction schedulers.
//
// Masking, lazy rescaling, probabilities as bf16 over the score columns, bounded waits and
// the device status word are as in the single-tile kernel (prefill_sm100.cuh), which keeps
// head dim 256, additive masks and key-range splits.
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
    // s_full p_full pv_done o_full o_empty turn
    static constexpr int NUM_BARS = 4 + 2 * K_STAGES + 2 * V_STAGES + 12;
    static constexpr int SMEM_BYTES = (2 + K_STAGES + V_STAGES) * TILE_BYTES + NUM_BARS * 8 + 16 + 1024;
    static constexpr int SOFTMAX_WARPS = 8;  // four per pipeline
    static constexpr int PRODUCER_WARP = 8;
    static constexpr int ISSUER_WARP = 9;    // + pipeline
    static constexpr int THREADS = 32 * 11;
    static constexpr int MAX_REGS = 168;     // 65536 registers over 12 allocated warps
};

// One unit of work: 256 query tokens of one head; per tile the key blocks [lo, hi) it can see.
struct PairWork {
    int q0, h, b, kvh;
    int lo[2], hi[2];
    int ulo, uhi;  // union of the two ranges (contiguous)
    bool live[2];  // the tile has rows below seq
    // Selected without dynamic indexing, so the struct stays in registers.
    __device__ __forceinline__ int lo_of(int s) const { return s ? lo[1] : lo[0]; }
    __device__ __forceinline__ int hi_of(int s) const { return s ? hi[1] : hi[0]; }
    __device__ __forceinline__ bool live_of(int s) const { return s ? live[1] : live[0]; }
};

__device__ __forceinline__ PairWork decode_pair(const PrefillParams& p, const TileCursor& cur) {
    PairWork t;
    t.h = cur.h;
    t.b = cur.z;
    t.kvh = t.h / (p.nq / p.nkv);
    t.q0 = cur.qt * 2 * PairCfg::BM;
    const int off = p.kv_len - p.seq;
    const bool causal = (p.mask_type == 3);
    const bool windowed = causal && p.window > 0 && p.window != 0x7fffffff;
    t.ulo = 0x7fffffff;
    t.uhi = 0;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const int qs = t.q0 + s * PairCfg::BM;
        t.live[s] = qs < p.seq;
        int blk_lo = 0, blk_hi = 0;
        if (t.live[s]) {
            blk_hi = (p.kv_len + PairCfg::BN - 1) / PairCfg::BN;
            if (causal) {
                const int q_last = min(qs + PairCfg::BM - 1, p.seq - 1);
                const int last_key = min(p.kv_len - 1, q_last + off);
                blk_hi = last_key >= 0 ? last_key / PairCfg::BN + 1 : 0;
                if (windowed) blk_lo = max(0, qs + off - p.window + 1) / PairCfg::BN;
            }
            if (blk_hi < blk_lo) blk_hi = blk_lo;
        }
        t.lo[s] = blk_lo;
        t.hi[s] = blk_hi;
        if (blk_hi > blk_lo) {
            t.ulo = min(t.ulo, blk_lo);
            t.uhi = max(t.uhi, blk_hi);
        }
    }
    if (t.uhi == 0) t.ulo = 0;
    return t;
}

template <bool GATE>  // the gated epilogue is an instance of its own: 13 KB of code the common kernel does not carry
__global__ void __maxnreg__(PairCfg::MAX_REGS)
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
    uint64_t* p_full = s_full + 2;
    uint64_t* pv_done = p_full + 2;  // one phase per key block: O += P V of that block has completed
    uint64_t* o_full = pv_done + 2;  // one phase per tile
    uint64_t* o_empty = o_full + 2;  // one phase per tile: the softmax warps have read O out
    uint64_t* turn = o_empty + 2;    // one phase per union key block: the pipeline's softmax warps are past it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NUM_BARS);
    uint32_t* abort_slot = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) *abort_slot = (*reinterpret_cast<volatile uint32_t*>(p.fault) != 0u) ? 1u : 0u;
    __syncthreads();
    if (*abort_slot) return;
#ifdef ARC_TRACE_CTAS
    const long long ck0 = clock64();
#endif

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&q_full[s], 1);
            mbar_init(&q_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 128);
            mbar_init(&pv_done[s], 1);
            mbar_init(&o_full[s], 1);
            mbar_init(&o_empty[s], 128);
            mbar_init(&turn[s], 128);
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
    }
    if (warp == C::PRODUCER_WARP) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == C::PRODUCER_WARP) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&tm_q);
            prefetch_tensormap(&tm_k);
            prefetch_tensormap(&tm_v);
            int gk = 0, gv = 0;        // key blocks loaded into each ring so far
            int tq[2] = {0, 0};        // tiles with key blocks loaded so far, per pipeline
            bool ok = true;
            TileCursor cur;
            for (cur.init(p); ok && cur.w < p.total_tiles; cur.advance(p)) {
                const PairWork pw = decode_pair(p, cur);
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    if (pw.hi[s] == pw.lo[s]) continue;
                    if (tq[s] > 0 && !mbar_wait(&q_empty[s], (tq[s] - 1) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_EMPTY, 0x300u + s);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&q_full[s], C::TILE_BYTES);
#pragma unroll
                    for (int c = 0; c < C::CH; ++c)
                        tma_load_4d(sQ + s * C::TILE_BYTES + c * C::CHUNK_BYTES, &tm_q, &q_full[s], c * 64, pw.h,
                                    pw.q0 + s * C::BM, pw.b);
                    ++tq[s];
                }
                // K stays at most two blocks ahead of V; both rings fill in the order of use.
                const int n = pw.uhi - pw.ulo;
                int uk = 0, uv = 0;
                while (ok && (uk < n || uv < n)) {
                    if (uk < n && (uk <= uv + 1 || uv >= n)) {
                        const int st = gk % KS;
                        if (gk >= KS && !mbar_wait(&k_empty[st], ((gk / KS) - 1) & 1)) {
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
                        if (gv >= VS && !mbar_wait(&v_empty[st], ((gv / VS) - 1) & 1)) {
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
    } else if (warp == C::ISSUER_WARP || warp == C::ISSUER_WARP + 1) {
        // ------------------------------------------------------------------ MMA issuer of one pipeline
        if (lane == 0) {
            const int s = warp - C::ISSUER_WARP;
            constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, false);
            constexpr uint32_t IDESC_PV = make_idesc_bf16(128, HD, true);
            const uint32_t tS = tmem_base + C::COL_S + s * 128;
            const uint32_t tO = tmem_base + C::COL_O + s * 128;
            // Every operand descriptor the thread will ever need, built once (only the address
            // field, bytes >> 4 in the low word, differs): per MMA nothing is left to compute.
            const uint64_t dQ = make_smem_desc_sw128(smem_u32(sQ + s * C::TILE_BYTES), 16, 1024);
            const uint64_t dK = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t dV = make_smem_desc_sw128(smem_u32(sV), C::CHUNK_BYTES, 1024);
            uint64_t aQ[8], bK[8], bV[8];  // K and V: stage 0; the other stage is TILE_BYTES further
            uint32_t aP[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t o = ((kk >> 2) * C::CHUNK_BYTES + (kk & 3) * 32) >> 4;  // 16 head-dim columns
                aQ[kk] = dQ + o;
                bK[kk] = dK + o;
                // 16 keys of V: 8-key groups 1024 bytes apart; of P: 8 packed columns, each 32-key
                // chunk at the start of its own 32 score columns
                bV[kk] = dV + ((kk * 2048) >> 4);
                aP[kk] = tS + (kk >> 1) * 32 + (kk & 1) * 8;
            }
            static_assert(KS == 2 && VS == 2 && HD == 128, "descriptor tables assume two stages and head dim 128");
            int gu = 0;  // union key blocks passed so far (ring position, same in both issuers)
            int g = 0;   // key blocks of this pipeline issued so far
            int tq = 0;  // tiles of this pipeline with key blocks so far
            bool ok = true;
            // S = Q K(j)^T for ring position r; releases the K stage.  For a block this pipeline does
            // not use, only the release (once the stage has been filled, so arrivals stay in step).
            auto scores = [&](int r, bool active, bool last) -> bool {
                if (!mbar_wait(&k_full[r % KS], (r / KS) & 1)) {
                    report_fault(p.fault, FAULT_WAIT_K, r);
                    return false;
                }
                if (!active) {
                    mbar_arrive(&k_empty[r % KS]);
                    return true;
                }
                tc_fence_after_sync();
                {
                    uint64_t b[8];
                    const uint64_t stage = (uint64_t)((r & 1) * (C::TILE_BYTES >> 4));
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) b[kk] = bK[kk] + stage;
                    umma_ss_x8(tS, aQ, b, IDESC_QK, 0u);
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
                if (hi > lo && !mbar_wait(&q_full[s], tq & 1)) {
                    report_fault(p.fault, FAULT_WAIT_Q, tq);
                    break;
                }
                // Position j: O += P(j) V(j), then S(j+1).  The loop starts one position early, so that
                // the tile's first scores come out of the same (single) place in the code.
                for (int j = pw.ulo - 1; ok && j < pw.uhi; ++j) {
                    const bool act = j >= lo && j < hi;
                    if (j >= pw.ulo && !mbar_wait(&v_full[gu % VS], (gu / VS) & 1)) {
                        report_fault(p.fault, FAULT_WAIT_V, gu);
                        ok = false;
                        break;
                    }
                    if (j < pw.ulo) {
                        // nothing to accumulate yet
                    } else if (act) {
                        if (!mbar_wait(&p_full[s], g & 1)) {
                            report_fault(p.fault, FAULT_WAIT_P, g);
                            ok = false;
                            break;
                        }
                        if (j == lo && tq > 0 && !mbar_wait(&o_empty[s], (tq - 1) & 1)) {
                            report_fault(p.fault, FAULT_WAIT_O, 0x100u + tq);
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        // P from tensor memory: each 32-key chunk keeps its 16 bf16x2 columns at the
                        // start of its own 32 score columns.  V is MN-major: 64-element head-dim
                        // chunks 16 KB apart, 8-key groups 1024 bytes apart.
                        {
                            uint64_t b[8];
                            const uint64_t stage = (uint64_t)((gu & 1) * (C::TILE_BYTES >> 4));
#pragma unroll
                            for (int kk = 0; kk < 8; ++kk) b[kk] = bV[kk] + stage;
                            umma_ts_x8(tO, aP, b, IDESC_PV, j > lo ? 1u : 0u);
                        }
                        umma_commit(&v_empty[gu % VS]);
                        umma_commit(&pv_done[s]);
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
    } else {
        // ------------------------------------------------------------------ softmax / epilogue
        // Warps 0-3 serve tile A, warps 4-7 tile B; a thread owns one query row.
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
        uint32_t wa[32], wb[32];
#ifdef ARC_PREFILL_TRACE
        int tpos = 0;
#ifndef ARC_TR_THREAD
#define ARC_TR_THREAD 0
#endif
#ifndef ARC_TR_CTA
#define ARC_TR_CTA 0
#endif
#ifndef ARC_TR_MIN
#define ARC_TR_MIN 0
#endif
        const bool tr = p.trace && blockIdx.x == ARC_TR_CTA && threadIdx.x == ARC_TR_THREAD;
#ifndef ARC_TR_SKIP
#define ARC_TR_SKIP 0
#endif
#define ARC_TP(code) do { if (tr && tpos < 200 && (code) >= ARC_TR_MIN && tq >= ARC_TR_SKIP) { p.trace[2 * tpos] = (code); p.trace[2 * tpos + 1] = clock64(); ++tpos; } } while (0)
#else
#define ARC_TP(code) do { } while (0)
#endif

        TileCursor cur;
        for (cur.init(p); ok && cur.w < p.total_tiles; cur.advance(p)) {
            const PairWork pw = decode_pair(p, cur);
            if (pw.uhi == pw.ulo) {
                // No key block for either tile: zero output for the rows that exist.
                const int t = pw.q0 + s * C::BM + r;
                if (pw.live_of(s) && t < p.seq) {
                    const long long eoff = pw.b * p.o_stride_b + t * p.o_stride_t + (long long)pw.h * HD;
                    uint4* dst = reinterpret_cast<uint4*>(p.out + eoff);
                    for (int i = 0; i < HD / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                    if (p.out_lse) p.out_lse[((long long)pw.b * p.seq + t) * p.nq + pw.h] = -CUDART_INF_F;
                }
                continue;
            }
            const int t = pw.q0 + s * C::BM + r;
            const long long row = ((long long)pw.b * p.seq + t) * p.nq + pw.h;
            const long long eoff = pw.b * p.o_stride_b + t * p.o_stride_t + (long long)pw.h * HD;
            const bool store = pw.live_of(s) && t < p.seq;
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
            ARC_TP(1000 + hi - lo);
            // Both pipelines walk every key block of the pair, used or not, and take turns at the
            // exponentials (the two warps of a scheduler share one ex2 unit): A's block u goes after
            // B's block u - 1, B's block u after A's block u.  That keeps the pipelines half a
            // period apart, so that one computes while the tensor pipe works for the other.
            for (int j = pw.ulo; j < pw.uhi; ++j, ++gu) {
                const bool act = j >= lo && j < hi;
                const int kc = j * C::BN;
                bool full = false;
                float m_eff = 0.f;
                if (act) {
                    ARC_TP(10);
                    if (!mbar_wait_warp(&s_full[s], g & 1)) {
                        report_fault(p.fault, FAULT_WAIT_S, g);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    ARC_TP(11);
                    // Every key of the block visible to every row of the warp (seven blocks in nine
                    // with a 1024-key window): no per-element tests and no per-chunk votes.
                    full = __all_sync(0xffffffffu, rm.lo <= kc && kc + C::BN <= rm.hi);
                    // Pass 1: row maximum of the block, 64 keys per round.  The loops are kept rolled and
                    // the masked form has a single body: the kernel has to stay small enough for the
                    // instruction cache, and the masked blocks (window edge, diagonal) are the cold code.
                    float mr[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                    float ms[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                    if (full) {
                        // the hot path: the next chunk loads while one is reduced
                        tmem_ld32(tS, wa);
                        tmem_ld32(tS + 32, wb);
                        tmem_wait_ld();
                        chunk_max<0>(wa, mr, sl, kc, rm);
                        tmem_ld32(tS + 64, wa);
                        chunk_max<0>(wb, mr, sl, kc + 32, rm);
                        tmem_ld32(tS + 96, wb);
                        tmem_wait_ld();
                        chunk_max<0>(wa, mr, sl, kc + 64, rm);
                        tmem_ld32(tS, wa);  // first chunk again, for the exponentials
                        chunk_max<0>(wb, mr, sl, kc + 96, rm);
                    } else {
                        // cold path (window edge, diagonal): one 32-key chunk at a time through one body
#pragma unroll 1
                        for (int c = 0; c < 128; c += 32) {
                            if (chunk_class(kc + c, rm) == 2) continue;
                            tmem_ld32(tS + c, wb);
                            tmem_wait_ld();
                            chunk_max<1>(wb, ms, sl, kc + c, rm);
                        }
                        tmem_ld32(tS, wa);
                    }
                    const float bm = fmaxf(fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * sl,
                                           fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3])));
                    const float m_new = fmaxf(m, bm);
                    if (j == lo) {
                        m = m_new;
                    } else if (__any_sync(0xffffffffu, m_new > m + 8.0f)) {
                        // Rare: some row's maximum grows by more than 2^8.  Once O += P V of the previous
                        // block has landed, rescale those rows of O in tensor memory.
                        const bool need = m_new > m + 8.0f;
                        const float alpha = !need ? 1.0f : (m_new == -CUDART_INF_F ? 1.0f : fast_exp2(m - m_new));
                        tmem_wait_ld();
                        if (!mbar_wait_warp(&pv_done[s], (g - 1) & 1)) {
                            report_fault(p.fault, FAULT_WAIT_O, g);
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
#pragma unroll 1
                        for (int c = 0; c < HD / 32; ++c) {
                            tmem_ld32(tO + c * 32, wb);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 32; ++e) wb[e] = __float_as_uint(__uint_as_float(wb[e]) * alpha);
                            tmem_st32(tO + c * 32, wb);
                        }
                        tmem_wait_st();
                        l *= alpha;
                        if (need) m = m_new;
                        tmem_ld32(tS, wa);
                    }
                    m_eff = (m == -CUDART_INF_F) ? 0.f : m;
                    tmem_ld32(tS + 32, wb);
                    ARC_TP(12);
                }
                // my turn?
                {
                    uint64_t* other = &turn[s ^ 1];
                    const bool must = (s == 1) || gu > 0;
                    const uint32_t parity = (uint32_t)((s == 1) ? gu : gu - 1) & 1u;
                    if (must && !mbar_wait_warp(other, parity)) {
                        report_fault(p.fault, FAULT_WAIT_FULL, 0x400u + s);
                        ok = false;
                        break;
                    }
                }
                if (act) {
                    ARC_TP(14);
                    // Pass 2: probabilities as bf16, each 32-key chunk over the first 16 of its own 32
                    // score columns; row sum in fp32.  Rolled, 64 keys per round.
                    float ls4[4] = {0.f, 0.f, 0.f, 0.f};
                    uint32_t pk[16];
                    if (full) {
                        // unrolled on purpose: rolling these four saves 5 KB of code but costs 3 %
                        tmem_wait_ld();
                        chunk_exp<0>(wa, pk, ls4, sl, m_eff, kc, rm);
                        tmem_st16(tS, pk);
                        tmem_ld32(tS + 64, wa);
                        chunk_exp<0>(wb, pk, ls4, sl, m_eff, kc + 32, rm);
                        tmem_st16(tS + 32, pk);
                        tmem_ld32(tS + 96, wb);
                        tmem_wait_ld();
                        chunk_exp<0>(wa, pk, ls4, sl, m_eff, kc + 64, rm);
                        tmem_st16(tS + 64, pk);
                        chunk_exp<0>(wb, pk, ls4, sl, m_eff, kc + 96, rm);
                        tmem_st16(tS + 96, pk);
                    } else {
                        tmem_wait_ld();
#pragma unroll 1
                        for (int c = 0; c < 128; c += 32) {
                            if (chunk_class(kc + c, rm) == 2) {
#pragma unroll
                                for (int e = 0; e < 16; ++e) pk[e] = 0u;
                            } else {
                                tmem_ld32(tS + c, wb);
                                tmem_wait_ld();
                                chunk_exp<1>(wb, pk, ls4, sl, m_eff, kc + c, rm);
                            }
                            tmem_st16(tS + c, pk);
                        }
                    }
                    l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(&p_full[s]);
                    ++g;
                    ARC_TP(13);
                }
                mbar_arrive(&turn[s]);
                if (act && j + 1 == hi) {
                    // The tile's last key block is on its way: read the accumulator out now, before the
                    // turns for the blocks only the other tile still uses.
                    ARC_TP(20);

                    // Accumulator out: one thread writes the 256 contiguous bytes of its row.
                    if (!mbar_wait_warp(&o_full[s], tq & 1)) {
                        report_fault(p.fault, FAULT_WAIT_O, tq);
                        ok = false;
                        break;
                    }
                    ++tq;
                    tc_fence_after_sync();
                    ARC_TP(21);
                    const float inv = l > 0.f ? 1.0f / l : 0.f;
                    const float lse = l > 0.f ? (m + fast_log2(l)) * 0.6931471805599453f : -CUDART_INF_F;
                    uint16_t* dst = p.out + eoff;
                    const uint16_t* gp = GATE ? p.gate + eoff : nullptr;
                    const bool wide = (reinterpret_cast<uintptr_t>(dst) & 31u) == 0;
                    auto store_chunk = [&](const uint32_t (&w)[32], int c) {
                        if (store) {
        #pragma unroll
                            for (int e = 0; e < 32; e += 16) {
                                uint32_t ov[8];
        #pragma unroll
                                for (int hh = 0; hh < 2; ++hh) {
                                    float o[8];
        #pragma unroll
                                    for (int u = 0; u < 8; ++u) o[u] = __uint_as_float(w[e + hh * 8 + u]) * inv;
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
                                uint16_t* q = dst + c * 32 + e;
                                if (wide) {
                                    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(q), "r"(ov[0]),
                                                 "r"(ov[1]), "r"(ov[2]), "r"(ov[3]), "r"(ov[4]), "r"(ov[5]), "r"(ov[6]), "r"(ov[7])
                                                 : "memory");
                                } else {
                                    *reinterpret_cast<uint4*>(q) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
                                    *reinterpret_cast<uint4*>(q + 8) = make_uint4(ov[4], ov[5], ov[6], ov[7]);
                                }
                            }
                        }
                    };
                    // two 32-column chunks per round: their loads are in flight together
        #pragma unroll 1
                    for (int c = 0; c < HD / 32; c += 2) {
                        tmem_ld32(tO + c * 32, wa);
                        tmem_ld32(tO + c * 32 + 32, wb);
                        tmem_wait_ld();
                        if (c + 2 == HD / 32) {
                            // O is in registers: the next tile may overwrite the accumulator.
                            tc_fence_before_sync();
                            mbar_arrive(&o_empty[s]);
                        }
                        store_chunk(wa, c);
                        store_chunk(wb, c + 1);
                    }
                    if (store && p.out_lse) p.out_lse[row] = lse;
                    ARC_TP(22);
                }
            }
            if (!ok) break;
            if (hi == lo) {
                // Nothing visible for this tile: zero output.
                if (store) {
                    uint4* dst = reinterpret_cast<uint4*>(p.out + eoff);
                    for (int i = 0; i < HD / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                    if (p.out_lse) p.out_lse[row] = -CUDART_INF_F;
                }
                continue;
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
#ifdef ARC_TRACE_CTAS
    if (threadIdx.x == 0 && p.trace) p.trace[800 + blockIdx.x] = clock64() - ck0;
#endif
    if (warp == C::PRODUCER_WARP) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace arc
