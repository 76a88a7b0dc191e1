// HBM-bound split-KV decode kernel for sm_100a, plus the log-sum-exp merges.
//
// One new query token per sequence attends to that sequence's contiguous KV
// cache rows of (nkv, hd) bf16 (the reference's per-layer cache,
// src/modeling/qwen3_5/cache.hpp:9-14).  The key ranges of all sequences are
// laid end to end and cut into one equal share per CTA (persistent grid, one CTA
// per SM), so the load is balanced whatever the per-sequence lengths are and a
// CTA streams one long contiguous run of cache rows.
//
// Inside a CTA a producer warp streams the cache through a ring of
// shared-memory stages with TMA: the K and V caches are described as 2-D tensors
// (row = one position, all KV heads), and one copy moves a 64-element column
// chunk of a whole stage of rows (16-64 rows, 2-8 KB) with the 128-byte swizzle,
// so ldmatrix reads are bank-conflict free without padding and the copy engine
// sees few, large requests.  Consumer warps each own one KV head
// and a 16-key slice of every stage.  The GQA group of that head (<= 8 query
// heads per n-tile) forms the N dimension of the warp MMAs, so K and V are read
// from HBM and from shared memory exactly once per group:
//     S^T (16 keys x 8 heads) = K_tile (16 x hd) * Q^T (hd x 8)
//     O^T (hd x 8 heads)     += V_tile^T (hd x 16) * P^T (16 x 8)
// Online softmax state (max, sum) is per head = per accumulator column pair,
// reduced across the key rows with warp shuffles.  Each (CTA, sequence) pair a
// share touches yields partial (normalised out, lse) records: one per slice, or —
// for the last segment of a share, which is most of them — one for the CTA, the
// slices folded through shared memory first; the merge kernel folds the records
// and applies the optional sigmoid output gate
// (src/modeling/qwen3_5_moe/kernels.hpp:80-88) while writing bf16.
//
// The reference kernels this replaces read K/V once per query head and never
// split the key range (src/modeling/qwen3_5/kernels.hpp:761-905), or fold the
// group into the MMA rows but launch only nkv*4 work-groups (:910-1054).
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include "ptx.cuh"

namespace arc {

constexpr int DECODE_MAX_BATCH = 2048;

struct DecodeParams {
    const uint16_t* q;
    const int* kv_len;
    const long long* kv_row_offset;
    float* part_o;    // [(slot * slices + slice)][nq][HD]
    float* part_lse;  // [(slot * slices + slice)][nq]
    uint32_t* fault;
    int batch, nq, nkv, kv_len_uniform;
    long long q_stride_b, kv_stride_b, kv_stride_t;
    float scale_log2;
    int nkv_cta;  // KV heads handled by one CTA (grid.y = nkv / nkv_cta)
    int slices;   // 16-key slices per stage; consumer warps = nkv_cta * slices
    int stages;
    int ncta;     // grid.x
    int max_kv_len;            // > 0: no sequence may be longer
    long long kv_rows_total;   // rows addressable from k and v
};

// Prefix sums of the per-sequence lengths into shared memory: cum[b] = keys
// before sequence b, cum[batch] = total.  Called by every thread of the block.
__device__ __forceinline__ void build_len_prefix(const int* kv_len, int kv_len_uniform, int batch,
                                                 long long* cum) {
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
        int len = kv_len ? kv_len[b] : kv_len_uniform;
        cum[b + 1] = len > 0 ? len : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        long long run = 0;
        cum[0] = 0;
        for (int b = 0; b < batch; ++b) {
            run += cum[b + 1];
            cum[b + 1] = run;
        }
    }
    __syncthreads();
}

__device__ __forceinline__ long long share_size(long long total, int ncta, int tile_keys) {
    long long per = (total + ncta - 1) / ncta;
    per = (per + tile_keys - 1) / tile_keys * tile_keys;
    return per > 0 ? per : tile_keys;
}

// All consumer warps of the CTA (named barrier 1; the producer warp does not take part).
__device__ __forceinline__ void consumer_sync(int consumer_warps) {
    asm volatile("bar.sync 1, %0;" ::"r"(consumer_warps * 32) : "memory");
}

template <int HD, int NT>
__global__ void __launch_bounds__(288, 1)
    sdpa_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int ncw = p.nkv_cta * p.slices;  // consumer warps
    const int tk = 16 * p.slices;          // keys per stage
    const int row_bytes = p.nkv_cta * HD * 2;
    const int nchunks = p.nkv_cta * (HD / 64);  // 64-element column chunks per row
    const int chunk_bytes = tk * 128;           // one chunk of one stage: tk rows x 128 bytes
    const int tile_bytes = tk * row_bytes;      // one of K / V
    const int stage_bytes = 2 * tile_bytes;

    uint8_t* stage_base = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * stage_bytes);
    uint64_t* empty = full + p.stages;
    long long* cum = reinterpret_cast<long long*>(empty + p.stages);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int head0 = blockIdx.y * p.nkv_cta;  // first KV head of this CTA
    const int G = p.nq / p.nkv;

    grid_launch_dependents();  // the merge kernel may be scheduled now; it waits for this grid before reading
    // A fault recorded by an earlier CTA or launch: do not start new waits.
    __shared__ uint32_t abort_flag;
    // Everything the prologue reads from global memory is asked for at once: after an L2 flush each of these is
    // an HBM round trip, and taken one after the other (status word and lengths, then row offsets, then the
    // descriptors at the first copy) they kept the first K / V request waiting for several microseconds.
    if (p.kv_row_offset)
        for (int b = threadIdx.x * 16; b < p.batch; b += blockDim.x * 16) prefetch_l2(p.kv_row_offset + b);
    if (threadIdx.x == 32) {
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    if (threadIdx.x == 0) {
        abort_flag = *reinterpret_cast<volatile uint32_t*>(p.fault);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], ncw);
        }
        fence_mbar_init();
    }
    build_len_prefix(p.kv_len, p.kv_len_uniform, p.batch, cum);
    if (abort_flag != 0u) return;
    // Lengths and row offsets live on the device, so this is where they can be checked: a sequence
    // that reaches past the cache (the copies would read zero rows and fold them in as score-0
    // keys) or past the stated bound stops the launch with a status instead of a wrong result.
    for (int b = threadIdx.x; b < p.batch; b += blockDim.x) {
        const long long len = cum[b + 1] - cum[b];
        const long long row0 = p.kv_row_offset ? p.kv_row_offset[b] : (long long)b * p.kv_stride_b;
        if ((len > 0 && (row0 < 0 || row0 + len > p.kv_rows_total)) || (p.max_kv_len > 0 && len > p.max_kv_len)) {
            report_fault(p.fault, FAULT_BAD_KV_RANGE, (uint32_t)b);
            abort_flag = 1u;
        }
    }
    __syncthreads();
    if (abort_flag != 0u) return;
    const long long total = cum[p.batch];
    const long long per = share_size(total, p.ncta, tk);
    const long long g0 = (long long)blockIdx.x * per;
    const long long g1 = min(total, g0 + per);

    if (g0 >= g1) return;  // (the barriers were set up before the prefix's block-wide syncs)

    int b_first = 0;
    while (b_first < p.batch - 1 && cum[b_first + 1] <= g0) ++b_first;

    if (warp == ncw) {
        // ------------------------------------------------------------------ producer
        int it = 0;
        bool ok = true;
        int b = b_first;
        long long g = g0;
        while (ok && g < g1) {
            while (cum[b + 1] <= g) ++b;
            const long long seg_end = min(g1, cum[b + 1]);
            const long long row0 = (p.kv_row_offset ? p.kv_row_offset[b] : (long long)b * p.kv_stride_b) + (g - cum[b]);
            const int seg_keys = (int)(seg_end - g);
            for (int k0 = 0; k0 < seg_keys; k0 += tk, ++it) {
                const int st = it % p.stages;
                if (it >= p.stages && !mbar_wait_warp(&empty[st], ((it / p.stages) - 1) & 1)) {
                    if (lane == 0) report_fault(p.fault, FAULT_WAIT_EMPTY, it);
                    ok = false;
                    break;
                }
                // A stage always carries tk full rows: rows past the segment end
                // are masked by the consumers, rows past the cache end read as zero.
                if (lane == 0) mbar_arrive_expect_tx(&full[st], (uint32_t)stage_bytes);
                __syncwarp();
                uint8_t* dst = stage_base + (size_t)st * stage_bytes;
                const int row = (int)(row0 + k0);
                for (int c = lane; c < 2 * nchunks; c += 32) {
                    const int is_v = c >= nchunks;
                    const int cc = c - is_v * nchunks;
                    tma_load_2d(dst + (size_t)is_v * tile_bytes + (size_t)cc * chunk_bytes, is_v ? &tm_v : &tm_k,
                                &full[st], head0 * HD + cc * 64, row);
                }
            }
            g = seg_end;
        }
        // Drain: every copy issued above has landed before the CTA retires.
        if (lane == 0) {
            for (int back = 1; back <= p.stages && back <= it; ++back) {
                const int j = it - back;
                mbar_wait(&full[j % p.stages], (j / p.stages) & 1);
            }
        }
    } else if (warp < ncw) {
        // ------------------------------------------------------------------ consumers
        const int hl = warp % p.nkv_cta;  // local KV head
        const int slice = warp / p.nkv_cta;
        const int kvh = head0 + hl;
        const int g4 = lane >> 2;  // accumulator row group
        const int q4 = lane & 3;   // accumulator column pair
        const float sl = p.scale_log2;

        int it = 0;
        bool ok = true;
        bool folded = false;  // this warp has been through the two barriers of the in-CTA fold
        int b = b_first;
        long long g = g0;
        while (ok && g < g1) {
            while (cum[b + 1] <= g) ++b;
            const long long seg_end = min(g1, cum[b + 1]);
            const int seg_keys = (int)(seg_end - g);

            // Q^T fragments (B operand, hd x 8 heads) for this head's GQA group.
            uint32_t qf[NT][HD / 16][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int n = nt * 8 + g4;
                const bool valid = n < G;
                const uint16_t* qp = p.q + (long long)b * p.q_stride_b + ((long long)kvh * G + (valid ? n : 0)) * HD + q4 * 2;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    qf[nt][kk][0] = valid ? *reinterpret_cast<const uint32_t*>(qp + kk * 16) : 0u;
                    qf[nt][kk][1] = valid ? *reinterpret_cast<const uint32_t*>(qp + kk * 16 + 8) : 0u;
                }
            }
            float m[NT][2], l[NT][2];
            float o[NT][HD / 16][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                m[nt][0] = m[nt][1] = -CUDART_INF_F;
                l[nt][0] = l[nt][1] = 0.f;
#pragma unroll
                for (int mt = 0; mt < HD / 16; ++mt) o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.f;
            }

            for (int k0 = 0; k0 < seg_keys; k0 += tk, ++it) {
                const int st = it % p.stages;
                if (!mbar_wait_warp(&full[st], (it / p.stages) & 1)) {
                    if (lane == 0) report_fault(p.fault, FAULT_WAIT_FULL, it);
                    ok = false;
                    break;
                }
                const int nk = min(tk, seg_keys - k0);
                const int nvalid = min(16, nk - slice * 16);  // keys of this warp's slice
                if (nvalid > 0) {
                    // Swizzled addressing: 16-byte unit u of row r sits at unit u ^ (r & 7).
                    const uint32_t sK = smem_u32(stage_base + (size_t)st * stage_bytes) + hl * (HD / 64) * chunk_bytes;
                    const uint32_t sV = sK + tile_bytes;
                    const int key_k = slice * 16 + (lane & 15);
                    const int key_v = slice * 16 + (lane & 7) + (lane >> 4) * 8;
                    const uint32_t a_k = sK + key_k * 128;
                    const uint32_t a_v = sV + key_v * 128;
                    const int xk = key_k & 7, hk = lane >> 4;
                    const int xv = key_v & 7, hv = (lane >> 3) & 1;
                    if (nvalid < 16) {
                        // Rows past the segment end may hold anything (another sequence, or
                        // never-written cache); clear this warp's V rows so 0 * x stays 0.
                        for (int i = lane; i < (16 - nvalid) * (HD / 8); i += 32) {
                            const int key = slice * 16 + nvalid + i / (HD / 8);
                            const int u = i % (HD / 8);
                            const uint32_t a = sV + (u >> 3) * chunk_bytes + key * 128 + (u & 7) * 16;
                            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(a), "r"(0u) : "memory");
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                    }

                    float acc[NT][2][4];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) acc[nt][hh][0] = acc[nt][hh][1] = acc[nt][hh][2] = acc[nt][hh][3] = 0.f;
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk) {
                        uint32_t a[4];
                        ldmatrix_x4(a, a_k + (kk >> 2) * chunk_bytes + ((((kk & 3) * 2 + hk) ^ xk) << 4));
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[nt][kk & 1], a, qf[nt][kk][0], qf[nt][kk][1]);
                    }
                    const bool v_lo = g4 < nvalid, v_hi = g4 + 8 < nvalid;
                    uint32_t pb[NT][2];
                    bool any_rescale = false;
                    float alpha[NT][2];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        float x[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float s = (acc[nt][0][e] + acc[nt][1][e]) * sl;
                            x[e] = ((e < 2) ? v_lo : v_hi) ? s : -CUDART_INF_F;
                        }
                        float pr[4];
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            float mx = fmaxf(x[u], x[u + 2]);
                            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                            const float m_new = fmaxf(m[nt][u], mx);
                            const float m_eff = (m_new == -CUDART_INF_F) ? 0.f : m_new;
                            alpha[nt][u] = (m_new == -CUDART_INF_F) ? 1.f : fast_exp2(m[nt][u] - m_new);
                            pr[u] = fast_exp2(x[u] - m_eff);
                            pr[u + 2] = fast_exp2(x[u + 2] - m_eff);
                            l[nt][u] = l[nt][u] * alpha[nt][u] + pr[u] + pr[u + 2];
                            m[nt][u] = m_new;
                            any_rescale |= alpha[nt][u] != 1.f;
                        }
                        pb[nt][0] = movmatrix_trans(pack_bf16x2(pr[0], pr[1]));
                        pb[nt][1] = movmatrix_trans(pack_bf16x2(pr[2], pr[3]));
                    }
                    if (__any_sync(0xffffffffu, any_rescale)) {
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int mt = 0; mt < HD / 16; ++mt) {
                                o[nt][mt][0] *= alpha[nt][0];
                                o[nt][mt][1] *= alpha[nt][1];
                                o[nt][mt][2] *= alpha[nt][0];
                                o[nt][mt][3] *= alpha[nt][1];
                            }
                    }
#pragma unroll
                    for (int mt = 0; mt < HD / 16; ++mt) {
                        uint32_t a[4];
                        ldmatrix_x4_trans(a, a_v + (mt >> 2) * chunk_bytes + ((((mt & 3) * 2 + hv) ^ xv) << 4));
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(o[nt][mt], a, pb[nt][0], pb[nt][1]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[st]);
            }

            // Partial record of this (CTA, sequence, slice): normalised out + natural-log lse.
            // The last segment of the share (for most CTAs the only one) is folded across the slices inside
            // the CTA first: the stages are free by then, so each warp leaves its record in shared memory,
            // and the warps of a KV head combine them into ONE record per (CTA, sequence), stored in slice
            // 0's slot; the other slices' slots are marked empty (lse = -inf).  The merge kernel then reads
            // `slices` times fewer records.  Earlier segments (a sequence boundary inside the share) write
            // one record per slice.
            const bool fold_here = p.slices > 1 && seg_end == g1;  // CTA-uniform
            float* rec = reinterpret_cast<float*>(stage_base);     // [warp][NT * 8 heads][HD]
            float* rec_lse = rec + (size_t)ncw * NT * 8 * HD;      // [warp][NT * 8]
            if (fold_here) {
                consumer_sync(ncw);  // every warp is through with the stages; no copy is in flight any more
                folded = true;
            }
            if (ok) {
                const long long part = ((long long)blockIdx.x + b) * p.slices + slice;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float inv[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        float ls = l[nt][u];
                        ls += __shfl_xor_sync(0xffffffffu, ls, 4);
                        ls += __shfl_xor_sync(0xffffffffu, ls, 8);
                        ls += __shfl_xor_sync(0xffffffffu, ls, 16);
                        inv[u] = ls > 0.f ? 1.f / ls : 0.f;
                        const int n = nt * 8 + q4 * 2 + u;
                        const float lse = ls > 0.f ? (m[nt][u] + fast_log2(ls)) * 0.6931471805599453f : -CUDART_INF_F;
                        if (g4 == 0) {
                            if (fold_here) rec_lse[warp * NT * 8 + n] = lse;
                            else if (n < G) p.part_lse[part * p.nq + (long long)kvh * G + n] = lse;
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int n = nt * 8 + q4 * 2 + u;
                        if (fold_here || n < G) {
                            float* dst = fold_here ? rec + ((size_t)warp * NT * 8 + n) * HD
                                                   : p.part_o + (part * p.nq + (long long)kvh * G + n) * HD;
#pragma unroll
                            for (int mt = 0; mt < HD / 16; ++mt) {
                                dst[mt * 16 + g4] = o[nt][mt][u] * inv[u];
                                dst[mt * 16 + g4 + 8] = o[nt][mt][u + 2] * inv[u];
                            }
                        }
                    }
                }
            }
            if (fold_here) {
                consumer_sync(ncw);  // all records of the CTA are in shared memory
                // The `slices` warps of this KV head share its G x HD output values, four per step.
                const long long part0 = ((long long)blockIdx.x + b) * p.slices;
                for (int item = slice * 32 + lane; item < G * (HD / 4); item += p.slices * 32) {
                    const int n = item / (HD / 4), d = (item % (HD / 4)) * 4;
                    float mx = -CUDART_INF_F;
                    for (int sidx = 0; sidx < p.slices; ++sidx)
                        mx = fmaxf(mx, rec_lse[(sidx * p.nkv_cta + hl) * NT * 8 + n]);
                    float z = 0.f;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (mx > -CUDART_INF_F) {
                        for (int sidx = 0; sidx < p.slices; ++sidx) {
                            const int w = sidx * p.nkv_cta + hl;
                            const float li = rec_lse[w * NT * 8 + n];
                            if (li == -CUDART_INF_F) continue;
                            const float wt = __expf(li - mx);
                            z += wt;
                            const float4 ov = *reinterpret_cast<const float4*>(rec + ((size_t)w * NT * 8 + n) * HD + d);
                            acc.x = fmaf(wt, ov.x, acc.x);
                            acc.y = fmaf(wt, ov.y, acc.y);
                            acc.z = fmaf(wt, ov.z, acc.z);
                            acc.w = fmaf(wt, ov.w, acc.w);
                        }
                        const float iz = 1.f / z;
                        acc = make_float4(acc.x * iz, acc.y * iz, acc.z * iz, acc.w * iz);
                    }
                    const long long row = part0 * p.nq + (long long)kvh * G + n;
                    *reinterpret_cast<float4*>(p.part_o + row * HD + d) = acc;
                    if (d == 0) p.part_lse[row] = mx > -CUDART_INF_F ? mx + __logf(z) : -CUDART_INF_F;
                }
                if (slice > 0 && lane < G) p.part_lse[(part0 + slice) * p.nq + (long long)kvh * G + lane] = -CUDART_INF_F;
            }
            g = seg_end;
        }
        // A warp that gave up a wait never reached the fold: it still meets the others at both barriers.
        if (p.slices > 1 && !folded) {
            consumer_sync(ncw);
            consumer_sync(ncw);
        }
    }
}

// ---------------------------------------------------------------------------
// Merge of the decode partials.  grid = (nq, batch); the block recomputes the
// same share boundaries the decode kernel used to find the records of its
// sequence: CTAs [c_first, c_last] x slices, record index (cta + b)*slices + s.
// ---------------------------------------------------------------------------
struct DecodeMergeParams {
    const float* part_o;
    const float* part_lse;
    const int* kv_len;
    const uint16_t* gate;
    uint16_t* out;
    float* out_f32;
    float* out_lse;
    int batch, nq, kv_len_uniform;
    int ncta, slices;
    long long o_stride_b;
    // Sequence-sharded decode over NVLink peer memory (x_world > 1): every rank's exchange
    // buffer base address; this rank's index; a step counter that grows by one per call.
    const unsigned long long* x_peers;
    int x_world, x_rank;
    uint32_t x_step;
    long long x_wait_cycles;  // bound of the wait for the other ranks' records
    uint32_t* fault;
};

// Layout of one rank's exchange buffer: [2 parities][world sources][rows] records of HD + 2 words, a word
// being 8 bytes = (value bits, step).  Every value travels with the step number it belongs to, so a
// receiver recognises a word as soon as it lands: no fence between data and a separate flag, one NVLink
// crossing per exchange instead of three (stores, their acknowledgement, the flag).  Words HD and HD + 1
// hold the row's log-sum-exp and padding.  8-byte stores are single transactions; a 16-byte store may be
// split, which is fine because each half carries its own step.
constexpr int XCHG_MAX_WORLD = 16;  // ranks of one exchange (one NVSwitch box has 8)
__host__ __device__ inline size_t xchg_record_words(int hd) { return (size_t)hd + 2; }
__host__ __device__ inline size_t xchg_total_bytes(int world, long long rows, int hd) {
    return (size_t)2 * world * rows * xchg_record_words(hd) * 8;
}

__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float sigmoid_gate(float attn, uint16_t gate_bits) {
    const float g = bf16_bits_to_f32(gate_bits);
    return bf16_round(attn) * (1.0f / (1.0f + __expf(-g)));
}

constexpr int MERGE_THREADS = 256;

// Block-wide max / sum over MERGE_THREADS threads (result to every thread).
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch[0];
#pragma unroll
    for (int w = 1; w < MERGE_THREADS / 32; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
    return r;
}

// XCHG: the instance that also exchanges records with other GPUs.  It keeps every source's values in
// registers; the plain merge — hundreds of small blocks for a large batch — stays lean enough for five blocks
// per SM.
template <int HD, bool XCHG>
__global__ void __launch_bounds__(MERGE_THREADS) sdpa_decode_merge_kernel(const DecodeMergeParams p) {
    extern __shared__ uint8_t smem_raw[];
    long long* cum = reinterpret_cast<long long*>(smem_raw);
    float* red = reinterpret_cast<float*>(cum + p.batch + 2);      // 8 floats
    float* acc_sm = red + 8;                                        // (warps) x HD
    float* wgt = acc_sm + (MERGE_THREADS / 32) * HD;                // one weight per record
    __shared__ int n_live_sm;
    // What does not depend on the decode kernel's results happens while it still runs: the length prefix, and
    // requests for the lines the tail will need (this row's gate values, the status word) into L2.
    if (p.gate && p.out && threadIdx.x < HD * 2 / 128)
        prefetch_l2(p.gate + (long long)blockIdx.y * p.o_stride_b + (long long)blockIdx.x * HD + threadIdx.x * 64);
    if (threadIdx.x == 32) prefetch_l2(p.fault);
    build_len_prefix(p.kv_len, p.kv_len_uniform, p.batch, cum);
    grid_dependency_wait();                                        // from here on its partial records are read
    if (*reinterpret_cast<volatile uint32_t*>(p.fault) != 0u) return;  // block-uniform: a status is set, no work
    const int h = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long total = cum[p.batch];
    const long long per = share_size(total, p.ncta, 16 * p.slices);
    const long long k_begin = cum[b], k_end = cum[b + 1];
    constexpr int VPL = HD / 32;  // output values per lane
    float acc[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
    float lse = -CUDART_INF_F, inv = 0.f;
    if (k_end > k_begin) {  // block-uniform
        const int c_first = (int)(k_begin / per), c_last = (int)((k_end - 1) / per);
        const int n_parts = (c_last - c_first + 1) * p.slices;
        const long long part0 = ((long long)c_first + b) * p.slices;
        // weights: every thread takes a strided set of records
        float mx = -CUDART_INF_F;
        for (int i = threadIdx.x; i < n_parts; i += MERGE_THREADS) {
            const float li = p.part_lse[(part0 + i) * p.nq + h];
            wgt[i] = li;
            mx = fmaxf(mx, li);
        }
        mx = block_reduce(mx, true, red);
        float z = 0.f;
        if (mx > -CUDART_INF_F) {
            for (int i = threadIdx.x; i < n_parts; i += MERGE_THREADS) {
                const float w = __expf(wgt[i] - mx);  // exp(-inf) = 0 for empty records
                wgt[i] = w;
                z += w;
            }
        }
        z = block_reduce(z, false, red);  // also orders the wgt[] writes before the reads below
        if (z > 0.f) {
            inv = 1.f / z;
            lse = mx + __logf(z);
            // Most records carry no weight (the decode kernel folds the slices of a share's last segment
            // into slice 0's slot and marks the others empty; slots of other sequences' shares): warp 0
            // lists the live ones, in order, so that the fold below is spread evenly and always adds in the
            // same order.
            int* live = reinterpret_cast<int*>(wgt + n_parts);
            if (warp == 0) {
                int base = 0;
                for (int i0 = 0; i0 < n_parts; i0 += 32) {
                    const int i = i0 + lane;
                    const bool on = i < n_parts && wgt[i] != 0.f;
                    const uint32_t bal = __ballot_sync(0xffffffffu, on);
                    if (on) live[base + __popc(bal & ((1u << lane) - 1u))] = i;
                    base += __popc(bal);
                }
                if (lane == 0) n_live_sm = base;
            }
            __syncthreads();
            const int n_live = n_live_sm;
            // each warp folds every 8th live record, four at a time so that their loads are in flight
            // together (one record after the other, the loop ran at one L2 latency per record);
            // a lane owns VPL consecutive output values
            constexpr int NW = MERGE_THREADS / 32, U = 4;
            for (int j0 = warp; j0 < n_live; j0 += NW * U) {
                float w[U];
                float4 ov[U][VPL / 4];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int jj = j0 + u * NW;
                    const int i = jj < n_live ? live[jj] : 0;
                    w[u] = jj < n_live ? wgt[i] : 0.f;
                    const float* src = p.part_o + ((part0 + i) * p.nq + h) * HD + lane * VPL;
#pragma unroll
                    for (int j = 0; j < VPL / 4; ++j)
                        ov[u][j] = w[u] != 0.f ? *reinterpret_cast<const float4*>(src + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
#pragma unroll
                    for (int j = 0; j < VPL / 4; ++j) {
                        acc[4 * j] = fmaf(w[u], ov[u][j].x, acc[4 * j]);
                        acc[4 * j + 1] = fmaf(w[u], ov[u][j].y, acc[4 * j + 1]);
                        acc[4 * j + 2] = fmaf(w[u], ov[u][j].z, acc[4 * j + 2]);
                        acc[4 * j + 3] = fmaf(w[u], ov[u][j].w, acc[4 * j + 3]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc_sm[warp * HD + lane * VPL + j] = acc[j];
    __syncthreads();
    const long long row = (long long)b * p.nq + h;
    if (p.out_lse && threadIdx.x == 0) p.out_lse[row] = lse;
    const int d = threadIdx.x * 2;
    float a0 = 0.f, a1 = 0.f;
    if (threadIdx.x < HD / 2) {
#pragma unroll
        for (int w = 0; w < MERGE_THREADS / 32; ++w) {
            a0 += acc_sm[w * HD + d];
            a1 += acc_sm[w * HD + d + 1];
        }
        a0 *= inv;
        a1 *= inv;
        if (p.out_f32) *reinterpret_cast<float2*>(p.out_f32 + row * HD + d) = make_float2(a0, a1);
    }
    if (XCHG && p.x_world > 1) {
        // Sequence-sharded: this rank's (out, lse) of the row goes straight into every rank's exchange
        // buffer over NVLink as plain peer stores of (value, step) words.  Then the block waits — for a
        // bounded time — until the words of every source rank show this step, and folds the records.
        // Thread t < HD / 2 sends and receives values 2t, 2t + 1 (one 16-byte store / load); thread HD / 2
        // does the same for the log-sum-exp word and hands the sources' values round through shared memory.
        const long long rows = (long long)p.batch * p.nq;
        const int par = (int)(p.x_step & 1u);
        const size_t rw = xchg_record_words(HD) / 2;  // 16-byte units per record
        const size_t slot = ((size_t)par * p.x_world + p.x_rank) * rows + row;
        const bool sender = threadIdx.x <= HD / 2;
        if (sender) {
            const uint4 word = threadIdx.x < HD / 2 ? make_uint4(__float_as_uint(a0), p.x_step, __float_as_uint(a1), p.x_step)
                                                    : make_uint4(__float_as_uint(lse), p.x_step, 0u, p.x_step);
            for (int dst = 0; dst < p.x_world; ++dst)
                st_volatile_v4(reinterpret_cast<uint4*>(p.x_peers[dst]) + slot * rw + threadIdx.x, word);
        }
        const uint4* mine = reinterpret_cast<const uint4*>(p.x_peers[p.x_rank]);
        __shared__ int x_timeout;
        __shared__ float x_lse[XCHG_MAX_WORLD];
        if (threadIdx.x == 0) x_timeout = 0;
        __syncthreads();
        float b0 = 0.f, b1 = 0.f, z = 0.f;
        float2 rv[XCHG_MAX_WORLD];  // this thread's two values from every source
        if (sender) {
            const long long t0 = clock64();
            bool gave_up = false;
#pragma unroll
            for (int src = 0; src < XCHG_MAX_WORLD; ++src) {
                if (src >= p.x_world) break;
                const uint4* w = mine + (((size_t)par * p.x_world + src) * rows + row) * rw + threadIdx.x;
                uint4 v = ld_volatile_v4(w);
                while (!gave_up && (v.y != p.x_step || v.w != p.x_step)) {
                    if (clock64() - t0 > p.x_wait_cycles) {  // the peer never came
                        report_fault(p.fault, FAULT_WAIT_PEER, (uint32_t)src);
                        x_timeout = 1;
                        gave_up = true;
                        break;
                    }
                    v = ld_volatile_v4(w);
                }
                rv[src] = make_float2(__uint_as_float(v.x), __uint_as_float(v.z));
                if (threadIdx.x == HD / 2) x_lse[src] = rv[src].x;
            }
        }
        __syncthreads();  // x_lse[] and x_timeout are visible
        if (x_timeout) return;
        float mx = -CUDART_INF_F;
        for (int src = 0; src < p.x_world; ++src) mx = fmaxf(mx, x_lse[src]);
        if (mx > -CUDART_INF_F && threadIdx.x < HD / 2) {
#pragma unroll
            for (int src = 0; src < XCHG_MAX_WORLD; ++src) {
                if (src >= p.x_world) break;
                const float li = x_lse[src];
                if (li == -CUDART_INF_F) continue;
                const float wgt_s = __expf(li - mx);
                z += wgt_s;
                b0 = fmaf(wgt_s, rv[src].x, b0);
                b1 = fmaf(wgt_s, rv[src].y, b1);
            }
            b0 /= z;
            b1 /= z;
        }
        a0 = b0;
        a1 = b1;
    }
    if (threadIdx.x < HD / 2) {
        if (p.out) {
            const long long eoff = (long long)b * p.o_stride_b + (long long)h * HD + d;
            if (p.gate) {
                const uint32_t gw = *reinterpret_cast<const uint32_t*>(p.gate + eoff);
                a0 = sigmoid_gate(a0, (uint16_t)(gw & 0xffffu));
                a1 = sigmoid_gate(a1, (uint16_t)(gw >> 16));
            }
            *reinterpret_cast<uint32_t*>(p.out + eoff) = pack_bf16x2(a0, a1);
        }
    }
}

// ---------------------------------------------------------------------------
// Merge of `num_parts` uniformly strided partial sets: part_o (parts, rows, hd),
// part_lse (parts, rows), consecutive parts o_part_stride / lse_part_stride
// elements apart (so one packed record per part works too).  One block per row.  Used for split prefill tiles and
// for records gathered from other GPUs.  out rows are contiguous (rows, hd)
// unless row_tokens > 0, in which case row = (b, t, h) is scattered with the
// given strides (prefill output layout).
// ---------------------------------------------------------------------------
struct UniformMergeParams {
    const float* part_o;
    const float* part_lse;
    const uint16_t* gate;
    uint16_t* out;
    float* out_f32;
    float* out_lse;
    long long rows;
    long long o_part_stride, lse_part_stride;  // elements between consecutive parts
    int num_parts;
    int seq, nq;  // seq > 0: strided (b, t, h) addressing of out / gate
    long long o_stride_b, o_stride_t;
    const unsigned long long* out_copies;  // n_copies more output buffers, same offsets (prefill: other GPUs' buffers)
    int n_copies;
};

constexpr int UMERGE_ROWS = 8;  // rows per block of the uniform merge: one warp each

template <int HD>
__global__ void __launch_bounds__(32 * UMERGE_ROWS) sdpa_uniform_merge_kernel(const UniformMergeParams p) {
    grid_dependency_wait();  // launched behind the kernel that writes the partials, possibly before it has finished
    const long long row = (long long)blockIdx.x * UMERGE_ROWS + (threadIdx.x >> 5);
    if (row >= p.rows) return;
    const int lane = threadIdx.x & 31;
    constexpr int VPL = HD / 32;  // output values per lane: 4 or 8 consecutive ones
    const int d = lane * VPL;
    // One warp per row (a block per row spent its time being scheduled: thousands of 64-thread blocks).
    // Parts are taken four at a time with all their loads in flight together.
    constexpr int U = 4;
    float mx = -CUDART_INF_F;
    for (int i0 = 0; i0 < p.num_parts; i0 += U) {
        float li[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            li[u] = i0 + u < p.num_parts ? p.part_lse[(long long)(i0 + u) * p.lse_part_stride + row] : -CUDART_INF_F;
#pragma unroll
        for (int u = 0; u < U; ++u) mx = fmaxf(mx, li[u]);
    }
    float acc[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
    float lse = -CUDART_INF_F;
    if (mx > -CUDART_INF_F) {
        float z = 0.f;
        for (int i0 = 0; i0 < p.num_parts; i0 += U) {
            float li[U];
            float4 ov[U][VPL / 4];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool in = i0 + u < p.num_parts;
                li[u] = in ? p.part_lse[(long long)(i0 + u) * p.lse_part_stride + row] : -CUDART_INF_F;
                const float* src = p.part_o + (long long)(i0 + u) * p.o_part_stride + row * HD + d;
#pragma unroll
                for (int j = 0; j < VPL / 4; ++j)
                    ov[u][j] = (in && li[u] != -CUDART_INF_F) ? *reinterpret_cast<const float4*>(src + 4 * j)
                                                               : make_float4(0.f, 0.f, 0.f, 0.f);  // an empty part's record may hold anything
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (li[u] == -CUDART_INF_F) continue;
                const float w = __expf(li[u] - mx);
                z += w;
#pragma unroll
                for (int j = 0; j < VPL / 4; ++j) {
                    acc[4 * j] = fmaf(w, ov[u][j].x, acc[4 * j]);
                    acc[4 * j + 1] = fmaf(w, ov[u][j].y, acc[4 * j + 1]);
                    acc[4 * j + 2] = fmaf(w, ov[u][j].z, acc[4 * j + 2]);
                    acc[4 * j + 3] = fmaf(w, ov[u][j].w, acc[4 * j + 3]);
                }
            }
        }
        const float inv = 1.f / z;
#pragma unroll
        for (int j = 0; j < VPL; ++j) acc[j] *= inv;
        lse = mx + __logf(z);
    }
    if (p.out_f32) {
#pragma unroll
        for (int j = 0; j < VPL / 4; ++j)
            *reinterpret_cast<float4*>(p.out_f32 + row * HD + d + 4 * j) = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    }
    if (p.out_lse && lane == 0) p.out_lse[row] = lse;
    if (p.out) {
        long long eoff = row * HD + d;
        if (p.seq > 0) {
            const long long hh = row % p.nq;
            const long long t = (row / p.nq) % p.seq;
            const long long bb = row / ((long long)p.nq * p.seq);
            eoff = bb * p.o_stride_b + t * p.o_stride_t + hh * HD + d;
        }
        uint32_t packed[VPL / 2];
#pragma unroll
        for (int j = 0; j < VPL / 2; ++j) {
            float a0 = acc[2 * j], a1 = acc[2 * j + 1];
            if (p.gate) {
                const uint32_t gw = *reinterpret_cast<const uint32_t*>(p.gate + eoff + 2 * j);
                a0 = sigmoid_gate(a0, (uint16_t)(gw & 0xffffu));
                a1 = sigmoid_gate(a1, (uint16_t)(gw >> 16));
            }
            packed[j] = pack_bf16x2(a0, a1);
        }
        for (int c = -1; c < p.n_copies; ++c) {
            uint16_t* o = (c < 0 ? p.out : reinterpret_cast<uint16_t*>(p.out_copies[c])) + eoff;
            if (VPL == 8) *reinterpret_cast<uint4*>(o) = make_uint4(packed[0], packed[1], packed[VPL / 2 - 2], packed[VPL / 2 - 1]);
            else *reinterpret_cast<uint2*>(o) = make_uint2(packed[0], packed[1]);
        }
    }
}

// a[i] = bf16(f32(a[i]) * sigmoid(f32(gate[i]))) : src/modeling/qwen3_5_moe/kernels.hpp:80-88
__global__ void mul_sigmoid_kernel(uint16_t* a, const uint16_t* gate, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = bf16_bits_to_f32(gate[i]);
        const float sig = 1.0f / (1.0f + __expf(-g));
        a[i] = __bfloat16_as_ushort(__float2bfloat16_rn(bf16_bits_to_f32(a[i]) * sig));
    }
}

// Additive causal / sliding-window mask : src/common/kernels/attention_mask.hpp:12-38; with
// block_ids (one int per absolute position, -1 = text) tokens of the same non-negative block also
// see each other's future: fill_causal_mask_with_block_ids, attention_mask.hpp:44-73.
__global__ void fill_causal_mask_kernel(float* mask, const int* block_ids, int q_len, int kv_len, int past_offset,
                                        int window) {
    const long long n = (long long)q_len * kv_len;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int qi = (int)(i / kv_len), kvj = (int)(i % kv_len);
        const int q_global = past_offset + qi;
        const int kv_global = past_offset - (kv_len - q_len) + kvj;
        bool same_block = false;
        if (block_ids) {
            const int qb = block_ids[q_global];
            same_block = qb >= 0 && kv_global >= 0 && qb == block_ids[kv_global];
        }
        const bool causal = !same_block && kv_global > q_global;
        const bool too_far = (window != 0x7fffffff) && (kv_global < q_global - window + 1);
        mask[i] = (causal || too_far) ? -CUDART_INF_F : 0.0f;
    }
}

// First key each query row can no longer see under the causal rule extended by Gemma4's vision
// blocks (src/common/kernels/attention_mask.hpp:44-73): a query inside a block (same non-negative id,
// contiguous) sees the block's later keys as well.  ids[base + j] is key j's id; row t sits at key
// position t + off.  One thread per row; the scan runs to the end of the row's block at most.
__global__ void vision_span_kernel(const int* ids, int base, int off, int seq, int kv_len, int* vis_hi) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= seq) return;
    const int self = t + off;  // key index of the query's own position
    int hi = min(max(self + 1, 0), kv_len);
    if (self >= 0 && self < kv_len) {
        const int id = ids[base + self];
        if (id >= 0)
            while (hi < kv_len && ids[base + hi] == id) ++hi;
    }
    vis_hi[t] = hi;
}

}  // namespace arc
