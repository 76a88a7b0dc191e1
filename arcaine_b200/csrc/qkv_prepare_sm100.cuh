// What runs just before attention, as one HBM-bound kernel: RMSNorm (+ RoPE) of the projected
// Q and K rows, unit-RMS norm of V, and the append of K and V into the KV cache.
//
// The reference does this with separate launches per tensor and two memcpys into the cache
// (src/modeling/diffusion_gemma/attention.cpp:529-610 for the norms and RoPE, :1017-1020 for the
// cache append; the kernels are src/common/kernels/rms_norm.hpp:9-49 and
// src/modeling/diffusion_gemma/attention_kernels.hpp:99-153).  Here every element is read once
// and written once: Q in place, K and V straight to their cache rows.
//
// Arithmetic and rounding order follow the reference: the normalised value v * rsqrt(mean(v^2) +
// eps) * weight is rounded to bf16 first, and the rotation
//   x[p] = x0 c - x1 s,  x[p + hd/2] = x0 s + x1 c,   p < n_active_pairs
// works on those rounded values.  cos / sin come from a caller table (seq x n_active_pairs, as
// the reference's RopeTable) or are computed per token: angle = (offset + token) / theta^(2p/hd).
//
// Mapping: one CTA per group of consecutive tokens at a time (grid-stride), cos / sin of those
// tokens staged once in shared memory and shared by all their heads (the reference's "Fused"
// mode), one warp per
// (token, head) row segment: a lane holds eight consecutive elements of the row's first half and
// the matching eight of the second half (16-byte loads), so a rotation pair never leaves the lane
// and a warp covers 4 / 2 / 1 rows at once for head dim 128 / 256 / 512.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace arc {

struct QkvPrepareParams {
    uint16_t* q;            // (batch, seq, nq, hd) in place, or nullptr
    const uint16_t* k_src;  // (batch, seq, nkv, hd) projected K, or nullptr
    const uint16_t* v_src;  // projected V; nullptr with v_dst set: V is taken from k_src (before its norm)
    uint16_t* k_dst;        // cache row of the first token (may equal k_src)
    uint16_t* v_dst;        // or nullptr
    const uint16_t* q_weight;  // [hd] or nullptr (unit scale)
    const uint16_t* k_weight;
    const float* rope_cos;  // (seq, nap) or nullptr: computed inline
    const float* rope_sin;
    const int* pos_offset;  // [batch] position of each sequence's first token, or nullptr: pos0
    int batch, seq, nq, nkv, nap;
    long long q_stride_b, q_stride_t;
    long long ks_stride_b, ks_stride_t, vs_stride_b, vs_stride_t;
    long long kd_stride_b, kd_stride_t, vd_stride_b, vd_stride_t;
    long long rope_stride_b;  // elements between the tables of two sequences (0: shared)
    int pos0;
    float theta, eps;
    // Qwen3.5 multi-axis RoPE (src/modeling/qwen3_5/kernels.hpp:576-617): pairs (f, f + rot_half) inside the
    // first 2 * rot_half values of a row, frequency exponent 2 f / freq_denom, position taken from one of
    // three axes per frequency.  rot_half == hd / 2 with no positions is the plain form.
    int rot_half, freq_denom;
    const int* mrope_pos;  // (batch, 3, seq) or nullptr
    int sec1, sec2;        // sections of axes 1 and 2
    int v_copy;            // V rows are copied, not normalised
};

__device__ __forceinline__ int mrope_axis(int f, int sec1, int sec2) {
    if (f >= 1 && f < sec1 * 3 && f % 3 == 1) return 1;
    if (f >= 2 && f < sec2 * 3 && f % 3 == 2) return 2;
    return 0;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

__device__ __forceinline__ float bf16_rne(float x) {
    return __uint_as_float(static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x))) << 16);
}

// 256 threads = 8 warps.  A row of HD values is held by HD/16 lanes, each with eight consecutive
// values of the row's first half and the matching eight of the second half (two 16-byte loads),
// so a warp works on 32 / (HD/16) rows at once: 4 (HD 128), 2 (HD 256) or 1 (HD 512).  A CTA
// takes `tpc` consecutive tokens per round (the host picks tpc so that a round has work for all
// eight warps even when a rank holds only a few heads).
// QWEN: the Qwen3.5 form (pairs rot_half apart, per-axis positions, V copied); the common instance does not
// carry its branches.
// AHEAD: a warp issues the loads of its next pass before it works on this one (64 registers, four CTAs per SM:
// faster when a token has many rows); without it 40 registers and six CTAs per SM (faster for the few rows per
// token of a rank that holds a few heads).
template <int HD, bool QWEN, bool AHEAD>
__global__ void __launch_bounds__(256) qkv_prepare_kernel(const QkvPrepareParams p, const int tpc) {
    constexpr int LPR = HD / 16;    // lanes per row
    constexpr int RPW = 32 / LPR;   // rows per warp and pass
    constexpr int MAX_TPC = 1024 / (HD / 2);
    __shared__ float s_cos2[2][1024];  // [round parity][token in round][pair]: one barrier per round is enough
    __shared__ float s_sin2[2][1024];
    __shared__ float s_inv[HD / 2];    // rotation frequencies, computed once
    __shared__ int s_bt[2][2 * 16];     // [round parity][token in round] -> (batch index, token in sequence)
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR;     // which of the warp's rows
    const int li = lane % LPR;      // position inside the row
    const int rows_q = p.q ? p.nq : 0;
    const int rows_k = p.k_src && p.k_dst ? p.nkv : 0;
    const int rows_v = p.v_dst ? p.nkv : 0;
    const int rows = rows_q + rows_k + rows_v;
    const int tokens = p.batch * p.seq;  // the host refuses more than 2^31 - 1 tokens
    const int rounds = (tokens + tpc - 1) / tpc;
    (void)MAX_TPC;

    if (p.nap > 0 && !p.rope_cos) {
        for (int pr = threadIdx.x; pr < p.nap; pr += blockDim.x)
            s_inv[pr] = 1.0f / powf(p.theta, 2.0f * pr / static_cast<float>(QWEN ? p.freq_denom : HD));
        __syncthreads();
    }
    int it = 0;
    for (int rd = blockIdx.x; rd < rounds; rd += gridDim.x, ++it) {
        const int tk0 = rd * tpc;
        float* s_cos = s_cos2[it & 1];
        float* s_sin = s_sin2[it & 1];
        // The tokens of this round, split into (sequence, position) once: the row loop below would
        // otherwise divide per row.
        int* s_tok = s_bt[it & 1];
        if (threadIdx.x < tpc && tk0 + (int)threadIdx.x < tokens) {
            const int tk = tk0 + threadIdx.x;
            const int b = tk / p.seq;
            s_tok[2 * threadIdx.x] = b;
            s_tok[2 * threadIdx.x + 1] = tk - b * p.seq;
        }
        if (p.nap > 0) {
            for (int idx = threadIdx.x; idx < tpc * p.nap; idx += blockDim.x) {
                const int tl = idx / p.nap, pr = idx - tl * p.nap;
                const int tk = tk0 + tl;
                if (tk >= tokens) break;
                const int b = tk / p.seq;
                const int t = tk - b * p.seq;
                float c, s;
                if (p.rope_cos) {
                    const long long ti = (long long)b * p.rope_stride_b + (long long)t * p.nap + pr;
                    c = p.rope_cos[ti];
                    s = p.rope_sin[ti];
                } else {
                    const int pos = (QWEN && p.mrope_pos)
                                        ? p.mrope_pos[((long long)b * 3 + mrope_axis(pr, p.sec1, p.sec2)) * p.seq + t]
                                        : (p.pos_offset ? p.pos_offset[b] : p.pos0) + t;
                    sincosf(static_cast<float>(pos) * s_inv[pr], &s, &c);
                }
                s_cos[tl * (HD / 2) + pr] = c;
                s_sin[tl * (HD / 2) + pr] = s;
            }
        }
        // Readers of these buffers two rounds ago finished before every thread reached the previous
        // round's barrier, so one barrier per round orders both directions.
        __syncthreads();
        const float inv_rows = 1.0f / static_cast<float>(rows);
        const int slots = tpc * rows;  // (token in round, row) pairs of this round
        // AHEAD: the addresses of the next pass's rows are worked out and their loads issued before this pass's
        // rows are processed, so that a warp has two passes' worth of loads in flight instead of waiting out one
        // DRAM latency per pass.
        struct Pass {
            const uint16_t* weight;
            uint16_t* dst;
            uint4 rl, rh;
            int tl;
            bool valid, rope, norm;
        };
        auto fetch = [&](int r0) -> Pass {
            Pass f;
            const int slot = r0 + sub;
            f.tl = static_cast<int>((static_cast<float>(slot) + 0.5f) * inv_rows);  // exact: slot < 2^20
            const int r = slot - f.tl * rows;
            const int tk = tk0 + f.tl;
            f.valid = slot < slots && tk < tokens;
            const int b = f.valid ? s_tok[2 * f.tl] : 0;
            const int t = f.valid ? s_tok[2 * f.tl + 1] : 0;
            const uint16_t* src = nullptr;
            f.dst = nullptr;
            f.weight = nullptr;
            f.rope = false;
            f.norm = true;
            if (f.valid) {
                if (r < rows_q) {
                    src = f.dst = p.q + b * p.q_stride_b + t * p.q_stride_t + (long long)r * HD;
                    f.weight = p.q_weight;
                    f.rope = true;
                } else if (r < rows_q + rows_k) {
                    const int h = r - rows_q;
                    src = p.k_src + b * p.ks_stride_b + t * p.ks_stride_t + (long long)h * HD;
                    f.dst = p.k_dst + b * p.kd_stride_b + t * p.kd_stride_t + (long long)h * HD;
                    f.weight = p.k_weight;
                    f.rope = true;
                } else {
                    const int h = r - rows_q - rows_k;
                    src = p.v_src ? p.v_src + b * p.vs_stride_b + t * p.vs_stride_t + (long long)h * HD
                                  : p.k_src + b * p.ks_stride_b + t * p.ks_stride_t + (long long)h * HD;
                    f.dst = p.v_dst + b * p.vd_stride_b + t * p.vd_stride_t + (long long)h * HD;
                    f.norm = !(QWEN && p.v_copy);
                }
            }
            f.rl = make_uint4(0u, 0u, 0u, 0u);
            f.rh = f.rl;
            if (f.valid) {
                f.rl = *reinterpret_cast<const uint4*>(src + li * 8);
                f.rh = *reinterpret_cast<const uint4*>(src + HD / 2 + li * 8);
            }
            return f;
        };
        Pass nxt;
        if (AHEAD) nxt = fetch(warp * RPW);
        for (int r0 = warp * RPW; r0 < slots; r0 += 8 * RPW) {
            const Pass cur = AHEAD ? nxt : fetch(r0);
            if (AHEAD && r0 + 8 * RPW < slots) nxt = fetch(r0 + 8 * RPW);
            const bool valid = cur.valid, rope = cur.rope, norm = cur.norm;
            const int tl = cur.tl;
            const uint16_t* weight = cur.weight;
            uint16_t* dst = cur.dst;
            const uint4 rl = cur.rl, rh = cur.rh;
            float lo[8], hi[8];
            unpack8(rl, lo);
            unpack8(rh, hi);
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rms_inv = rsqrtf(ss / static_cast<float>(HD) + p.eps);
            if (!norm) {
                // appended as it is
            } else if (weight) {
                float wl[8], wh[8];
                unpack8(*reinterpret_cast<const uint4*>(weight + li * 8), wl);
                unpack8(*reinterpret_cast<const uint4*>(weight + HD / 2 + li * 8), wh);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    lo[e] = bf16_rne(lo[e] * rms_inv * wl[e]);
                    hi[e] = bf16_rne(hi[e] * rms_inv * wh[e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    lo[e] = bf16_rne(lo[e] * rms_inv);
                    hi[e] = bf16_rne(hi[e] * rms_inv);
                }
            }
            if (QWEN && p.rot_half != HD / 2) {
                // Pairs (f, f + rot_half) both sit in the row's first half, rot_half / 8 lanes apart: the
                // partner's values come by shuffle (every lane takes part; only the rotary lanes update).
                const int dl = p.rot_half >> 3;
                const bool mine = rope && li < 2 * dl;
                const bool first = (li & dl) == 0;
                const float* tc = s_cos + tl * (HD / 2);
                const float* ts = s_sin + tl * (HD / 2);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float other = __shfl_xor_sync(0xffffffffu, lo[e], dl);
                    const int pr = (li & (dl - 1)) * 8 + e;
                    if (mine && pr < p.nap) {
                        const float c = tc[pr], s = ts[pr];
                        lo[e] = first ? lo[e] * c - other * s : other * s + lo[e] * c;
                    }
                }
            } else if (rope) {
                const float* tc = s_cos + tl * (HD / 2);
                const float* ts = s_sin + tl * (HD / 2);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int pr = li * 8 + e;
                    if (pr < p.nap) {
                        const float c = tc[pr], s = ts[pr];
                        const float x0 = lo[e], x1 = hi[e];
                        lo[e] = x0 * c - x1 * s;
                        hi[e] = x0 * s + x1 * c;
                    }
                }
            }
            if (valid) {
                *reinterpret_cast<uint4*>(dst + li * 8) = pack8(lo);
                *reinterpret_cast<uint4*>(dst + HD / 2 + li * 8) = pack8(hi);
            }
        }
    }
}

}  // namespace arc
