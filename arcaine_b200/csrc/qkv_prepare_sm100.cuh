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
// Mapping: one CTA per token at a time (grid-stride), cos / sin of the token staged once in
// shared memory and shared by all its heads (the reference's "Fused" mode), one warp per
// (token, head) row, each lane holding hd/64 elements of the row's first half and the matching
// elements of the second half, so a rotation pair never leaves the lane.
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
};

template <int E> struct RowVec;  // E consecutive bf16
template <> struct RowVec<2> { using type = uint32_t; };
template <> struct RowVec<4> { using type = uint2; };
template <> struct RowVec<8> { using type = uint4; };

template <int E>
__device__ __forceinline__ void unpack_row(const typename RowVec<E>::type& raw, float (&f)[E]) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <int E>
__device__ __forceinline__ typename RowVec<E>::type pack_row(const float (&f)[E]) {
    typename RowVec<E>::type raw;
    uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
    for (int i = 0; i < E / 2; ++i) w[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
    return raw;
}

__device__ __forceinline__ float bf16_rne(float x) {
    return __uint_as_float(static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x))) << 16);
}

// HD = 64 * E.  256 threads: 8 warps, each takes rows (heads of Q, then K, then V) of the token.
template <int E>
__global__ void __launch_bounds__(256) qkv_prepare_kernel(const QkvPrepareParams p) {
    constexpr int HD = 64 * E;
    __shared__ float s_cos[HD / 2];
    __shared__ float s_sin[HD / 2];
    using Vec = typename RowVec<E>::type;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rows_q = p.q ? p.nq : 0;
    const int rows_k = p.k_src && p.k_dst ? p.nkv : 0;
    const int rows_v = p.v_dst ? p.nkv : 0;
    const int rows = rows_q + rows_k + rows_v;
    const long long tokens = (long long)p.batch * p.seq;

    for (long long tk = blockIdx.x; tk < tokens; tk += gridDim.x) {
        const int b = static_cast<int>(tk / p.seq);
        const int t = static_cast<int>(tk - (long long)b * p.seq);
        if (p.nap > 0) {
            __syncthreads();  // the previous token's readers are done
            for (int pr = threadIdx.x; pr < p.nap; pr += blockDim.x) {
                float c, s;
                if (p.rope_cos) {
                    const long long ti = (long long)b * p.rope_stride_b + (long long)t * p.nap + pr;
                    c = p.rope_cos[ti];
                    s = p.rope_sin[ti];
                } else {
                    const int pos = (p.pos_offset ? p.pos_offset[b] : p.pos0) + t;
                    const float inv_freq = 1.0f / powf(p.theta, 2.0f * pr / static_cast<float>(HD));
                    const float angle = static_cast<float>(pos) * inv_freq;
                    c = cosf(angle);
                    s = sinf(angle);
                }
                s_cos[pr] = c;
                s_sin[pr] = s;
            }
            __syncthreads();
        }
        for (int r = warp; r < rows; r += 8) {
            const uint16_t* src;
            uint16_t* dst;
            const uint16_t* weight;
            bool rope;
            if (r < rows_q) {
                src = dst = p.q + b * p.q_stride_b + t * p.q_stride_t + (long long)r * HD;
                weight = p.q_weight;
                rope = true;
            } else if (r < rows_q + rows_k) {
                const int h = r - rows_q;
                src = p.k_src + b * p.ks_stride_b + t * p.ks_stride_t + (long long)h * HD;
                dst = p.k_dst + b * p.kd_stride_b + t * p.kd_stride_t + (long long)h * HD;
                weight = p.k_weight;
                rope = true;
            } else {
                const int h = r - rows_q - rows_k;
                src = p.v_src ? p.v_src + b * p.vs_stride_b + t * p.vs_stride_t + (long long)h * HD
                              : p.k_src + b * p.ks_stride_b + t * p.ks_stride_t + (long long)h * HD;
                dst = p.v_dst + b * p.vd_stride_b + t * p.vd_stride_t + (long long)h * HD;
                weight = nullptr;
                rope = false;
            }
            float lo[E], hi[E];
            unpack_row<E>(*reinterpret_cast<const Vec*>(src + lane * E), lo);
            unpack_row<E>(*reinterpret_cast<const Vec*>(src + HD / 2 + lane * E), hi);
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rms_inv = rsqrtf(ss / static_cast<float>(HD) + p.eps);
            if (weight) {
                float wl[E], wh[E];
                unpack_row<E>(*reinterpret_cast<const Vec*>(weight + lane * E), wl);
                unpack_row<E>(*reinterpret_cast<const Vec*>(weight + HD / 2 + lane * E), wh);
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    lo[e] = bf16_rne(lo[e] * rms_inv * wl[e]);
                    hi[e] = bf16_rne(hi[e] * rms_inv * wh[e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    lo[e] = bf16_rne(lo[e] * rms_inv);
                    hi[e] = bf16_rne(hi[e] * rms_inv);
                }
            }
            if (rope) {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const int pr = lane * E + e;
                    if (pr < p.nap) {
                        const float c = s_cos[pr], s = s_sin[pr];
                        const float x0 = lo[e], x1 = hi[e];
                        lo[e] = x0 * c - x1 * s;
                        hi[e] = x0 * s + x1 * c;
                    }
                }
            }
            *reinterpret_cast<Vec*>(dst + lane * E) = pack_row<E>(lo);
            *reinterpret_cast<Vec*>(dst + HD / 2 + lane * E) = pack_row<E>(hi);
        }
    }
}

}  // namespace arc
