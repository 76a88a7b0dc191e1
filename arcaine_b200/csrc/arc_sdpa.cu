// C ABI of the sm_100a attention library: argument validation, launch plans,
// TMA tensor maps and kernel launches.  Nothing here allocates device memory or
// synchronises a stream (except the explicit status query); scratch is provided
// by the caller and sized by the *_workspace_bytes functions.
#include "../../include/arc_sdpa.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <mutex>

#include "decode_sm100.cuh"
#include "prefill_pair_sm100.cuh"
#include "qkv_prepare_sm100.cuh"
#include "prefill_sm100.cuh"

namespace arc {

// Per-device status word written by kernels whose bounded waits give up.
__device__ uint32_t g_fault_words[2];

constexpr int kMaxDevices = 64;
// The decode kernel keeps a few bytes of static shared memory; the dynamic part
// may use the opt-in maximum minus this reserve.
constexpr int kDecodeStaticSmem = 1024;
// Dynamic shared memory the decode merge kernel may ask for (it is opted in to this much).
constexpr int kMergeSmemOptin = 64 * 1024;

struct DeviceState {
    std::atomic<bool> ready{false};  // set (release) once everything below is written
    uint32_t* fault = nullptr;
    int sm_count = 0;
    int smem_optin = 0;
    // largest cluster size (2, 4 or 8; 0 = none) the cluster form of the prefill kernel can be launched with, per head dim
    // [head dim 128 / 256][log2(cluster size)]: how many clusters of 2 or 4 CTAs of the cluster form of the
    // prefill kernel the device can hold at once (0: that size cannot be launched)
    int active_clusters[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
};

static DeviceState g_dev[kMaxDevices];
static std::mutex g_mu;
static std::atomic<uint64_t> g_launches{0};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

// Text of the most recent failing CUDA call on this thread (for diagnostics).
static thread_local char g_last_error[256] = "";

static int cuda_fail(const char* what, cudaError_t e) {
    std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    cudaGetLastError();
    return ARC_ERR_CUDA;
}

#define ARC_CUDA(call)                                      \
    do {                                                    \
        cudaError_t e_ = (call);                            \
        if (e_ != cudaSuccess) return cuda_fail(#call, e_); \
    } while (0)

template <typename K>
static cudaError_t opt_in_smem(K kernel, int bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// One-time set-up for the current device: status-word address, SM count, and the
// dynamic shared memory opt-in of every kernel.
static int device_state(DeviceState** out) {
    int dev = 0;
    ARC_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return ARC_ERR_CUDA;
    DeviceState& s = g_dev[dev];
    if (!s.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!s.ready.load(std::memory_order_relaxed)) {
            void* sym = nullptr;
            ARC_CUDA(cudaGetSymbolAddress(&sym, g_fault_words));
            s.fault = static_cast<uint32_t*>(sym);
            ARC_CUDA(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
            ARC_CUDA(cudaDeviceGetAttribute(&s.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
            if (!g_encode) {
                void* fn = nullptr;
                cudaDriverEntryPointQueryResult qres = cudaDriverEntryPointSymbolNotFound;
                ARC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
                if (qres != cudaDriverEntryPointSuccess || fn == nullptr) {
                    std::snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled not found in the driver");
                    return ARC_ERR_CUDA;
                }
                g_encode = reinterpret_cast<EncodeTiledFn>(fn);
            }
            ARC_CUDA(opt_in_smem(sdpa_prefill_pair_kernel<false, false>, PairCfg::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_pair_kernel<true, false>, PairCfg::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_pair_kernel<false, true>, PairCfg::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_pair_kernel<true, true>, PairCfg::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<128, false, false>, PrefillCfg<128>::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<128, false, true>, PrefillCfg<128>::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<128, true, true>, PrefillCfg<128>::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<256, false, false>, PrefillCfg<256>::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<256, false, true>, PrefillCfg<256>::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<256, true, true>, PrefillCfg<256>::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<128, false, false, true>, PrefillCfg<128>::SMEM_BYTES));
            ARC_CUDA(opt_in_smem(sdpa_prefill_kernel<256, false, false, true>, PrefillCfg<256>::SMEM_BYTES));
            for (int hi = 0; hi < 2; ++hi) {
                for (int cs = 2, lg = 1; cs <= 4; cs *= 2, ++lg) {
                    cudaLaunchConfig_t cfg{};
                    cfg.gridDim = dim3((unsigned)(s.sm_count / cs * cs));  // the answer is capped by the grid asked about
                    cfg.blockDim = dim3(hi ? PrefillCfg<256>::THREADS : PrefillCfg<128>::THREADS);
                    cfg.dynamicSmemBytes = hi ? PrefillCfg<256>::SMEM_BYTES : PrefillCfg<128>::SMEM_BYTES;
                    cudaLaunchAttribute attr[1];
                    attr[0].id = cudaLaunchAttributeClusterDimension;
                    attr[0].val.clusterDim.x = (unsigned)cs;
                    attr[0].val.clusterDim.y = 1;
                    attr[0].val.clusterDim.z = 1;
                    cfg.attrs = attr;
                    cfg.numAttrs = 1;
                    int n = 0;
                    const cudaError_t e = hi ? cudaOccupancyMaxActiveClusters(&n, sdpa_prefill_kernel<256, false, false, true>, &cfg)
                                             : cudaOccupancyMaxActiveClusters(&n, sdpa_prefill_kernel<128, false, false, true>, &cfg);
                    if (e == cudaSuccess && n > 0) s.active_clusters[hi][lg] = n;
                    else cudaGetLastError();
                }
            }
            ARC_CUDA(opt_in_smem(sdpa_decode_kernel<128, 1>, s.smem_optin - kDecodeStaticSmem));
            ARC_CUDA(opt_in_smem(sdpa_decode_kernel<128, 2>, s.smem_optin - kDecodeStaticSmem));
            ARC_CUDA(opt_in_smem(sdpa_decode_kernel<256, 1>, s.smem_optin - kDecodeStaticSmem));
            ARC_CUDA(opt_in_smem(sdpa_decode_kernel<256, 2>, s.smem_optin - kDecodeStaticSmem));
            ARC_CUDA(opt_in_smem(sdpa_decode_merge_kernel<128, false>, kMergeSmemOptin));
            ARC_CUDA(opt_in_smem(sdpa_decode_merge_kernel<256, false>, kMergeSmemOptin));
            ARC_CUDA(opt_in_smem(sdpa_decode_merge_kernel<128, true>, kMergeSmemOptin));
            ARC_CUDA(opt_in_smem(sdpa_decode_merge_kernel<256, true>, kMergeSmemOptin));
            s.ready.store(true, std::memory_order_release);
        }
    }
    *out = &s;
    return ARC_OK;
}

// Launch `kernel` behind the previous kernel of `stream` with programmatic serialization: its CTAs
// may be scheduled and run up to their grid_dependency_wait() while that kernel is still running,
// which takes the launch latency of a small follow-up kernel (a merge) off the critical path.
template <typename... KArgs, typename... Args>
static cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// (hd, heads, tokens, batch) view of a token-major bf16 tensor; box = 64 x 1 x 128 x 1, 128-byte swizzle.
static int make_tile_map(CUtensorMap* tm, const void* base, int hd, int heads, int tokens, int batch,
                         int64_t stride_t, int64_t stride_b) {
    cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)tokens, (cuuint64_t)batch};
    cuuint64_t sb = (cuuint64_t)(batch > 1 ? stride_b : stride_t * (int64_t)tokens) * 2u;
    cuuint64_t strides[3] = {(cuuint64_t)hd * 2u, (cuuint64_t)stride_t * 2u, sb};
    cuuint32_t box[4] = {64u, 1u, 128u, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        std::snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return ARC_ERR_CUDA;
    }
    return ARC_OK;
}

// (nkv*hd, rows) view of a KV cache whose rows are `stride_t` elements apart;
// box = 64 columns x `box_rows` rows, 128-byte swizzle; rows past `rows` read as zero.
static int make_cache_map(CUtensorMap* tm, const void* base, int row_elems, int64_t rows, int64_t stride_t,
                          int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)row_elems, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)stride_t * 2u};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        std::snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled (cache) failed with CUresult %d", (int)r);
        return ARC_ERR_CUDA;
    }
    return ARC_OK;
}

// ---------------------------------------------------------------------------
// Prefill plan
// ---------------------------------------------------------------------------
struct PrefillPlan {
    int q_tiles = 0;
    int splits = 1;
    int cluster = 0;         // > 0: the splits are the CTAs of a thread-block cluster of this size, folded in the kernel
    long long rows = 0;
    size_t split_bytes = 0;  // partial records of key-range splits, at the start of the workspace
    size_t ws_bytes = 0;     // all of the workspace: partial records, then the per-row span ends of block_ids
};

static int plan_prefill(const arc_sdpa_prefill_params* p, int sm_count, const int* active_clusters, PrefillPlan* plan) {
    if (!p) return ARC_ERR_NULL_POINTER;
    if (p->batch <= 0 || p->seq <= 0 || p->kv_len <= 0 || p->nq <= 0 || p->nkv <= 0 || p->nq % p->nkv != 0)
        return ARC_ERR_BAD_SHAPE;
    if (p->hd != 128 && p->hd != 256) return ARC_ERR_UNSUPPORTED_HEAD_DIM;
    if (!(p->scale > 0.f) || !std::isfinite(p->scale)) return ARC_ERR_BAD_SHAPE;
    if (p->mask_type != ARC_MASK_NONE && p->mask_type != ARC_MASK_EXPLICIT && p->mask_type != ARC_MASK_CAUSAL)
        return ARC_ERR_BAD_SHAPE;
    if (p->num_splits < 0) return ARC_ERR_BAD_SHAPE;
    plan->q_tiles = (p->seq + 127) / 128;
    plan->rows = (long long)p->batch * p->seq * p->nq;
    const int kv_blocks = (p->kv_len + 127) / 128;
    int splits = p->num_splits;
    const long long tiles = (long long)plan->q_tiles * p->nq * p->batch;
    if (splits == 0) {
        // Split the key range only when the tiles alone leave most SMs idle and there are enough key blocks
        // to pay for folding the parts again (measured: about 8 us for the fold against 1.3-2 us per key
        // block; with fewer than ten blocks a tile is faster in one piece, and more than eight parts cost
        // more than they save).
        splits = 1;
        if (tiles * 2 <= sm_count && kv_blocks >= 10) {
            splits = (int)(sm_count / tiles);
            if (splits > kv_blocks / 2) splits = kv_blocks / 2;
            if (splits > 8) splits = 8;
            if (splits < 1) splits = 1;
        }
    }
    if (splits > kv_blocks) splits = kv_blocks;
    if (splits > 64) splits = 64;
    // A split the library chose itself is run as a thread-block cluster where the device allows it: the
    // CTAs of a tile fold their accumulators through distributed shared memory in the same launch, no
    // partial records, no merge kernel, no workspace.  An explicit num_splits keeps the two-launch form.
    // All tiles' clusters must be resident at once (clusters are placed inside one GPC each, so fewer fit
    // than SMs / size suggests; a second wave would double the time).  Head dim 256 only: at head dim 128 the two-launch form measured
    // 5-7 us faster (the cluster instance of that kernel does not fit its register budget without spills).
    if (p->num_splits == 0 && (splits == 2 || splits == 4) && p->hd == 256 && active_clusters &&
        p->mask_type != ARC_MASK_EXPLICIT) {
        // (two or four parts: with eight, a CTA reads seven eighths of its rows from the others and the
        // two-launch form measured 2-3 us faster; three parts would have to become two)
        const int lg = splits == 2 ? 1 : 2;
        if (active_clusters[lg] >= tiles) {
            plan->cluster = splits;
            splits = 1;
        }
    }
    plan->splits = splits;
    plan->split_bytes = splits > 1 ? (size_t)splits * plan->rows * ((size_t)p->hd + 1) * sizeof(float) : 0;
    plan->split_bytes = (plan->split_bytes + 15) & ~(size_t)15;
    plan->ws_bytes = plan->split_bytes;
    if (p->block_ids) {
        if (p->mask_type != ARC_MASK_CAUSAL || p->block_ids_offset < 0) return ARC_ERR_BAD_SHAPE;
        plan->ws_bytes += ((size_t)p->seq * sizeof(int32_t) + 15) & ~(size_t)15;
    }
    return ARC_OK;
}

template <int HD>
static int launch_prefill(const arc_sdpa_prefill_params* p, const PrefillPlan& plan, DeviceState* ds,
                          cudaStream_t stream) {
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tile_map(&tq, p->q, HD, p->nq, p->seq, p->batch, p->q_stride_t, p->q_stride_b)) != ARC_OK) return rc;
    if ((rc = make_tile_map(&tk, p->k, HD, p->nkv, p->kv_len, p->batch, p->k_stride_t, p->k_stride_b)) != ARC_OK) return rc;
    if ((rc = make_tile_map(&tv, p->v, HD, p->nkv, p->kv_len, p->batch, p->v_stride_t, p->v_stride_b)) != ARC_OK) return rc;

    PrefillParams kp{};
    kp.out = static_cast<uint16_t*>(p->out);
    kp.out_copies = reinterpret_cast<const unsigned long long*>(p->out_copies);
    kp.n_copies = p->out_copies ? p->out_copy_count : 0;
    kp.gate = static_cast<const uint16_t*>(p->gate);
    kp.mask = p->mask_type == ARC_MASK_EXPLICIT ? p->mask : nullptr;
    kp.out_lse = p->out_lse;
    kp.part_o = plan.splits > 1 ? static_cast<float*>(p->workspace) : nullptr;
    kp.part_lse = kp.part_o ? kp.part_o + (size_t)plan.splits * plan.rows * HD : nullptr;
    if (p->block_ids) {
        // span ends per query row, once per call: a few microseconds instead of a (seq, kv_len) f32 mask
        int* vis = reinterpret_cast<int*>(static_cast<unsigned char*>(p->workspace) + plan.split_bytes);
        vision_span_kernel<<<(unsigned)((p->seq + 255) / 256), 256, 0, stream>>>(p->block_ids, p->block_ids_offset,
                                                                               p->kv_len - p->seq, p->seq, p->kv_len, vis);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        ARC_CUDA(cudaGetLastError());
        kp.vis_hi = vis;
    }
    kp.fault = ds->fault;
    kp.batch = p->batch;
    kp.seq = p->seq;
    kp.kv_len = p->kv_len;
    kp.nq = p->nq;
    kp.nkv = p->nkv;
    kp.o_stride_b = p->o_stride_b;
    kp.o_stride_t = p->o_stride_t;
    kp.scale_log2 = p->scale * 1.4426950408889634f;
    kp.mask_type = p->mask_type;
    kp.window = p->window;
    kp.num_splits = plan.splits;
    kp.group = p->nq / p->nkv;
    kp.group_shift = -1;
    kp.tail_base = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == kp.group) kp.group_shift = sh;

    // Head dim 128: two query tiles per CTA (prefill_pair_sm100.cuh) when that is the faster way to cover
    // the tiles.  ARC_SDPA_PREFILL_KERNEL=single|pair overrides the choice (for A/B measurements).
    if (HD == 128 && plan.splits == 1 && plan.cluster == 0 && !(kp.mask_type == 1 && kp.mask != nullptr) && kp.vis_hi == nullptr) {
        static const int forced = [] {
            const char* e = std::getenv("ARC_SDPA_PREFILL_KERNEL");
            if (!e) return 0;
            return std::strcmp(e, "pair") == 0 ? 2 : (std::strcmp(e, "single") == 0 ? 1 : 0);
        }();
        // A CTA takes two 128-row tiles: the same tokens of two heads of one KV group when the group
        // size is even (both tiles then see exactly the same key blocks), else 256 tokens of one head.
        const bool head_pair = ((p->nq / p->nkv) & 1) == 0;
        const long long pair_tiles = head_pair ? (long long)plan.q_tiles * (p->nq / 2) * p->batch
                                               : (long long)((p->seq + 255) / 256) * p->nq * p->batch;
        // Measured: a pair of tiles costs 1.7 single tiles.  Tiles come in waves of one per SM, so the
        // kernel with the cheaper whole number of waves wins (512 pair tiles on 148 SMs are 4 waves,
        // the same rows as 1024 single tiles are 7: the single-tile kernel is then faster).
        const long long single_tiles = (long long)plan.q_tiles * p->nq * p->batch;
        const long long sms = ds->sm_count;
        // The pairs left over after the last whole wave of CTAs are cut into their two heads when every SM then
        // gets at most one of them: a second launch (the one-tile kernel, one CTA per tile, scheduled behind this
        // one as SMs free up) takes them, and no SM runs a whole pair while the others idle.  A single tile
        // costs about one tile of the one-tile kernel.
        const long long full_waves = pair_tiles / sms, left = pair_tiles - full_waves * sms;
        const bool cut_tail = head_pair && full_waves > 0 && left > 0 && 2 * left <= sms;
        const double cost_pair = cut_tail ? 1.7 * (double)full_waves + 1.05 : 1.7 * (double)((pair_tiles + sms - 1) / sms);
        const double cost_single = (double)((single_tiles + sms - 1) / sms);
        const bool use_pair = forced == 2 || (forced == 0 && cost_pair <= cost_single);
        if (use_pair) {
            if (pair_tiles > 0x7fffffffLL) return ARC_ERR_TOO_LARGE;
            kp.head_pair = head_pair ? 1 : 0;
            kp.cur_heads = head_pair ? p->nq / 2 : p->nq;
            kp.q_tiles = head_pair ? plan.q_tiles : (p->seq + 255) / 256;
            const long long pair_units = cut_tail ? full_waves * sms : pair_tiles;
            kp.total_tiles = (int)pair_units;
            const unsigned ctas = (unsigned)(pair_units < ds->sm_count ? pair_units : ds->sm_count);
            if (kp.n_copies > 0) {
                if (kp.gate) sdpa_prefill_pair_kernel<true, true><<<ctas, PairCfg::THREADS, PairCfg::SMEM_BYTES, stream>>>(tq, tk, tv, kp);
                else sdpa_prefill_pair_kernel<false, true><<<ctas, PairCfg::THREADS, PairCfg::SMEM_BYTES, stream>>>(tq, tk, tv, kp);
            } else if (kp.gate) {
                sdpa_prefill_pair_kernel<true, false><<<ctas, PairCfg::THREADS, PairCfg::SMEM_BYTES, stream>>>(tq, tk, tv, kp);
            } else {
                sdpa_prefill_pair_kernel<false, false><<<ctas, PairCfg::THREADS, PairCfg::SMEM_BYTES, stream>>>(tq, tk, tv, kp);
            }
            g_launches.fetch_add(1, std::memory_order_relaxed);
            ARC_CUDA(cudaGetLastError());
            if (cut_tail) {
                PrefillParams tp = kp;
                tp.head_pair = 0;
                tp.cur_heads = p->nq;
                tp.q_tiles = plan.q_tiles;
                tp.tail_base = (int)pair_units;
                tp.total_tiles = (int)(2 * left);
                tp.num_splits = 1;
                const dim3 grid((unsigned)(2 * left)), block(PrefillCfg<128>::THREADS);
                if (tp.gate)
                    ARC_CUDA(launch_dependent(sdpa_prefill_kernel<128, false, true>, grid, block, (size_t)PrefillCfg<128>::SMEM_BYTES, stream, tq, tk, tv, tp));
                else
                    ARC_CUDA(launch_dependent(sdpa_prefill_kernel<128, false, false>, grid, block, (size_t)PrefillCfg<128>::SMEM_BYTES, stream, tq, tk, tv, tp));
                g_launches.fetch_add(1, std::memory_order_relaxed);
            }
            return ARC_OK;
        }
    }

    kp.q_tiles = plan.q_tiles;
    kp.cur_heads = p->nq;
    kp.head_pair = 0;
    if (plan.cluster > 0) {
        // Few tiles: the key range of every tile is split over the CTAs of a thread-block cluster, which
        // fold their accumulators through distributed shared memory — one launch, nothing in global memory
        // but the result.  Clusters walk the tile list together.
        const long long tiles = (long long)plan.q_tiles * p->nq * p->batch;
        if (tiles > 0x7fffffffLL) return ARC_ERR_TOO_LARGE;
        kp.total_tiles = (int)tiles;
        kp.num_splits = 1;
        const long long nclusters = tiles;  // the plan made sure that many are resident at once
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)(nclusters * plan.cluster));
        cfg.blockDim = dim3(PrefillCfg<HD>::THREADS);
        cfg.dynamicSmemBytes = PrefillCfg<HD>::SMEM_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)plan.cluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        ARC_CUDA(cudaLaunchKernelEx(&cfg, sdpa_prefill_kernel<HD, false, false, true>, tq, tk, tv, kp));
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return ARC_OK;
    }
    // Persistent grid: one CTA per SM (fewer if there are fewer tiles), tiles dealt round-robin.
    const long long total_tiles = (long long)plan.q_tiles * p->nq * p->batch * plan.splits;
    if (total_tiles > 0x7fffffffLL) return ARC_ERR_TOO_LARGE;
    kp.total_tiles = (int)total_tiles;
    const unsigned ctas = (unsigned)(total_tiles < ds->sm_count ? total_tiles : ds->sm_count);
    // The additive-mask form is a kernel of its own: the common one stays small.
    if (kp.mask_type == 1 && kp.mask != nullptr)
        sdpa_prefill_kernel<HD, true, true><<<ctas, PrefillCfg<HD>::THREADS, PrefillCfg<HD>::SMEM_BYTES, stream>>>(tq, tk, tv, kp);
    else if (kp.gate && plan.splits == 1)
        sdpa_prefill_kernel<HD, false, true><<<ctas, PrefillCfg<HD>::THREADS, PrefillCfg<HD>::SMEM_BYTES, stream>>>(tq, tk, tv, kp);
    else
        sdpa_prefill_kernel<HD, false, false><<<ctas, PrefillCfg<HD>::THREADS, PrefillCfg<HD>::SMEM_BYTES, stream>>>(tq, tk, tv, kp);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    ARC_CUDA(cudaGetLastError());

    if (plan.splits > 1) {
        UniformMergeParams mp{};
        mp.part_o = kp.part_o;
        mp.part_lse = kp.part_lse;
        mp.gate = kp.gate;
        mp.out = kp.out;
        mp.out_f32 = nullptr;
        mp.out_lse = p->out_lse;
        mp.rows = plan.rows;
        mp.num_parts = plan.splits;
        mp.o_part_stride = plan.rows * HD;
        mp.lse_part_stride = plan.rows;
        mp.seq = p->seq;
        mp.nq = p->nq;
        mp.o_stride_b = p->o_stride_b;
        mp.o_stride_t = p->o_stride_t;
        mp.out_copies = kp.out_copies;
        mp.n_copies = kp.n_copies;
        ARC_CUDA(launch_dependent(sdpa_uniform_merge_kernel<HD>, dim3((unsigned)((plan.rows + UMERGE_ROWS - 1) / UMERGE_ROWS)),
                                  dim3(32 * UMERGE_ROWS), 0, stream, mp));
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return ARC_OK;
}

// ---------------------------------------------------------------------------
// Decode plan
// ---------------------------------------------------------------------------
struct DecodePlan {
    int nkv_cta = 1, groups = 1, slices = 1, stages = 2, ncta = 1, nt = 1;
    int smem_bytes = 0;
    long long parts = 0;
    size_t ws_bytes = 0;
    size_t merge_smem = 0;
};

static int plan_decode(const arc_sdpa_decode_params* p, int sm_count, int smem_optin, DecodePlan* plan) {
    if (!p) return ARC_ERR_NULL_POINTER;
    if (p->batch <= 0 || p->nq <= 0 || p->nkv <= 0 || p->nq % p->nkv != 0) return ARC_ERR_BAD_SHAPE;
    if (p->batch > DECODE_MAX_BATCH) return ARC_ERR_TOO_LARGE;
    if (p->hd != 128 && p->hd != 256) return ARC_ERR_UNSUPPORTED_HEAD_DIM;
    if (!(p->scale > 0.f) || !std::isfinite(p->scale)) return ARC_ERR_BAD_SHAPE;
    if (!p->kv_len && p->kv_len_uniform < 0) return ARC_ERR_BAD_SHAPE;
    if (p->kv_rows_total < 0 || p->kv_rows_total > 0x7fffffffLL) return ARC_ERR_BAD_SHAPE;
    // An empty cache (a sequence-sharded rank whose slice holds no keys) is fine as long as the
    // host-side length says so too.
    if (p->kv_rows_total == 0 && (p->kv_len || p->kv_len_uniform != 0)) return ARC_ERR_BAD_SHAPE;
    if (p->max_kv_len < 0) return ARC_ERR_BAD_SHAPE;
    if (p->max_kv_len > 0 && !p->kv_len && p->kv_len_uniform > p->max_kv_len) return ARC_ERR_BAD_SHAPE;
    if (!p->kv_len && !p->kv_row_offset && p->kv_len_uniform > 0 &&
        (int64_t)(p->batch - 1) * p->kv_stride_b + p->kv_len_uniform > p->kv_rows_total)
        return ARC_ERR_BAD_SHAPE;  // everything is known on the host: refuse at once
    const int G = p->nq / p->nkv;
    if (G > 16) return ARC_ERR_UNSUPPORTED_GQA;
    plan->nt = G > 8 ? 2 : 1;
    // Heads per CTA: the largest divisor of nkv whose row (all its heads) is <= 2 KB.
    const int max_heads = 1024 / p->hd;  // 8 for hd 128, 4 for hd 256
    int nkv_cta = 1;
    for (int c = 1; c <= p->nkv && c <= max_heads; ++c)
        if (p->nkv % c == 0) nkv_cta = c;
    plan->nkv_cta = nkv_cta;
    plan->groups = p->nkv / nkv_cta;
    const int row_bytes = nkv_cta * p->hd * 2;
    int slices = (64 * 1024) / (32 * row_bytes);
    if (slices > 8 / nkv_cta) slices = 8 / nkv_cta;
    if (slices < 1) slices = 1;
    plan->slices = slices;
    const int stage_bytes = 2 * 16 * slices * row_bytes;
    const int fixed = 1024 + 2 * 8 * 8 + (p->batch + 2) * 8;
    int stages = (smem_optin - kDecodeStaticSmem - fixed) / stage_bytes;
    if (stages > 4) stages = 4;
    if (stages < 2) return ARC_ERR_TOO_LARGE;
    plan->stages = stages;
    plan->smem_bytes = stages * stage_bytes + fixed;
    int ncta = p->num_ctas > 0 ? p->num_ctas : sm_count / plan->groups;
    if (ncta < 1) ncta = 1;
    if (ncta > 1024) ncta = 1024;
    plan->ncta = ncta;
    plan->parts = ((long long)ncta + p->batch) * slices;
    plan->ws_bytes = (size_t)plan->parts * p->nq * ((size_t)p->hd + 1) * sizeof(float);
    // the merge kernel keeps the length prefix, a row of partial sums per warp and one weight plus one
    // list entry per record of a sequence (at most ncta + 1 shares) in shared memory
    plan->merge_smem = (size_t)(p->batch + 2) * 8 + 8 * sizeof(float) + (size_t)(MERGE_THREADS / 32) * p->hd * sizeof(float) +
                       (size_t)(ncta + 1) * slices * (sizeof(float) + sizeof(int));
    if (plan->merge_smem > (size_t)kMergeSmemOptin) return ARC_ERR_TOO_LARGE;
    return ARC_OK;
}

template <int HD>
static int launch_decode(const arc_sdpa_decode_params* p, const DecodePlan& plan, DeviceState* ds,
                         cudaStream_t stream) {
    CUtensorMap tk, tv;
    int rc;
    const bool empty_cache = p->kv_rows_total == 0;  // nothing to read: only the merge runs (all records empty)
    if (!empty_cache) {
        if ((rc = make_cache_map(&tk, p->k, p->nkv * HD, p->kv_rows_total, p->kv_stride_t, 16 * plan.slices)) != ARC_OK) return rc;
        if ((rc = make_cache_map(&tv, p->v, p->nkv * HD, p->kv_rows_total, p->kv_stride_t, 16 * plan.slices)) != ARC_OK) return rc;
    }
    DecodeParams kp{};
    kp.q = static_cast<const uint16_t*>(p->q);
    kp.kv_len = p->kv_len;
    kp.kv_row_offset = reinterpret_cast<const long long*>(p->kv_row_offset);
    kp.part_o = static_cast<float*>(p->workspace);
    kp.part_lse = kp.part_o + (size_t)plan.parts * p->nq * HD;
    kp.fault = ds->fault;
    kp.batch = p->batch;
    kp.nq = p->nq;
    kp.nkv = p->nkv;
    kp.kv_len_uniform = p->kv_len_uniform;
    kp.q_stride_b = p->q_stride_b;
    kp.kv_stride_b = p->kv_stride_b;
    kp.kv_stride_t = p->kv_stride_t;
    kp.scale_log2 = p->scale * 1.4426950408889634f;
    kp.nkv_cta = plan.nkv_cta;
    kp.slices = plan.slices;
    kp.stages = plan.stages;
    kp.ncta = plan.ncta;
    kp.max_kv_len = p->max_kv_len;
    kp.kv_rows_total = p->kv_rows_total;

    dim3 grid((unsigned)plan.ncta, (unsigned)plan.groups, 1);
    const unsigned threads = 32u * (unsigned)(plan.nkv_cta * plan.slices + 1);
    if (!empty_cache) {
        if (plan.nt == 1)
            sdpa_decode_kernel<HD, 1><<<grid, threads, plan.smem_bytes, stream>>>(tk, tv, kp);
        else
            sdpa_decode_kernel<HD, 2><<<grid, threads, plan.smem_bytes, stream>>>(tk, tv, kp);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        ARC_CUDA(cudaGetLastError());
    }

    DecodeMergeParams mp{};
    mp.part_o = kp.part_o;
    mp.part_lse = kp.part_lse;
    mp.kv_len = p->kv_len;
    mp.gate = static_cast<const uint16_t*>(p->gate);
    mp.out = static_cast<uint16_t*>(p->out);
    mp.out_f32 = p->out_f32;
    mp.out_lse = p->out_lse;
    mp.batch = p->batch;
    mp.nq = p->nq;
    mp.kv_len_uniform = p->kv_len_uniform;
    mp.ncta = plan.ncta;
    mp.slices = plan.slices;
    mp.o_stride_b = p->o_stride_b;
    mp.x_peers = reinterpret_cast<const unsigned long long*>(p->xchg_peers);
    mp.x_world = p->xchg_world;
    mp.x_rank = p->xchg_rank;
    mp.x_step = p->xchg_step;
    mp.x_wait_cycles = p->xchg_wait_cycles > 0 ? p->xchg_wait_cycles : 2000000000LL;
    mp.fault = ds->fault;
    dim3 mgrid((unsigned)p->nq, (unsigned)p->batch, 1);
    const bool xchg = mp.x_world > 1;
    if (empty_cache) {
        if (xchg) sdpa_decode_merge_kernel<HD, true><<<mgrid, MERGE_THREADS, plan.merge_smem, stream>>>(mp);
        else sdpa_decode_merge_kernel<HD, false><<<mgrid, MERGE_THREADS, plan.merge_smem, stream>>>(mp);
        ARC_CUDA(cudaGetLastError());
    } else if (xchg) {
        ARC_CUDA(launch_dependent(sdpa_decode_merge_kernel<HD, true>, mgrid, dim3(MERGE_THREADS), plan.merge_smem, stream, mp));
    } else {
        ARC_CUDA(launch_dependent(sdpa_decode_merge_kernel<HD, false>, mgrid, dim3(MERGE_THREADS), plan.merge_smem, stream, mp));
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return ARC_OK;
}

}  // namespace arc

// ===========================================================================
// extern "C"
// ===========================================================================
using namespace arc;

extern "C" const char* arc_sdpa_status_string(int status) {
    switch (status) {
        case ARC_OK: return "ok";
        case ARC_ERR_BAD_SHAPE: return "bad shape or parameter";
        case ARC_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
        case ARC_ERR_UNSUPPORTED_HEAD_DIM: return "head_dim must be 128 or 256";
        case ARC_ERR_WORKSPACE_TOO_SMALL: return "workspace missing or too small";
        case ARC_ERR_CUDA: return "CUDA call failed";
        case ARC_ERR_COLLECTIVE: return "collective failed";
        case ARC_ERR_DEVICE_WAIT_TIMEOUT: return "a bounded device-side wait gave up";
        case ARC_ERR_NULL_POINTER: return "required pointer is null";
        case ARC_ERR_UNSUPPORTED_GQA: return "more than 16 query heads per KV head";
        case ARC_ERR_TOO_LARGE: return "size beyond a fixed limit";
        case ARC_ERR_DEVICE_BAD_RANGE: return "a device-side kv_len or kv_row_offset reaches past the cache";
        default: return "unknown status";
    }
}

extern "C" size_t arc_sdpa_prefill_workspace_bytes(const arc_sdpa_prefill_params* p) {
    DeviceState* ds = nullptr;
    int sm = 148;
    if (device_state(&ds) == ARC_OK) sm = ds->sm_count;
    PrefillPlan plan;
    if (plan_prefill(p, sm, ds ? ds->active_clusters[p && p->hd == 256 ? 1 : 0] : nullptr, &plan) != ARC_OK) return 0;
    return plan.ws_bytes;
}

extern "C" int arc_sdpa_prefill(const arc_sdpa_prefill_params* p, void* stream) {
    if (!p) return ARC_ERR_NULL_POINTER;
    if (!p->q || !p->k || !p->v || !p->out) return ARC_ERR_NULL_POINTER;
    if (p->mask_type == ARC_MASK_EXPLICIT && !p->mask) return ARC_ERR_NULL_POINTER;
    if (p->out_copy_count < 0 || p->out_copy_count > 15 || (p->out_copy_count > 0 && !p->out_copies)) return ARC_ERR_BAD_SHAPE;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc != ARC_OK) return rc;
    PrefillPlan plan;
    if ((rc = plan_prefill(p, ds->sm_count, ds->active_clusters[p->hd == 256 ? 1 : 0], &plan)) != ARC_OK) return rc;
    if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out) ||
        (p->gate && !aligned16(p->gate)))
        return ARC_ERR_ALIGNMENT;
    const int64_t strides[8] = {p->q_stride_b, p->q_stride_t, p->k_stride_b, p->k_stride_t,
                                p->v_stride_b, p->v_stride_t, p->o_stride_b, p->o_stride_t};
    for (int64_t s : strides)
        if (s < 0 || (s & 7) != 0) return ARC_ERR_ALIGNMENT;
    if (p->q_stride_t < (int64_t)p->nq * p->hd || p->o_stride_t < (int64_t)p->nq * p->hd ||
        p->k_stride_t < (int64_t)p->nkv * p->hd || p->v_stride_t < (int64_t)p->nkv * p->hd)
        return ARC_ERR_BAD_SHAPE;
    if (plan.ws_bytes > 0) {
        if (!p->workspace || p->workspace_bytes < plan.ws_bytes) return ARC_ERR_WORKSPACE_TOO_SMALL;
        if (!aligned16(p->workspace)) return ARC_ERR_ALIGNMENT;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return p->hd == 128 ? launch_prefill<128>(p, plan, ds, st) : launch_prefill<256>(p, plan, ds, st);
}

extern "C" size_t arc_sdpa_decode_workspace_bytes(const arc_sdpa_decode_params* p) {
    DeviceState* ds = nullptr;
    if (device_state(&ds) != ARC_OK) return 0;
    DecodePlan plan;
    if (plan_decode(p, ds->sm_count, ds->smem_optin, &plan) != ARC_OK) return 0;
    return plan.ws_bytes;
}

extern "C" size_t arc_sdpa_exchange_bytes(int32_t world, int32_t batch, int32_t nq, int32_t hd) {
    if (world <= 0 || batch <= 0 || nq <= 0 || hd <= 0) return 0;
    return xchg_total_bytes(world, (long long)batch * nq, hd);
}

extern "C" int arc_sdpa_decode(const arc_sdpa_decode_params* p, void* stream) {
    if (!p) return ARC_ERR_NULL_POINTER;
    if (!p->q || ((!p->k || !p->v) && p->kv_rows_total != 0)) return ARC_ERR_NULL_POINTER;
    if (!p->out && !p->out_f32) return ARC_ERR_NULL_POINTER;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc != ARC_OK) return rc;
    DecodePlan plan;
    if ((rc = plan_decode(p, ds->sm_count, ds->smem_optin, &plan)) != ARC_OK) return rc;
    if (!aligned16(p->q) || (p->kv_rows_total != 0 && (!aligned16(p->k) || !aligned16(p->v))) || (p->out && !aligned16(p->out)) ||
        (p->gate && !aligned16(p->gate)) || (p->out_f32 && !aligned16(p->out_f32)))
        return ARC_ERR_ALIGNMENT;
    if ((p->q_stride_b & 7) || (p->o_stride_b & 7) || (p->kv_stride_t & 7) || p->kv_stride_t < (int64_t)p->nkv * p->hd ||
        p->q_stride_b < 0 || p->o_stride_b < 0 || p->kv_stride_b < 0)
        return ARC_ERR_ALIGNMENT;
    if (p->gate && !p->out) return ARC_ERR_NULL_POINTER;
    if (p->xchg_world > 1) {
        if (!p->xchg_peers || !p->out) return ARC_ERR_NULL_POINTER;
        if (p->xchg_rank < 0 || p->xchg_rank >= p->xchg_world || p->xchg_world > XCHG_MAX_WORLD) return ARC_ERR_BAD_SHAPE;
    }
    if (!p->workspace || p->workspace_bytes < plan.ws_bytes) return ARC_ERR_WORKSPACE_TOO_SMALL;
    if (!aligned16(p->workspace)) return ARC_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return p->hd == 128 ? launch_decode<128>(p, plan, ds, st) : launch_decode<256>(p, plan, ds, st);
}

// ---------------------------------------------------------------------------
// Decode without any caller-provided or allocated scratch.
//
// Some callers have nowhere to get a workspace from: a serving process whose
// memory planner has already handed every free byte of the GPU to its own arena
// (Arcaine's per-GPU arena works that way), or a thin foreign-function caller
// that owns no device allocator at all; and cudaMalloc on a decode loop would
// also stall the whole device.  For them the split-KV partial records live in
// the fixed array below, which is part of the library image: every GPU that
// loads the library carries these 8 MiB until the process exits.
//
// In host code the array's name is only a handle; the device address is looked
// up once per device (with that device current) and that address is what the
// kernels receive.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[ARC_STATIC_SCRATCH_BYTES];
static std::atomic<void*> g_static_scratch_addr[arc::kMaxDevices];

static int static_scratch_address(void** out) {
    int dev = 0;
    ARC_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= arc::kMaxDevices) return ARC_ERR_CUDA;
    void* ptr = g_static_scratch_addr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        std::lock_guard<std::mutex> lock(arc::g_mu);
        ptr = g_static_scratch_addr[dev].load(std::memory_order_relaxed);
        if (ptr == nullptr) {
            ARC_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
            g_static_scratch_addr[dev].store(ptr, std::memory_order_release);
        }
    }
    *out = ptr;
    return ARC_OK;
}

extern "C" int arc_sdpa_decode_static(const arc_sdpa_decode_params* p, void* stream) {
    if (!p) return ARC_ERR_NULL_POINTER;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != ARC_OK) return rc;
    arc_sdpa_decode_params q = *p;
    q.workspace = nullptr;
    q.workspace_bytes = 0;
    const size_t need = arc_sdpa_decode_workspace_bytes(&q);
    if (need > (size_t)ARC_STATIC_SCRATCH_BYTES) {
        std::snprintf(g_last_error, sizeof(g_last_error),
                      "arc_sdpa_decode_static: this shape needs %zu bytes of scratch, the built-in array holds %zu",
                      need, (size_t)ARC_STATIC_SCRATCH_BYTES);
        return ARC_ERR_TOO_LARGE;
    }
    q.workspace = scratch;
    q.workspace_bytes = ARC_STATIC_SCRATCH_BYTES;
    return arc_sdpa_decode(&q, stream);
}

extern "C" int arc_sdpa_merge(const float* part_out, const float* part_lse, int32_t num_parts, int64_t rows,
                              int32_t hd, int64_t part_out_stride, int64_t part_lse_stride, const void* gate,
                              void* out_bf16, float* out_f32, float* out_lse, void* stream) {
    if (!part_out || !part_lse) return ARC_ERR_NULL_POINTER;
    if (!out_bf16 && !out_f32) return ARC_ERR_NULL_POINTER;
    if (num_parts <= 0 || rows <= 0 || rows > 0x7fffffffLL) return ARC_ERR_BAD_SHAPE;
    if (hd != 128 && hd != 256) return ARC_ERR_UNSUPPORTED_HEAD_DIM;
    if (gate && !out_bf16) return ARC_ERR_NULL_POINTER;
    if (!aligned16(part_out) || (out_bf16 && !aligned16(out_bf16)) || (out_f32 && !aligned16(out_f32)) ||
        (gate && !aligned16(gate)))
        return ARC_ERR_ALIGNMENT;
    UniformMergeParams mp{};
    mp.part_o = part_out;
    mp.part_lse = part_lse;
    mp.gate = static_cast<const uint16_t*>(gate);
    mp.out = static_cast<uint16_t*>(out_bf16);
    mp.out_f32 = out_f32;
    mp.out_lse = out_lse;
    mp.rows = rows;
    mp.num_parts = num_parts;
    mp.seq = 0;
    mp.o_part_stride = part_out_stride > 0 ? part_out_stride : rows * hd;
    mp.lse_part_stride = part_lse_stride > 0 ? part_lse_stride : rows;
    if ((mp.o_part_stride & 3) != 0) return ARC_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (unsigned)((rows + UMERGE_ROWS - 1) / UMERGE_ROWS);
    if (hd == 128)
        sdpa_uniform_merge_kernel<128><<<blocks, 32 * UMERGE_ROWS, 0, st>>>(mp);
    else
        sdpa_uniform_merge_kernel<256><<<blocks, 32 * UMERGE_ROWS, 0, st>>>(mp);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? ARC_OK : ARC_ERR_CUDA;
}

extern "C" int arc_mul_sigmoid_inplace(void* a, const void* gate, int64_t n, void* stream) {
    if (!a || !gate) return ARC_ERR_NULL_POINTER;
    if (n < 0) return ARC_ERR_BAD_SHAPE;
    if (n == 0) return ARC_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    mul_sigmoid_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t*>(a), static_cast<const uint16_t*>(gate), n);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? ARC_OK : ARC_ERR_CUDA;
}

extern "C" int arc_qkv_prepare(const arc_qkv_prepare_params* p, void* stream) {
    if (!p) return ARC_ERR_NULL_POINTER;
    if (p->batch <= 0 || p->seq < 0 || p->nq < 0 || p->nkv < 0) return ARC_ERR_BAD_SHAPE;
    if (p->hd != 128 && p->hd != 256 && p->hd != 512) return ARC_ERR_UNSUPPORTED_HEAD_DIM;
    if (p->n_active_pairs < 0 || p->n_active_pairs > p->hd / 2) return ARC_ERR_BAD_SHAPE;
    if ((p->rope_cos == nullptr) != (p->rope_sin == nullptr)) return ARC_ERR_NULL_POINTER;
    if (p->n_active_pairs > 0 && !p->rope_cos && !(p->theta > 0.f)) return ARC_ERR_BAD_SHAPE;
    if (p->k_src && !p->k_dst) return ARC_ERR_NULL_POINTER;
    if (p->v_dst && !p->v_src && !p->k_src) return ARC_ERR_NULL_POINTER;
    if (!p->q && !p->k_src && !p->v_dst) return ARC_OK;
    if (p->seq == 0) return ARC_OK;
    // Shared K/V projection (v_src NULL): V comes from the raw K rows, so K must not be rewritten
    // in place — another warp may already have normalised and rotated the row V is read from.
    if (p->v_dst && !p->v_src && p->k_dst == p->k_src) return ARC_ERR_BAD_SHAPE;
    const int row_count = (p->q ? p->nq : 0) + (p->k_src ? p->nkv : 0) + (p->v_dst ? p->nkv : 0);
    if (row_count == 0) return ARC_OK;  // pointers given, but no heads
    auto aligned = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
    if (!aligned(p->q) || !aligned(p->k_src) || !aligned(p->v_src) || !aligned(p->k_dst) || !aligned(p->v_dst) ||
        !aligned(p->q_weight) || !aligned(p->k_weight))
        return ARC_ERR_ALIGNMENT;
    const int64_t strides[] = {p->q_stride_b, p->q_stride_t, p->k_src_stride_b, p->k_src_stride_t, p->v_src_stride_b,
                               p->v_src_stride_t, p->k_dst_stride_b, p->k_dst_stride_t, p->v_dst_stride_b, p->v_dst_stride_t};
    for (int64_t st : strides)
        if (st < 0 || st % 8 != 0) return ARC_ERR_ALIGNMENT;
    // a token's heads must fit between two tokens
    const int64_t qrow = (int64_t)p->nq * p->hd, kvrow = (int64_t)p->nkv * p->hd;
    if ((p->q && p->q_stride_t < qrow) || (p->k_src && (p->k_src_stride_t < kvrow || p->k_dst_stride_t < kvrow)) ||
        (p->v_src && p->v_src_stride_t < kvrow) || (p->v_dst && p->v_dst_stride_t < kvrow))
        return ARC_ERR_BAD_SHAPE;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc != ARC_OK) return rc;

    QkvPrepareParams kp{};
    kp.q = static_cast<uint16_t*>(p->q);
    kp.k_src = static_cast<const uint16_t*>(p->k_src);
    kp.v_src = static_cast<const uint16_t*>(p->v_src);
    kp.k_dst = static_cast<uint16_t*>(p->k_dst);
    kp.v_dst = static_cast<uint16_t*>(p->v_dst);
    kp.q_weight = static_cast<const uint16_t*>(p->q_weight);
    kp.k_weight = static_cast<const uint16_t*>(p->k_weight);
    kp.rope_cos = p->rope_cos;
    kp.rope_sin = p->rope_sin;
    kp.pos_offset = p->pos_offset;
    kp.batch = p->batch;
    kp.seq = p->seq;
    kp.nq = p->nq;
    kp.nkv = p->nkv;
    kp.nap = p->n_active_pairs;
    kp.q_stride_b = p->q_stride_b;
    kp.q_stride_t = p->q_stride_t;
    kp.ks_stride_b = p->k_src_stride_b;
    kp.ks_stride_t = p->k_src_stride_t;
    kp.vs_stride_b = p->v_src_stride_b;
    kp.vs_stride_t = p->v_src_stride_t;
    kp.kd_stride_b = p->k_dst_stride_b;
    kp.kd_stride_t = p->k_dst_stride_t;
    kp.vd_stride_b = p->v_dst_stride_b;
    kp.vd_stride_t = p->v_dst_stride_t;
    kp.rope_stride_b = p->rope_stride_b;
    kp.pos0 = p->pos0;
    kp.theta = p->theta;
    kp.eps = p->eps;
    kp.rot_half = p->rot_half > 0 ? p->rot_half : p->hd / 2;
    kp.freq_denom = p->freq_denom > 0 ? p->freq_denom : p->hd;
    kp.mrope_pos = p->mrope_positions;
    kp.sec1 = p->mrope_section[1];
    kp.sec2 = p->mrope_section[2];
    kp.v_copy = p->v_copy ? 1 : 0;
    if (kp.rot_half != p->hd / 2) {
        const int rh = kp.rot_half;
        if (rh < 8 || (rh & (rh - 1)) != 0 || rh > p->hd / 4 || p->n_active_pairs > rh) return ARC_ERR_BAD_SHAPE;
    }
    // A CTA works on `tpc` consecutive tokens per round: enough (token, head) rows for its eight warps
    // (each takes 512 / hd rows per pass), within the shared-memory angle table of 1024 pairs.
    const long long tokens = (long long)p->batch * p->seq;
    if (tokens > 0x7fffffffLL) return ARC_ERR_TOO_LARGE;
    const int rows = row_count;
    const int rows_per_pass = 8 * (512 / p->hd);
    int tpc = (8 * rows_per_pass + rows - 1) / rows;  // about eight passes per warp and round
    const int max_tpc = 1024 / (p->hd / 2);
    if (tpc > max_tpc) tpc = max_tpc;
    if (tpc < 1) tpc = 1;
    const long long rounds = (tokens + tpc - 1) / tpc;
    const long long cap = (long long)ds->sm_count * 8;  // eight CTAs per SM keep enough loads in flight
    const unsigned ctas = (unsigned)(rounds < cap ? rounds : cap);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool qwen = kp.rot_half != p->hd / 2 || kp.freq_denom != p->hd || kp.mrope_pos != nullptr || kp.v_copy;
    // (measured on config 3's pre-processing: 64 rows per token 220 -> 207 us with the look-ahead form, 8 rows per
    // token 43 -> 45 us)
    const bool ahead = rows >= 24;
    auto launch = [&](auto hd_tag, auto qwen_tag) {
        constexpr int H = decltype(hd_tag)::value;
        constexpr bool Q = decltype(qwen_tag)::value;
        if (ahead) qkv_prepare_kernel<H, Q, true><<<ctas, 256, 0, st>>>(kp, tpc);
        else qkv_prepare_kernel<H, Q, false><<<ctas, 256, 0, st>>>(kp, tpc);
    };
    auto launch_hd = [&](auto qwen_tag) {
        if (p->hd == 128) launch(std::integral_constant<int, 128>{}, qwen_tag);
        else if (p->hd == 256) launch(std::integral_constant<int, 256>{}, qwen_tag);
        else launch(std::integral_constant<int, 512>{}, qwen_tag);
    };
    if (qwen) launch_hd(std::true_type{});
    else launch_hd(std::false_type{});
    g_launches.fetch_add(1, std::memory_order_relaxed);
    ARC_CUDA(cudaGetLastError());
    return ARC_OK;
}

static int fill_mask(float* mask, const int32_t* block_ids, int32_t q_len, int32_t kv_len, int32_t past_offset,
                     int32_t sliding_window, void* stream);

extern "C" int arc_fill_causal_mask(float* mask, int32_t q_len, int32_t kv_len, int32_t past_offset,
                                    int32_t sliding_window, void* stream) {
    return fill_mask(mask, nullptr, q_len, kv_len, past_offset, sliding_window, stream);
}

extern "C" int arc_fill_causal_mask_with_block_ids(float* mask, const int32_t* block_ids, int32_t q_len,
                                                   int32_t kv_len, int32_t past_offset, int32_t sliding_window,
                                                   void* stream) {
    // Positions past_offset - (kv_len - q_len) .. past_offset + q_len - 1 are looked up.
    if (block_ids && past_offset - (kv_len - q_len) < 0) return ARC_ERR_BAD_SHAPE;
    return fill_mask(mask, block_ids, q_len, kv_len, past_offset, sliding_window, stream);
}

static int fill_mask(float* mask, const int32_t* block_ids, int32_t q_len, int32_t kv_len, int32_t past_offset,
                     int32_t sliding_window, void* stream) {
    if (!mask) return ARC_ERR_NULL_POINTER;
    if (q_len < 0 || kv_len < 0) return ARC_ERR_BAD_SHAPE;
    const long long n = (long long)q_len * kv_len;
    if (n == 0) return ARC_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fill_causal_mask_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        mask, block_ids, q_len, kv_len, past_offset, sliding_window);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? ARC_OK : ARC_ERR_CUDA;
}

extern "C" int arc_sdpa_device_status(uint32_t* fault_code, uint32_t* fault_detail) {
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc != ARC_OK) return rc;
    uint32_t w[2] = {0, 0};
    if (cudaDeviceSynchronize() != cudaSuccess) return ARC_ERR_CUDA;
    if (cudaMemcpy(w, ds->fault, sizeof(w), cudaMemcpyDeviceToHost) != cudaSuccess) return ARC_ERR_CUDA;
    if (fault_code) *fault_code = w[0];
    if (fault_detail) *fault_detail = w[1];
    if (w[0] == 0) return ARC_OK;
    return w[0] == FAULT_BAD_KV_RANGE ? ARC_ERR_DEVICE_BAD_RANGE : ARC_ERR_DEVICE_WAIT_TIMEOUT;
}

extern "C" int arc_sdpa_clear_device_status(void) {
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc != ARC_OK) return rc;
    if (cudaDeviceSynchronize() != cudaSuccess) return ARC_ERR_CUDA;
    return cudaMemset(ds->fault, 0, 2 * sizeof(uint32_t)) == cudaSuccess ? ARC_OK : ARC_ERR_CUDA;
}

extern "C" const char* arc_sdpa_last_error(void) { return g_last_error; }

extern "C" uint64_t arc_sdpa_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
