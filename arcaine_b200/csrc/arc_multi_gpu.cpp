// Host-side multi-GPU helpers of the C ABI: partition planning, set-up of the in-kernel record exchange
// and the NCCL all-gather + merge form of it.  Plain host code; NCCL is reached through dlsym so that the
// library neither links against it nor needs its header.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <numeric>
#include <vector>

#include "../../include/arc_sdpa.h"

extern "C" int arc_plan_head_shards(int32_t nq, int32_t nkv, int32_t batch, int32_t world, int32_t rank,
                                    arc_head_shard* out) {
    if (!out) return ARC_ERR_NULL_POINTER;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || batch <= 0 || world <= 0 || rank < 0 || rank >= world)
        return ARC_ERR_BAD_SHAPE;
    const int group = nq / nkv;
    int head_ways = 1;
    for (int d = 1; d <= world; ++d)
        if (world % d == 0 && nkv % d == 0) head_ways = d;
    const int batch_ways = world / head_ways;
    const int heads_per = nkv / head_ways;
    const int hw = rank % head_ways, bw = rank / head_ways;
    auto cut = [&](int i) { return std::min<int64_t>(batch, ((int64_t)batch * i + batch_ways - 1) / batch_ways); };
    out->kv_head_begin = hw * heads_per;
    out->kv_head_end = (hw + 1) * heads_per;
    out->q_head_begin = out->kv_head_begin * group;
    out->q_head_end = out->kv_head_end * group;
    out->batch_begin = (int32_t)cut(bw);
    out->batch_end = (int32_t)cut(bw + 1);
    return ARC_OK;
}

extern "C" int arc_plan_seq_shards(int64_t kv_len, int32_t world, int32_t rank, int32_t align, int64_t* begin,
                                   int64_t* end) {
    if (!begin || !end) return ARC_ERR_NULL_POINTER;
    if (kv_len < 0 || world <= 0 || rank < 0 || rank >= world || align < 0) return ARC_ERR_BAD_SHAPE;
    const int64_t a = align > 0 ? align : 64;
    int64_t per = (kv_len + world - 1) / world;
    per = (per + a - 1) / a * a;
    *begin = std::min<int64_t>(kv_len, (int64_t)rank * per);
    *end = std::min<int64_t>(kv_len, (int64_t)(rank + 1) * per);
    return ARC_OK;
}

extern "C" int arc_plan_batch_shards(const int32_t* kv_len, int32_t batch, int32_t world, int32_t* owner) {
    if (!kv_len || !owner) return ARC_ERR_NULL_POINTER;
    if (batch < 0 || world <= 0) return ARC_ERR_BAD_SHAPE;
    std::vector<int> order(batch);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return kv_len[a] > kv_len[b]; });
    std::vector<int64_t> load(world, 0);
    std::vector<int> count(world, 0);
    for (int i : order) {
        int best = 0;
        for (int r = 1; r < world; ++r)
            if (load[r] < load[best] || (load[r] == load[best] && count[r] < count[best])) best = r;
        owner[i] = best;
        load[best] += kv_len[i] > 0 ? kv_len[i] : 0;
        ++count[best];
    }
    return ARC_OK;
}

extern "C" int arc_sdpa_exchange_init(void* buffer, int32_t world, int32_t batch, int32_t nq, int32_t hd,
                                      const uint64_t* peers, uint64_t* peers_dev, void* stream) {
    if (!buffer || !peers || !peers_dev) return ARC_ERR_NULL_POINTER;
    const size_t bytes = arc_sdpa_exchange_bytes(world, batch, nq, hd);
    if (bytes == 0) return ARC_ERR_BAD_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(buffer, 0, bytes, st) != cudaSuccess) return ARC_ERR_CUDA;
    if (cudaMemcpyAsync(peers_dev, peers, (size_t)world * sizeof(uint64_t), cudaMemcpyHostToDevice, st) != cudaSuccess)
        return ARC_ERR_CUDA;
    return ARC_OK;
}

extern "C" size_t arc_sdpa_record_floats(int32_t batch, int32_t nq, int32_t hd) {
    if (batch <= 0 || nq <= 0 || hd <= 0) return 0;
    const size_t n = (size_t)batch * nq * hd + (size_t)batch * nq;
    return (n + 3) / 4 * 4;
}

namespace {
// ncclAllGather(sendbuff, recvbuff, sendcount, datatype, comm, stream); ncclFloat32 = 7; ncclSuccess = 0
using AllGatherFn = int (*)(const void*, void*, size_t, int, void*, cudaStream_t);
AllGatherFn g_allgather = nullptr;
std::once_flag g_nccl_once;

AllGatherFn nccl_allgather() {
    std::call_once(g_nccl_once, [] {
        void* sym = dlsym(RTLD_DEFAULT, "ncclAllGather");  // the copy already in the process (torch's, the caller's)
        if (!sym) {
            if (void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL)) sym = dlsym(lib, "ncclAllGather");
        }
        g_allgather = reinterpret_cast<AllGatherFn>(sym);
    });
    return g_allgather;
}
}  // namespace

extern "C" int arc_sdpa_allgather_merge(const float* record, float* gathered, int32_t world, int32_t batch, int32_t nq,
                                        int32_t hd, const void* gate, void* out_bf16, void* comm, void* stream) {
    if (!record || !gathered || !out_bf16 || !comm) return ARC_ERR_NULL_POINTER;
    if (world <= 0) return ARC_ERR_BAD_SHAPE;
    const size_t n = arc_sdpa_record_floats(batch, nq, hd);
    if (n == 0) return ARC_ERR_BAD_SHAPE;
    AllGatherFn fn = nccl_allgather();
    if (!fn) return ARC_ERR_COLLECTIVE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (fn(record, gathered, n, /*ncclFloat32*/ 7, comm, st) != 0) return ARC_ERR_COLLECTIVE;
    const int64_t rows = (int64_t)batch * nq;
    // records are n floats apart; inside one, lse follows the rows * hd outputs
    return arc_sdpa_merge(gathered, gathered + rows * hd, world, rows, hd, (int64_t)n, (int64_t)n, gate, out_bf16, nullptr,
                          nullptr, stream);
}
