// Inline-PTX building blocks for the sm_100a attention kernels: mbarriers with
// bounded waits, TMA (tensor-map and plain bulk copies, never multicast),
// tcgen05 tensor-memory management / MMA / load / store, and the warp-level
// ldmatrix / mma.sync / movmatrix pieces the HBM-bound decode kernel uses.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace arc {

// ---------------------------------------------------------------------------
// Error reporting from device code: a kernel that gives up on a wait records
// where in a caller-visible status word and returns; it never traps or spins
// without bound.
// ---------------------------------------------------------------------------
enum DeviceFault : uint32_t {
    FAULT_NONE = 0,
    FAULT_WAIT_Q = 1,
    FAULT_WAIT_K = 2,
    FAULT_WAIT_V = 3,
    FAULT_WAIT_S = 4,
    FAULT_WAIT_P = 5,
    FAULT_WAIT_O = 6,
    FAULT_WAIT_EMPTY = 7,
    FAULT_WAIT_FULL = 8,
    FAULT_WAIT_PEER = 9,
    FAULT_BAD_KV_RANGE = 10,  // not a wait: a sequence's rows reach past the cache, or its length past the stated bound
};

// First fault wins; `detail` says which iteration / barrier gave up.
__device__ __forceinline__ void report_fault(uint32_t* fault, uint32_t code, uint32_t detail) {
    if (atomicCAS(fault, 0u, code) == 0u) fault[1] = detail;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute
// may start (be scheduled, run its prologue) while the kernel before it in the stream is still
// running; it must call grid_dependency_wait() before touching anything that kernel writes.  The
// earlier kernel calls grid_launch_dependents() once its CTAs no longer need the SM resources the
// next one is waiting for to be scheduled (here: at its very start — the dependent grids are small).
// Without the attribute both are no-ops.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Register budget per warp group (four consecutive warps; every thread of the
// group executes the same statement): a group that needs few registers hands
// them back so that another can take more than the launch-time share.
// ---------------------------------------------------------------------------
template <int REGS>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}

template <int REGS>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Make generic-proxy writes to shared memory visible to the async proxy (TMA / tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                     smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// The same with a suspend-time hint: the hardware may keep the thread asleep, without issuing
// anything, until the phase completes or about `hint_ns` have passed.  A waiting warp then takes
// no issue slots from the warps of its scheduler that have work.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Non-blocking: has the phase with the given parity completed?
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for the phase with the given parity to complete.  Gives up after
// ~`limit_cycles` SM clocks (default: about a second) and returns false; the
// caller records a fault and unwinds.
// The polling loop is one out-of-line function: waits are all over the kernels and their code
// would otherwise be repeated at every site (the kernels have to fit the instruction cache).
// GROUP gives warp groups that run under different register budgets (setmaxnreg) a copy each:
// the assembler cannot place a function that is called from regions with different budgets.
template <int GROUP>
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, long long limit_cycles) {
    const long long t0 = clock64();
    while (!mbar_try_wait_hint(bar, parity, 200000u)) {
        if (clock64() - t0 > limit_cycles) return false;
    }
    return true;
}

template <int GROUP = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          long long limit_cycles = 2000000000LL) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow<GROUP>(bar, parity, limit_cycles);
}

// The same for waits that are long and not urgent (an epilogue waiting for a whole tile): the
// thread sleeps between polls, so that it does not take issue slots from the warps that work.
template <int GROUP>
__device__ __noinline__ bool mbar_wait_relaxed_slow(uint64_t* bar, uint32_t parity, long long limit_cycles) {
    long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(100);
        if ((++spins & 0x3Fu) == 0 && clock64() - t0 > limit_cycles) return false;
    }
    return true;
}

template <int GROUP = 0>
__device__ __forceinline__ bool mbar_wait_relaxed_warp(uint64_t* bar, uint32_t parity,
                                                       long long limit_cycles = 2000000000LL) {
    bool ok = mbar_try_wait(bar, parity);
    if (!ok) ok = mbar_wait_relaxed_slow<GROUP>(bar, parity, limit_cycles);
    return __all_sync(0xffffffffu, ok);
}

// Same, with a warp-uniform answer (every lane polls; all must succeed), so the
// warp-collective tcgen05 / ldmatrix instructions that follow never see a
// partially exited warp.
template <int GROUP = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_wait<GROUP>(bar, parity));
}

// ---------------------------------------------------------------------------
// Thread-block clusters: rank, shared memory of the other CTAs (distributed shared memory) and
// mbarriers across the cluster.  A CTA may only be read while it is alive: every CTA therefore
// waits for the others' "done reading" arrivals before it exits.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}

// All threads of all CTAs of the cluster (every thread must still be running).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Ask a line of global memory into L2 (no register, no wait).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }

// Address of this CTA's shared-memory location `saddr` in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ float2 ld_cluster_f32x2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
    return v;
}

// Arrive on an mbarrier of another CTA of the cluster (address from map_to_cta); release at cluster
// scope, so this thread's earlier shared-memory writes are visible to whoever acquires the phase.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}

// Bounded wait on a local mbarrier whose arrivals come from the whole cluster (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, long long limit_cycles = 2000000000LL) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(200000u)
            : "memory");
        if (ok) return true;
        if (clock64() - t0 > limit_cycles) return false;
    }
}

// ---------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 4-D tiled load, one CTA, completion on an mbarrier.  c0 is the innermost
// coordinate and must be a multiple of 8 elements for 16-bit data (16 bytes).
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tmap, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// The same tile brought into L2 only (no shared-memory destination, nothing to wait for): a later
// load of it then completes with L2 latency instead of DRAM latency.
__device__ __forceinline__ void tma_prefetch_4d(const void* tmap, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// 2-D tiled load (c0 innermost, multiple of 8 elements for 16-bit data).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Plain 1-D bulk copy global -> shared (both 16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes,
                                             uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: tensor memory + 5th-generation MMA (single-CTA group)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor (64-bit): start address, leading / stride
// byte offsets (all >> 4), descriptor version 1 (Blackwell) at bit 46, 128-byte
// swizzle (layout type 2) at bits 61-63.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulate.
// b_mn_major: B operand stored MN-major (N contiguous) instead of K-major.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, bool b_mn_major) {
    return (1u << 4)                       // D format f32
           | (1u << 7)                     // A format bf16
           | (1u << 10)                    // B format bf16
           | ((b_mn_major ? 1u : 0u) << 16)  // B major
           | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Eight MMAs of one K = 128 slab in a single statement: the issuing thread spends eight issue
// slots instead of eight rounds of address arithmetic, which matters because it shares an
// instruction scheduler with busy softmax warps.  The first MMA accumulates only if asked to.
__device__ __forceinline__ void umma_ss_x8(uint32_t d_tmem, const uint64_t (&a)[8], const uint64_t (&b)[8],
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %18, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %9, %17, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %10, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %11, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %12, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %13, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %6, %14, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %15, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %8, %16, %17, q;\n\t}" ::"r"(d_tmem),
        "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(a[4]), "l"(a[5]), "l"(a[6]), "l"(a[7]), "l"(b[0]), "l"(b[1]),
        "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7]), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same with the A operand in tensor memory.
__device__ __forceinline__ void umma_ts_x8(uint32_t d_tmem, const uint32_t (&a)[8], const uint64_t (&b)[8],
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %18, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %9, %17, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %10, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %11, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %12, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %13, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %14, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%7], %15, %17, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%8], %16, %17, q;\n\t}" ::"r"(d_tmem),
        "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "l"(b[0]), "l"(b[1]),
        "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7]), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Warp-uniform forms: every lane executes the statement with identical operands and only the
// lane whose `leader` flag is set issues the instruction.  Keeping the surrounding address
// arithmetic uniform across the warp lets it live in the uniform datapath, which matters when
// the issuing warp shares its scheduler with busy warps.
__device__ __forceinline__ void umma_ss_lead(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate, uint32_t leader) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ void umma_ts_lead(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate, uint32_t leader) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ void umma_commit_lead(uint64_t* bar, uint32_t leader) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)),
        "r"(leader)
        : "memory");
}

// Arrive on an mbarrier once every tcgen05 operation issued so far by this
// thread has completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives
// columns [col, col+32) of TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---------------------------------------------------------------------------
// Scalar helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32 pairs (sm_100): one instruction works on two floats held in a 64-bit register.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Pack two floats into bf16x2 (round to nearest even); `lo` lands in bits 0-15.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float(static_cast<uint32_t>(b) << 16);
}

__device__ __forceinline__ float bf16_round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

// ---------------------------------------------------------------------------
// Warp-level tensor-core pieces (decode kernel)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr)
                 : "memory");
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr)
                 : "memory");
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Transpose an 8x8 matrix of 16-bit elements held across the warp.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

}  // namespace arc
