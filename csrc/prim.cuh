// Device primitives: system-scope loads/stores, bounded waits, mbarrier and 1-D bulk (TMA) copies.
//
// Same role as the reference's tma.cuh / barrier.cuh / math.cuh (csrc/include/nano_ep/tma.cuh:15-110,
// barrier.cuh:14-51), with one deliberate difference: no wait here is unbounded and nothing traps.
// A wait that runs out records a code in the rank's status words and returns false; callers skip
// the dependent work and still reach their block/grid exits, so the CUDA context stays usable.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "layout.hpp"

namespace nep {

// ---------------------------------------------------------------- status
struct StatusRef {
    uint32_t* dev;            // window ctrl words [0] code, [1] detail, [2] kernel tag (sticky, first error wins)
    volatile uint32_t* host;  // mapped pinned copy the host polls without a device sync
};

__device__ __forceinline__ void report(const StatusRef& s, uint32_t code, uint32_t detail, uint32_t tag) {
    if (atomicCAS(s.dev, 0u, code) == 0u) {
        s.dev[1] = detail;
        s.dev[2] = tag;
        s.host[1] = detail;
        s.host[2] = tag;
        __threadfence_system();
        s.host[0] = code;
    }
}

// ---------------------------------------------------------------- scoped memory ops
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// CTA-scope hand-over words in shared memory
__device__ __forceinline__ void st_release_cta_smem(int* p, int v) {
    asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cta_smem(const int* p) {
    int v;
    asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_f32(float* p, float v) {
    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// 16-byte global accessors that bypass L1 (peer memory and streaming data).
__device__ __forceinline__ int4 ld_nc_v4(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ int4 ld_cg_v4(const void* p) {
    int4 v;
    asm volatile("ld.global.cg.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// L2 eviction policy for data that is read or written exactly once (its lines are the first to go).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ uint64_t l2_evict_normal_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ int4 ld_cg_v4_hint(const void* p, uint64_t policy) {
    int4 v;
    asm volatile("ld.global.cg.L2::cache_hint.v4.s32 {%0,%1,%2,%3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(policy));
    return v;
}
__device__ __forceinline__ void st_v4_hint(void* p, int4 v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v4.s32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(policy) : "memory");
}
__device__ __forceinline__ void st_cg_v4(void* p, int4 v) {
    asm volatile("st.global.cg.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---------------------------------------------------------------- peer barrier
// Lane p < ranks publishes `epoch` into peer p's signal slot for this rank, then waits until
// peer p's value in the local slots reaches `epoch`.  Epochs only grow and are compared with >=,
// so a late waiter never misses a signal.  Must be called by one full warp.  Every earlier write
// of the calling block that peers will read has to be ordered before the call
// (__threadfence_system + __syncthreads when other threads wrote).  Returns false on timeout.
__device__ __forceinline__ bool peer_barrier_warp(
    void* const* peers, int rank, int ranks, int64_t signal_offset, uint64_t epoch, uint64_t timeout_ns, const StatusRef& status,
    uint32_t tag) {
    const int lane = threadIdx.x & 31;
    bool ok = true;
    if (lane < ranks) {
        fence_acq_rel_sys();
        auto* remote = reinterpret_cast<uint64_t*>(static_cast<char*>(peers[lane]) + signal_offset) + rank;
        st_release_sys(remote, epoch);
        const auto* local = reinterpret_cast<const uint64_t*>(static_cast<const char*>(peers[rank]) + signal_offset) + lane;
        const uint64_t start = global_timer_ns();
        uint32_t spins = 0;
        while (ld_acquire_sys(local) < epoch) {
            __nanosleep(32);
            if ((++spins & 63u) == 0u && global_timer_ns() - start > timeout_ns) {
                report(status, kBarrierTimeout, uint32_t(lane), tag);
                ok = false;
                break;
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    fence_acq_rel_sys();
    return ok;
}

// The two halves of the barrier on their own.  `peer_signal_warp`: lane p < ranks publishes `epoch` to peer p
// and returns at once.  `peer_wait_warp`: wait until every peer's value in the local slots reaches `epoch`.
__device__ __forceinline__ void peer_signal_warp(void* const* peers, int rank, int ranks, int64_t signal_offset, uint64_t epoch) {
    const int lane = threadIdx.x & 31;
    if (lane < ranks) {
        fence_acq_rel_sys();
        st_release_sys(reinterpret_cast<uint64_t*>(static_cast<char*>(peers[lane]) + signal_offset) + rank, epoch);
    }
}
__device__ __forceinline__ bool peer_wait_warp(
    void* const* peers, int rank, int ranks, int64_t signal_offset, uint64_t epoch, uint64_t timeout_ns, const StatusRef& status, uint32_t tag) {
    const int lane = threadIdx.x & 31;
    bool ok = true;
    if (lane < ranks) {
        const auto* local = reinterpret_cast<const uint64_t*>(static_cast<const char*>(peers[rank]) + signal_offset) + lane;
        const uint64_t start = global_timer_ns();
        uint32_t spins = 0;
        while (ld_acquire_sys(local) < epoch) {
            __nanosleep(32);
            if ((++spins & 63u) == 0u && global_timer_ns() - start > timeout_ns) {
                report(status, kBarrierTimeout, uint32_t(lane), tag);
                ok = false;
                break;
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    fence_acq_rel_sys();
    return ok;
}

// ---------------------------------------------------------------- mbarrier + bulk copies
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait; false (and a status report by the caller) when the limit is hit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t timeout_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0u && global_timer_ns() - start > timeout_ns) return false;
    }
    return true;
}

// global -> shared, completion counted in bytes on `bar`.  The source may be peer memory; this
// form delivers to this CTA only (plain unicast bulk copy).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_load_hint(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
// shared -> global (local or peer), tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- small math
__device__ __forceinline__ int warp_inclusive_sum(int v) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += n;
    }
    return v;
}

}  // namespace nep
