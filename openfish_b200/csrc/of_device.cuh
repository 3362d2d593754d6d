// of_device.cuh -- sm_100a device primitives shared by the decode kernels: mbarrier-tracked
// bulk asynchronous copies (global -> shared, no cluster multicast), bounded waits, warp
// reductions.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace ofd {

// Status codes a kernel can raise in the gpubuf's status word (0 = fine).
enum : int {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,  // a bulk copy never signalled its barrier within the time limit
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals)
                 : "memory");
}
// Make barrier initialisation visible to the asynchronous proxy before the first bulk copy.
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// How long a kernel waits for one asynchronous copy before it gives up, unless the host says
// otherwise: far beyond anything a healthy device needs (a copy takes microseconds).
constexpr uint64_t kDefaultWaitLimitNs = 2000000000ull;

// Wait for phase `parity` of `bar`, but never for longer than `limit_ns` and never once
// the block's abort flag is up.  On timeout the abort flag and the global status word are set
// and the caller carries on (with meaningless data) so that every barrier in the kernel is
// still reached and the kernel ends; the host then reports the status instead of results.
__device__ __forceinline__ void mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  volatile int *abort_flag, int *status,
                                                  uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return;
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (*abort_flag) return;
        if (mbar_try_wait(bar, parity)) return;
        if ((spin & 63u) == 0) {
            __nanosleep(64);
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) {
                *abort_flag = 1;
                atomicExch(status, kStatusWaitTimeout);
                return;
            }
        }
    }
}

// After an abort: give the copies this thread issued last (the newest into each ring slot; copy
// number i went to barrier i % ring with phase parity (i / ring) & 1) one more bounded chance to
// land, so that none of them is still writing into the block's shared memory when the block
// retires and the memory passes to another block.  `issued` = copies issued so far, in order.
__device__ __forceinline__ void mbar_drain_bounded(uint64_t *bars, int ring, int issued, uint64_t limit_ns) {
    const uint64_t t0 = global_timer_ns();
    for (int i = issued > ring ? issued - ring : 0; i < issued; ++i) {
        while (!mbar_try_wait(&bars[i % ring], (uint32_t)(i / ring) & 1u)) {
            __nanosleep(64);
            if (global_timer_ns() - t0 > limit_ns) return;
        }
    }
}

// 1-D bulk asynchronous copy global -> this CTA's shared memory, completion counted in bytes
// on `bar`.  dst, src and bytes must be multiples of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes,
                                         uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Eight floats {v0 v1 v2 v3} {v4 a b 0} to 32 bytes of shared memory at `addr` (a shared-window
// address, 16-byte aligned) if `flag`, as two predicated stores: no branch, so no divergence.
__device__ __forceinline__ void sts_entry_if(bool flag, uint32_t addr, const float (&v)[5], float a, float b) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %0, 0;\n\t"
        "@p st.shared.v4.f32 [%1], {%2, %3, %4, %5};\n\t"
        "@p st.shared.v4.f32 [%1+16], {%6, %7, %8, %9};\n\t}"
        ::"r"((int)flag), "r"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(a), "f"(b), "f"(0.f)
        : "memory");
}

// Order-preserving map float -> int32 (and back) so integer warp reductions can take a max.
__device__ __forceinline__ int float_order_key(float f) {
    const int i = __float_as_int(f);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float float_from_order_key(int k) {
    return __int_as_float(k ^ ((k >> 31) & 0x7fffffff));
}
__device__ __forceinline__ float warp_max(float v) {
    return float_from_order_key(__reduce_max_sync(0xffffffffu, float_order_key(v)));
}

}  // namespace ofd
