// Inline-PTX wrappers shared by the kernels that use mbarriers and bulk (TMA) copies: shared-memory addresses, mbarrier
// init / arrive / expect-tx / try-wait, a wall-clock bounded wait, and the 1-D bulk copy global -> shared.
#pragma once
#include <stdint.h>

namespace ltq {

constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // every device-side wait gives up after 2 s

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Announces bytes without arriving: the phase cannot complete before a later arrival, whatever lands meanwhile.
__device__ __forceinline__ void mbar_expect_tx_only(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false after WAIT_LIMIT_NS, or soon after another role has given up.
// The wall clock (%globaltimer) takes a few hundred nanoseconds to read, far longer than a barrier poll, so it is
// consulted only once per 4096 failed polls: a wait that is satisfied quickly never touches it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *status, uint32_t code, uint64_t limit_ns = WAIT_LIMIT_NS)
{
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 4095u) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = global_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort_flag = 1;
                atomicCAS(status, 0u, code);
                return false;
            }
        }
    }
}

// True in exactly one lane of a fully converged warp (the same lane every time).  Code that issues tcgen05.mma keeps
// its loop warp-uniform and lets only the elected lane execute the instruction: in that form the compiler holds the
// descriptors in uniform registers and a 128x256x32 MMA issues at the tensor pipe's own rate (~128 cycles); issued from
// a divergent single-lane branch the same instruction costs ~150-180 cycles and starves the pipe.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred P1;\n\t"
        "elect.sync _|P1, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, P1;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// Programmatic dependent launch.  griddep_wait: returns once every kernel this grid programmatically depends on has
// completed and its writes are visible (at once when the grid was launched without such a dependency).
// griddep_launch_dependents: this CTA no longer holds back the launch of the next kernel in the stream; that kernel
// starts when every CTA of this grid has said so or exited.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

}  // namespace ltq
