// Self-test of the device-side failure path: a kernel whose wait can never be satisfied (an mbarrier nothing arrives on)
// gives up after the requested limit, records its code in the device status word and returns normally, leaving the
// context usable.  This is how the bounded waits of the GEMM kernels are exercised without hanging or faulting a GPU.
#include "ltq_common.cuh"
#include "ltq_ptx.cuh"

namespace ltq {

__global__ void bounded_wait_probe_kernel(uint32_t *status, uint64_t limit_ns)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // parity 0 of a fresh barrier completes only after one arrival; none is ever made
    mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 0x900u, limit_ns);
}

cudaError_t launch_bounded_wait_probe(uint32_t *status, uint64_t limit_ns, cudaStream_t stream)
{
    bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(status, limit_ns);
    count_launch();
    return cudaGetLastError();
}

}  // namespace ltq
