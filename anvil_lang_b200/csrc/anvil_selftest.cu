// anvil_selftest.cu — a check of the failure path of the contraction templates' waits, without a failure.
//
// Every wait of the tensor-core templates (anvil_gemm_sm100.cuh) is an mbarrier wait with a clock limit: when the
// limit runs out the waiting thread records ANVIL_TC_TIMEOUT in the arena header's status word and the kernel
// returns normally, so the host sees "a kernel gave up waiting on a barrier" at its next fault check and the context
// stays usable. The entry point here runs that same wait (`anvil::tc::mbar_wait`) on a barrier that nothing ever
// arrives on, with a caller-chosen limit (about a millisecond in the test), and reports what the kernel recorded.
// It never traps, spins without bound or touches memory outside the arena header.
#include "anvil_cuda.h"
#include "anvil_gemm_sm100.cuh"

#include <cuda_runtime.h>

namespace {

__global__ void wait_on_a_barrier_nobody_arrives_on(uint32_t *status, long long limit_clocks, long long *waited) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        const uint32_t b = anvil::tc::smem_u32(&bar);
        anvil::tc::mbar_init(b, 1);                       // one arrival expected; none will come
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const long long t0 = clock64();
        const bool flipped = anvil::tc::mbar_wait(b, 0, limit_clocks);
        *waited = clock64() - t0;
        if (!flipped) atomicExch(status, anvil::tc::TIMEOUT);
    }
}

}  // namespace

extern "C" int anvil_rt_selftest_wait(anvil_rt *rt, long long limit_clocks, uint32_t *status_out, long long *waited_clocks) {
    if (!rt || !status_out || !waited_clocks) return 1;
    if (limit_clocks < 0 || limit_clocks > (1LL << 31)) return anvil_rt_set_error(rt, "anvil: selftest wait limit out of range");
    char *arena = (char *)anvil_rt_ptr(rt, 0);
    if (!arena) return anvil_rt_set_error(rt, "anvil: no arena");
    cudaStream_t st = (cudaStream_t)anvil_rt_stream(rt);
    long long *waited_dev = (long long *)(arena + ANVIL_RT_CHECK_OFF);       // 8 bytes of header scratch
    wait_on_a_barrier_nobody_arrives_on<<<1, 32, 0, st>>>((uint32_t *)(arena + ANVIL_RT_STATUS_OFF), limit_clocks, waited_dev);
    if (cudaGetLastError() != cudaSuccess) return anvil_rt_set_error(rt, "anvil: selftest launch failed");
    if (anvil_rt_d2h(rt, status_out, ANVIL_RT_STATUS_OFF, 4)) return 1;
    if (anvil_rt_d2h(rt, waited_clocks, ANVIL_RT_CHECK_OFF, 8)) return 1;
    return 0;
}
