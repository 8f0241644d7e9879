// mma_issue_rate — how fast one thread per SM can issue tcgen05.mma kind::tf32 on fixed shared-memory
// (or tensor-memory) tiles with no data movement: the ceiling of the contraction templates.
// Build (from the repository root):
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -I anvil_lang_b200/csrc \
//        -o anvil_lang_b200/_build/mma_issue_rate anvil_lang_b200/csrc/harness/mma_issue_rate.cu
#include <cstdio>
#include <cuda_runtime.h>
#include <stdint.h>
#include "anvil_gemm_sm100.cuh"
using namespace anvil::tc;
template <int BN, bool TS>
__global__ void __launch_bounds__(128, 1) mma_loop(int iters, float *out) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + 200 * 1024);
    uint32_t *slot = reinterpret_cast<uint32_t *>(smem + 200 * 1024 + 16);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 50 * 1024; i += 128) reinterpret_cast<float *>(smem)[i] = 0.001f * (i % 7);
    if (threadIdx.x == 0) { mbar_init(smem_u32(bar), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *slot;
    if (threadIdx.x == 0) {
        const uint32_t base = smem_u32(smem);
        const uint32_t LA = lbo_bytes(128), LB = lbo_bytes(BN);
        const uint32_t idesc = instr_desc(128, BN);
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint64_t da = smem_desc(base + 2 * j * LA, LA), db = smem_desc(base + 64 * 1024 + 2 * j * LB, LB);
                if (TS) {
                    mma_tf32_ts(tmem, tmem + 256 + 8 * j, db, idesc, 1u);
                    mma_tf32_ts(tmem, tmem + 256 + 8 * j, db, idesc, 1u);
                    mma_tf32_ts(tmem, tmem + 256 + 8 * j, db, idesc, 1u);
                } else {
                    mma_tf32(tmem, da, db, idesc, 1u); mma_tf32(tmem, da, db, idesc, 1u); mma_tf32(tmem, da, db, idesc, 1u);
                }
            }
        }
        mma_commit(smem_u32(bar));
        bool ok = mbar_wait(smem_u32(bar), 0);
        if (!ok) out[blockIdx.x] = -1.0f;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory"); }
}
template <int BN, bool TS> void run(const char *name) {
    float *out; cudaMalloc(&out, 4096); cudaMemset(out, 0, 4096);
    auto k = mma_loop<BN, TS>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
    const int iters = 2000;
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    k<<<148, 128, 201 * 1024>>>(100, out); cudaDeviceSynchronize();
    cudaEventRecord(a); k<<<148, 128, 201 * 1024>>>(iters, out); cudaEventRecord(b); cudaEventSynchronize(b);
    float ms; cudaEventElapsedTime(&ms, a, b);
    double mmas = 148.0 * iters * 12, flops = mmas * 2.0 * 128 * BN * 8;
    printf("%s: %.3f ms, %.1f ns per MMA per SM, %.0f TFLOP/s tf32 (%.0f as 3xTF32), err %s\n", name, ms, ms * 1e6 / (iters * 12), flops / ms / 1e9,
           flops / ms / 1e9 / 3, cudaGetErrorString(cudaGetLastError()));
    cudaFree(out);
}
int main() { run<128, false>("SS 128x128x8"); run<256, false>("SS 128x256x8"); run<64, false>("SS 128x64x8"); run<128, true>("TS 128x128x8"); run<256, true>("TS 128x256x8 (A cols 256..)"); return 0; }
