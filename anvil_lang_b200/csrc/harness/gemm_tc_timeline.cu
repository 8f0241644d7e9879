// gemm_tc_timeline — phase timeline of the CTA-pair contraction templates on transformer-sized products.
// The header's optional ANVIL_TC_TRACE hooks are defined here to write %globaltimer stamps; the program
// prints, per leader CTA, set-up / first full stage / main loop / epilogue / exit times for the one-launch
// pair kernel and the resident one, with a plain store and with a read-modify-write epilogue.
// Build (from the repository root):
//   nvcc -O3 -std=c++17 -fmad=false -gencode arch=compute_100a,code=sm_100a -I anvil_lang_b200/csrc \
//        -o anvil_lang_b200/_build/gemm_tc_timeline anvil_lang_b200/csrc/harness/gemm_tc_timeline.cu
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
#include <stdint.h>
__device__ unsigned long long g_trace[4096 * 8];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define ANVIL_TC_TRACE(slot) g_trace[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + (slot)] = gtime()
#include "anvil_gemm_sm100.cuh"
template <int M_, int N_, int K_, bool RMW>
struct Fn {
    const float *__restrict__ a; const float *__restrict__ b; float *c;
    static constexpr int M = M_, N = N_, K = K_, NB = 1;
    static constexpr float ALPHA = 1.0f;
    __device__ __forceinline__ void a4(int m, int k, int bt, float (&v)[4]) const {
        float4 q = *reinterpret_cast<const float4 *>(a + (long)m * K + k); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    __device__ __forceinline__ void b4(int k, int n, int bt, float (&v)[4]) const {
        v[0] = b[(long)k * N + n]; v[1] = b[(long)(k + 1) * N + n]; v[2] = b[(long)(k + 2) * N + n]; v[3] = b[(long)(k + 3) * N + n]; }
    __device__ __forceinline__ void epi_touch(int m, int n, int bt) const { if (RMW) asm volatile("prefetch.global.L2 [%0];" ::"l"(c + (long)m * N + n)); }
    __device__ __forceinline__ void a_touch(int m, int k, int bt) const { asm volatile("prefetch.global.L2 [%0];" ::"l"(a + (long)m * K + k)); }
    __device__ __forceinline__ void b_touch(int k, int n, int bt) const { asm volatile("prefetch.global.L2 [%0];" ::"l"(b + (long)k * N + n)); }
    __device__ __forceinline__ void b4n(int k, int n, int bt, float (&v)[4]) const {
        float4 q = *reinterpret_cast<const float4 *>(b + (long)k * N + n); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    static constexpr int NLD = RMW ? 1 : 0;
    __device__ __forceinline__ void epi_loads(int m, int n, int bt, float (&ld)[1]) const { ld[0] = c[(long)m * N + n]; }
    __device__ __forceinline__ void epi2(int m, int n, int bt, float acc, const float (&ld)[1]) const { c[(long)m * N + n] = RMW ? ld[0] + acc : acc; }
    __device__ __forceinline__ void epi(int m, int n, int bt, float acc) const { if (RMW) c[(long)m * N + n] += acc; else c[(long)m * N + n] = acc; }
};
template <class F, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(anvil::tc::THREADS, 1) kern(F f, uint32_t *status) {
    anvil::tc::gemm_tc_pair_tile<F, true, false, BN, 1>(f, nullptr, status);
}
template <class F, int ACCS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(anvil::tc::PP_THREADS, 1) kern_pp(F f, uint32_t *status) {
    anvil::tc::gemm_tc_pair_persistent<F, true, false, 1, ACCS>(f, nullptr, status);
}
template <int M, int N, int K, bool RMW, int ACCS> void run_pp(const char *name) {
    float *a, *b, *c; uint32_t *st;
    cudaMalloc(&a, sizeof(float) * M * K); cudaMalloc(&b, sizeof(float) * K * N); cudaMalloc(&c, sizeof(float) * M * N); cudaMalloc(&st, 4);
    cudaMemset(a, 0, sizeof(float) * M * K); cudaMemset(b, 0, sizeof(float) * K * N); cudaMemset(c, 0, sizeof(float) * M * N); cudaMemset(st, 0, 4);
    using F = Fn<M, N, K, RMW>;
    auto k = kern_pp<F, ACCS>;
    const int smem = anvil::tc::pp_smem_bytes();
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const int grid = 2 * (tiles < 74 ? tiles : 74);
    F f{a, b, c};
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < 3; i++) k<<<grid, anvil::tc::PP_THREADS, smem>>>(f, st);
    cudaDeviceSynchronize();
    cudaEventRecord(e0); k<<<grid, anvil::tc::PP_THREADS, smem>>>(f, st); cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    std::vector<unsigned long long> tr(grid * 8);
    cudaMemcpyFromSymbol(tr.data(), g_trace, tr.size() * 8);
    uint32_t hst; cudaMemcpy(&hst, st, 4, cudaMemcpyDeviceToHost);
    double d[5] = {0}; int n = 0;
    for (int i = 0; i < grid; i += 2) {
        const unsigned long long *r = &tr[i * 8];
        d[0] += (double)(r[1] - r[0]); d[1] += (double)(r[2] - r[1]); d[2] += (double)(r[3] - r[2]); d[3] += (double)(r[5] - r[3]); d[4] += (double)(r[6] - r[0]); n++;
    }
    printf("%s: %.1f us (%.0f TFLOP/s), status %x, err %s\n", name, ms * 1e3, 2.0 * M * N * K / ms / 1e9, hst, cudaGetErrorString(cudaGetLastError()));
    printf("   per leader CTA (us): setup %.2f | to first full %.2f | all MMAs issued %.2f | last epilogue after that %.2f | total %.2f\n",
           d[0] / n / 1e3, d[1] / n / 1e3, d[2] / n / 1e3, d[3] / n / 1e3, d[4] / n / 1e3);
    cudaFree(a); cudaFree(b); cudaFree(c); cudaFree(st);
}
template <int M, int N, int K, bool RMW, int BN> void run(const char *name) {
    float *a, *b, *c; uint32_t *st;
    cudaMalloc(&a, sizeof(float) * M * K); cudaMalloc(&b, sizeof(float) * K * N); cudaMalloc(&c, sizeof(float) * M * N); cudaMalloc(&st, 4);
    cudaMemset(a, 0, sizeof(float) * M * K); cudaMemset(b, 0, sizeof(float) * K * N); cudaMemset(c, 0, sizeof(float) * M * N); cudaMemset(st, 0, 4);
    using F = Fn<M, N, K, RMW>;
    auto k = kern<F, BN>;
    const int smem = anvil::tc::pair_smem_bytes(BN);
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const int tiles = ((M + 255) / 256) * ((N + BN - 1) / BN);
    F f{a, b, c};
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < 3; i++) k<<<2 * tiles, anvil::tc::THREADS, smem>>>(f, st);
    cudaDeviceSynchronize();
    cudaEventRecord(e0); k<<<2 * tiles, anvil::tc::THREADS, smem>>>(f, st); cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    std::vector<unsigned long long> tr(2 * tiles * 8);
    cudaMemcpyFromSymbol(tr.data(), g_trace, tr.size() * 8);
    uint32_t hst; cudaMemcpy(&hst, st, 4, cudaMemcpyDeviceToHost);
    unsigned long long t0 = ~0ull, tend = 0;
    for (int i = 0; i < 2 * tiles; i++) { t0 = std::min(t0, tr[i * 8]); tend = std::max(tend, tr[i * 8 + 6]); }
    double d[7] = {0}; int n = 0;
    double start_first = 0, start_second = 0; int nf = 0, ns = 0;
    for (int i = 0; i < 2 * tiles; i += 2) {     // leader CTAs
        const unsigned long long *r = &tr[i * 8];
        d[0] += (double)(r[1] - r[0]); d[1] += (double)(r[2] - r[1]); d[2] += (double)(r[3] - r[2]); d[3] += (double)(r[4] - r[3]);
        d[4] += (double)(r[5] - r[4]); d[5] += (double)(r[6] - r[5]); d[6] += (double)(r[6] - r[0]); n++;
        if (r[0] - t0 < 3000) { start_first += (double)(r[0] - t0); nf++; } else { start_second += (double)(r[0] - t0); ns++; }
    }
    printf("%s: %.1f us (%.0f TFLOP/s), status %x, err %s; span by globaltimer %.1f us\n", name, ms * 1e3, 2.0 * M * N * K / ms / 1e9, hst,
           cudaGetErrorString(cudaGetLastError()), (tend - t0) / 1e3);
    printf("   per leader CTA (us): setup %.2f | to first full %.2f | mainloop %.2f | commit->accum seen %.2f | epilogue %.2f | exit sync %.2f | total %.2f\n",
           d[0] / n / 1e3, d[1] / n / 1e3, d[2] / n / 1e3, d[3] / n / 1e3, d[4] / n / 1e3, d[5] / n / 1e3, d[6] / n / 1e3);
    printf("   first-wave CTAs %d start at %.2f us on average, later CTAs %d at %.2f us\n", nf, nf ? start_first / nf / 1e3 : 0.0, ns, ns ? start_second / ns / 1e3 : 0.0);
    cudaFree(a); cudaFree(b); cudaFree(c); cudaFree(st);
}
int main() {
    run<16384, 512, 512, false, 256>("16384x512x512 store   BN256");
    run<16384, 512, 512, true, 256>("16384x512x512 +=      BN256");
    run_pp<16384, 512, 512, false, 1>("16384x512x512 store   persistent, one accumulator");
    run_pp<16384, 512, 512, true, 1>("16384x512x512 +=      persistent, one accumulator");
    run_pp<16384, 512, 512, false, 2>("16384x512x512 store   persistent, two accumulators");
    run_pp<16384, 512, 2048, false, 2>("16384x512x2048 store  persistent, two accumulators");
    run_pp<16384, 2048, 512, false, 1>("16384x2048x512 store  persistent, one accumulator");
    run_pp<16384, 2048, 512, true, 1>("16384x2048x512 +=     persistent, one accumulator");
    run<16384, 512, 2048, false, 256>("16384x512x2048 store  BN256");
    run<16384, 2048, 512, false, 256>("16384x2048x512 store  BN256");
    return 0;
}
