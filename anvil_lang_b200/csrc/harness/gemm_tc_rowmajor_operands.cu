// gemm_tc_rowmajor_operands — weight-gradient shaped products (A read along m, B along n, split-k partials)
// through the resident pair kernel, on seeded data, with 64 entries checked against a float64 sum.
// An optional argument 0..4 runs one configuration only (for a one-kernel ncu capture).
// Build (from the repository root):
//   nvcc -O3 -std=c++17 -fmad=false -gencode arch=compute_100a,code=sm_100a -I anvil_lang_b200/csrc \
//        -o anvil_lang_b200/_build/gemm_tc_rowmajor_operands anvil_lang_b200/csrc/harness/gemm_tc_rowmajor_operands.cu
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>
#include <stdint.h>
#include "anvil_gemm_sm100.cuh"
template <int M_, int N_, int K_>
struct Fn {      // C[m, n] = sum_k X[k, m] * Y[k, n]
    const float *__restrict__ x; const float *__restrict__ y; float *c;
    static constexpr int M = M_, N = N_, K = K_, NB = 1, NLD = 0;
    static constexpr float ALPHA = 1.0f;
    __device__ __forceinline__ void a4(int m, int k, int bt, float (&v)[4]) const {
        v[0] = x[(long)k * M + m]; v[1] = x[(long)(k + 1) * M + m]; v[2] = x[(long)(k + 2) * M + m]; v[3] = x[(long)(k + 3) * M + m]; }
    __device__ __forceinline__ void b4(int k, int n, int bt, float (&v)[4]) const {
        v[0] = y[(long)k * N + n]; v[1] = y[(long)(k + 1) * N + n]; v[2] = y[(long)(k + 2) * N + n]; v[3] = y[(long)(k + 3) * N + n]; }
    __device__ __forceinline__ void a_touch(int m, int k, int bt) const { asm volatile("prefetch.global.L2 [%0];" ::"l"(x + (long)k * M + m)); }
    __device__ __forceinline__ void b_touch(int k, int n, int bt) const { asm volatile("prefetch.global.L2 [%0];" ::"l"(y + (long)k * N + n)); }
    __device__ __forceinline__ void a4m(int m, int k, int bt, float (&v)[4]) const {
        float4 q = *reinterpret_cast<const float4 *>(x + (long)k * M + m); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    __device__ __forceinline__ void b4n(int k, int n, int bt, float (&v)[4]) const {
        float4 q = *reinterpret_cast<const float4 *>(y + (long)k * N + n); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    __device__ __forceinline__ void epi_touch(int m, int n, int bt) const {}
    __device__ __forceinline__ void epi_loads(int m, int n, int bt, float (&ld)[1]) const {}
    __device__ __forceinline__ void epi2(int m, int n, int bt, float acc, const float (&ld)[1]) const { c[(long)m * N + n] = acc; }
    __device__ __forceinline__ void epi(int m, int n, int bt, float acc) const { c[(long)m * N + n] = acc; }
};
template <class F, int S, int ACCS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(anvil::tc::PP_THREADS, 1) kern_pp(F f, float *partial, uint32_t *status) {
    anvil::tc::gemm_tc_pair_persistent<F, false, false, S, ACCS>(f, partial, status);
}
template <int M, int N, int K, int S, int ACCS> void run(const char *name) {
    float *x, *y, *c, *part; uint32_t *st;
    cudaMalloc(&x, sizeof(float) * M * K); cudaMalloc(&y, sizeof(float) * K * N); cudaMalloc(&c, sizeof(float) * M * N);
    cudaMalloc(&part, sizeof(float) * M * N * S); cudaMalloc(&st, 4);
    std::vector<float> hx((size_t)M * K), hy((size_t)K * N);
    for (size_t i = 0; i < hx.size(); i++) hx[i] = (float)((i * 2654435761u >> 20) & 255) / 256.0f - 0.5f;
    for (size_t i = 0; i < hy.size(); i++) hy[i] = (float)((i * 40503u >> 7) & 255) / 256.0f - 0.5f;
    cudaMemcpy(x, hx.data(), hx.size() * 4, cudaMemcpyHostToDevice); cudaMemcpy(y, hy.data(), hy.size() * 4, cudaMemcpyHostToDevice);
    cudaMemset(st, 0, 4);
    using F = Fn<M, N, K>;
    auto k = kern_pp<F, S, ACCS>;
    const int smem = anvil::tc::pp_smem_bytes();
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const int work = ((M + 255) / 256) * ((N + 255) / 256) * S;
    const int grid = 2 * (work < 74 ? work : 74);
    F f{x, y, c};
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < 3; i++) k<<<grid, anvil::tc::PP_THREADS, smem>>>(f, part, st);
    cudaDeviceSynchronize();
    cudaEventRecord(e0); k<<<grid, anvil::tc::PP_THREADS, smem>>>(f, part, st); cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    uint32_t hst; cudaMemcpy(&hst, st, 4, cudaMemcpyDeviceToHost);
    // check a few entries against a double sum
    std::vector<float> hp((size_t)M * N * S);
    cudaMemcpy(hp.data(), S > 1 ? part : c, (S > 1 ? hp.size() : (size_t)M * N) * 4, cudaMemcpyDeviceToHost);
    double maxerr = 0, maxref = 0;
    for (int t = 0; t < 64; t++) {
        int m = (t * 37) % M, n = (t * 101 + 3) % N;
        double ref = 0; for (int kk = 0; kk < K; kk++) ref += (double)hx[(size_t)kk * M + m] * hy[(size_t)kk * N + n];
        double got = 0; for (int s = 0; s < S; s++) got += hp[((size_t)s * M + m) * N + n];
        maxerr = std::max(maxerr, std::abs(got - ref)); maxref = std::max(maxref, std::abs(ref));
    }
    printf("%s: %.1f us (%.0f TFLOP/s), grid %d, status %x, err %s, max |diff| %.2e of %.2e\n", name, ms * 1e3, 2.0 * M * N * K / ms / 1e9, grid, hst,
           cudaGetErrorString(cudaGetLastError()), maxerr, maxref);
    cudaFree(x); cudaFree(y); cudaFree(c); cudaFree(part); cudaFree(st);
}
int main(int argc, char **argv) {
    const int which = argc > 1 ? atoi(argv[1]) : -1;
    if (which < 0 || which == 0) run<512, 512, 16384, 18, 2>("512x512x16384 split 18");
    if (which < 0 || which == 1) run<512, 512, 16384, 37, 1>("512x512x16384 split 37 (one accumulator)");
    if (which < 0 || which == 2) run<2048, 512, 16384, 4, 2>("2048x512x16384 split 4");
    if (which < 0 || which == 3) run<2048, 512, 16384, 9, 2>("2048x512x16384 split 9");
    if (which < 0 || which == 4) run<512, 2048, 16384, 4, 2>("512x2048x16384 split 4");
    return 0;
}
