// anvil_gemm_simt.cuh — CUDA-core contraction template: C[b, m, n] = epilogue(alpha * sum_k A[b, m, k] * B[b, k, n]).
//
// The reference runs a contraction as one thread per output element with a serial loop over k that
// re-reads A and B from global memory (anvil/backend/cuda.py:282-313). This template is the
// general-purpose replacement: 128 x 128 x 16 tiles staged in shared memory, an 8 x 8 register tile
// per thread read with 128-bit shared loads, double-buffered global -> register -> shared
// prefetch. It takes a generated functor F, so operand prologues (max(x, 0), constant scales,
// gathered rows) and fused epilogues (bias, activation, residual, optimizer update, several stores)
// need no extra passes:
//
//   F::M, F::N, F::K, F::NB       extents (NB = independent products)
//   f.a(m, k, b), f.b(k, n, b)    operand values
//   f.epi(m, n, b, acc)           the kernel's statements for one output element
//
// Accumulation order is fixed (k ascending inside a split, splits combined in order), so results
// are bit-reproducible. It is also the fallback for shapes the tcgen05 template does not take.
#pragma once
#include <cuda_runtime.h>

namespace anvil {

constexpr int GS_BM = 128, GS_BN = 128, GS_BK = 16, GS_THREADS = 256, GS_PAD = 4;

// AK: A is contiguous along k (else along m). BNC: B is contiguous along n (else along k).
// SPLIT > 1: blockIdx.z / NB selects a k range and the tile goes to `partial` instead of f.epi.
template <class F, bool AK, bool BNC, int SPLIT>
__device__ __forceinline__ void gemm_simt_tile(const F &f, float *__restrict__ partial) {
    __shared__ __align__(16) float As[2][GS_BK][GS_BM + GS_PAD];
    __shared__ __align__(16) float Bs[2][GS_BK][GS_BN + GS_PAD];
    constexpr int M = F::M, N = F::N, K = F::K;
    constexpr int TILES_N = (N + GS_BN - 1) / GS_BN;
    const int t = threadIdx.x;
    const int tile_m = blockIdx.x / TILES_N, tile_n = blockIdx.x % TILES_N;
    const int bt = SPLIT > 1 ? blockIdx.y / SPLIT : blockIdx.y;
    const int sp = SPLIT > 1 ? blockIdx.y % SPLIT : 0;
    constexpr int KCH = ((K + SPLIT - 1) / SPLIT + GS_BK - 1) / GS_BK * GS_BK;   // k range of one split
    const int k_begin = sp * KCH;
    const int k_end = min(K, k_begin + KCH);
    const int m0 = tile_m * GS_BM, n0 = tile_n * GS_BN;

    float ra[8], rb[8];                    // global -> register staging (8 elements per operand per thread)
    auto fetch = [&](int k0) {
#pragma unroll
        for (int r = 0; r < 8; r++) {
            int mm, kk;
            if (AK) { kk = t % GS_BK; mm = t / GS_BK + (GS_THREADS / GS_BK) * r; }
            else { mm = t % GS_BM; kk = t / GS_BM + (GS_THREADS / GS_BM) * r; }
            const int m = m0 + mm, k = k0 + kk;
            ra[r] = (m < M && k < k_end) ? f.a(m, k, bt) : 0.0f;
            int nn, kb;
            if (BNC) { nn = t % GS_BN; kb = t / GS_BN + (GS_THREADS / GS_BN) * r; }
            else { kb = t % GS_BK; nn = t / GS_BK + (GS_THREADS / GS_BK) * r; }
            const int n = n0 + nn, k2 = k0 + kb;
            rb[r] = (n < N && k2 < k_end) ? f.b(k2, n, bt) : 0.0f;
        }
    };
    auto stage = [&](int buf) {
#pragma unroll
        for (int r = 0; r < 8; r++) {
            int mm, kk;
            if (AK) { kk = t % GS_BK; mm = t / GS_BK + (GS_THREADS / GS_BK) * r; }
            else { mm = t % GS_BM; kk = t / GS_BM + (GS_THREADS / GS_BM) * r; }
            As[buf][kk][mm] = ra[r];
            int nn, kb;
            if (BNC) { nn = t % GS_BN; kb = t / GS_BN + (GS_THREADS / GS_BN) * r; }
            else { kb = t % GS_BK; nn = t / GS_BK + (GS_THREADS / GS_BK) * r; }
            Bs[buf][kb][nn] = rb[r];
        }
    };

    const int tx = t % 16, ty = t / 16;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

    int buf = 0;
    if (k_begin < k_end) {
        fetch(k_begin);
        stage(0);
    }
    __syncthreads();
    for (int k0 = k_begin; k0 < k_end; k0 += GS_BK) {
        const bool more = k0 + GS_BK < k_end;
        if (more) fetch(k0 + GS_BK);
#pragma unroll
        for (int kk = 0; kk < GS_BK; kk++) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4 + 64]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4 + 64]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
        }
        if (more) stage(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }

#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int n = n0 + tx * 4 + (j & 3) + (j >> 2) * 64;
            if (n >= N) continue;
            if (SPLIT > 1) partial[(((long)bt * SPLIT + sp) * M + m) * N + n] = acc[i][j];
            else f.epi(m, n, bt, acc[i][j] * F::ALPHA);
        }
    }
}

// Second pass of a split-k product: partial tiles are added in split order, then the statements run.
template <class F, int SPLIT>
__device__ __forceinline__ void gemm_split_finish(const F &f, const float *__restrict__ partial) {
    constexpr long MN = (long)F::M * F::N;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < MN * F::NB; i += (long)gridDim.x * blockDim.x) {
        const int bt = (int)(i / MN);
        const long mn = i % MN;
        const int m = (int)(mn / F::N), n = (int)(mn % F::N);
        float ld[F::NLD > 0 ? F::NLD : 1];
        if (F::NLD > 0) f.epi_loads(m, n, bt, ld);          // what the statements read, before the first store
        float acc = 0.0f;
#pragma unroll 4
        for (int s = 0; s < SPLIT; s++) acc += partial[((long)bt * SPLIT + s) * MN + mn];
        f.epi2(m, n, bt, acc * F::ALPHA, ld);
    }
}

}  // namespace anvil
