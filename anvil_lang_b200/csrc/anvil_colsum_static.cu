// anvil_colsum_static.cu — column sums of a row-major f32 matrix without any allocation.
//
// out[j] = sum_i x[i * cols + j]. This is the split column reduction that the emitter generates for
// bias / gain gradients (32 consecutive outputs x 8 reduction slices per CTA, a shared-memory tree,
// several CTAs per output group whose partial sums are added in order by a second kernel). The
// generated kernels keep their partial sums in the scratch region of the cudaMalloc'd arena; this
// variant keeps them in a fixed array that is part of the library image, for callers that are not
// allowed to allocate device memory at the point of the call: code running inside a host framework
// that owns all device memory through its own pool, plug-ins loaded into a process whose memory
// budget is fixed at start-up, or latency-critical loops where an allocation (an implicit device
// synchronisation) is not acceptable.
//
// Costs and rules that follow from the fixed array:
//   * every GPU that loads libanvil_cuda.so holds ANVIL_COLSUM_STATIC_MAX_PARTIALS * 4 bytes (4 MiB)
//     until the process exits;
//   * cols * splits must not exceed ANVIL_COLSUM_STATIC_MAX_PARTIALS, else the call is refused;
//   * all calls share the array: two calls that overlap on the GPU (different streams, or different
//     host threads) race on it. Calls on one stream are ordered and safe. Nothing in it needs to start
//     at zero: the first kernel overwrites every partial sum the second kernel reads;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress) with
//     that device current; make that first call outside any stream capture.
#include "anvil_cuda.h"

#include <cuda_runtime.h>
#include <stdio.h>

static __device__ __align__(256) float g_colsum_partials[ANVIL_COLSUM_STATIC_MAX_PARTIALS];

namespace {

constexpr int OX = 32, RY = 8, MAX_DEVICES = 64;

__global__ void __launch_bounds__(OX * RY) colsum_part(const float *__restrict__ x, long rows, long cols, int splits,
                                                        long chunk, float *__restrict__ partials) {
    const int ox = threadIdx.x % OX, ry = threadIdx.x / OX;
    const long o = blockIdx.x * (long)OX + ox;
    const bool live = o < cols;
    const long col = live ? o : cols - 1;
    float acc = 0.0f;
    const long rbeg = blockIdx.y * chunk, rend = min(rows, rbeg + chunk);
    for (long r = rbeg + ry; r < rend; r += RY) acc = acc + x[r * cols + col];
    __shared__ float sm[RY][OX + 1];
    sm[ry][ox] = acc;
    __syncthreads();
    for (int s = RY / 2; s >= 1; s >>= 1) {
        if (ry < s) sm[ry][ox] = sm[ry][ox] + sm[ry + s][ox];
        __syncthreads();
    }
    if (ry == 0 && live) partials[o * splits + blockIdx.y] = sm[0][ox];
}

__global__ void __launch_bounds__(256) colsum_final(const float *__restrict__ partials, long cols, int splits,
                                                     float *__restrict__ out) {
    for (long j = blockIdx.x * 256L + threadIdx.x; j < cols; j += (long)gridDim.x * 256L) {
        float acc = 0.0f;
        for (int p = 0; p < splits; p++) acc = acc + partials[j * splits + p];
        out[j] = acc;
    }
}

float *g_partials_addr[MAX_DEVICES];      // device address of g_colsum_partials, per device

}  // namespace

extern "C" int anvil_colsum_f32_static(const float *x, long rows, long cols, float *out, void *cuda_stream) {
    // `out` is written whenever there is a column (zeros when there are no rows); `x` is read whenever there is an element
    if (rows < 0 || cols < 0 || (cols > 0 && !out) || (rows > 0 && cols > 0 && !x)) {
        fprintf(stderr, "anvil: anvil_colsum_f32_static: bad arguments\n");
        return 1;
    }
    if (cols == 0) return 0;
    // the split rule of the generated kernels: more CTAs per output group while the grid is small
    const long blocks = (cols + OX - 1) / OX;
    const long per_thread = rows / RY;
    long splits = 1;
    if (blocks < 148 && per_thread >= 64) {
        splits = 296 / blocks;
        if (per_thread / 32 < splits) splits = per_thread / 32;
        if (splits > 64) splits = 64;
        if (splits < 1) splits = 1;
    }
    if (cols * splits > (long)ANVIL_COLSUM_STATIC_MAX_PARTIALS) {
        fprintf(stderr, "anvil: anvil_colsum_f32_static: %ld columns x %ld splits exceed the fixed scratch of %ld partial sums\n",
                cols, splits, (long)ANVIL_COLSUM_STATIC_MAX_PARTIALS);
        return 2;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        fprintf(stderr, "anvil: anvil_colsum_f32_static: no usable current device\n");
        return 3;
    }
    if (!g_partials_addr[dev]) {               // once per device, with that device current
        float *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_colsum_partials);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "anvil: anvil_colsum_f32_static: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            return 3;
        }
        g_partials_addr[dev] = p;
    }
    float *partials = g_partials_addr[dev];
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const long chunk = (rows + splits - 1) / splits;
    colsum_part<<<dim3((unsigned)blocks, (unsigned)splits), OX * RY, 0, st>>>(x, rows, cols, (int)splits, chunk, partials);
    long fb = (cols + 255) / 256;
    if (fb > 1184) fb = 1184;
    colsum_final<<<(unsigned)fb, 256, 0, st>>>(partials, cols, (int)splits, out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "anvil: anvil_colsum_f32_static: launch failed: %s\n", cudaGetErrorString(e));
        return 3;
    }
    return 0;
}
