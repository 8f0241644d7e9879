// anvil_device.cuh — device-side helpers that every generated kernel includes: the scalar
// semantics of the IR, the fault record, and the fixed-order warp / block reductions.
//
// Scalar semantics restate anvil/backend/anvil_host.h:31-53 (which in turn follows
// anvil/interp.py:575-632): Python floor division and modulo with a zero divisor counted as 1,
// nan-propagating max/min, sign(0) = 0, truncating float -> int.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "anvil_rng.h"

#define ANVIL_DEV __device__ __forceinline__

namespace anvil {

struct Fault { int code; int pad; long long value; };

// First failed bounds check wins; the kernel carries on with a clamped index and the host reports
// the fault at its next synchronisation (anvil/backend/anvil_cuda.h:66-80).
ANVIL_DEV void fail(Fault *f, int code, long long value) {
    if (atomicCAS(&f->code, 0, code) == 0) f->value = value;
}

ANVIL_DEV long gather_index(const int *__restrict__ p, long off, long lo, long hi, Fault *f, int code) {
    long v = (long)p[off];
    if (v < lo || v >= hi) { fail(f, code, v); v = lo; }
    return v;
}

ANVIL_DEV int idiv(int a, int b) {
    if (b == 0) b = 1;
    int q = a / b, r = a % b;
    return (r != 0 && ((r < 0) != (b < 0))) ? q - 1 : q;
}
ANVIL_DEV int imod(int a, int b) {
    if (b == 0) b = 1;
    int r = a % b;
    return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r;
}
ANVIL_DEV float fmod_py(float a, float b) {
    float r = fmodf(a, b);
    return (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) ? r + b : r;
}
ANVIL_DEV float fmax_nan(float a, float b) { return (a != a || b != b) ? CUDART_NAN_F : (a > b ? a : b); }
ANVIL_DEV float fmin_nan(float a, float b) { return (a != a || b != b) ? CUDART_NAN_F : (a < b ? a : b); }
ANVIL_DEV int imax(int a, int b) { return a > b ? a : b; }
ANVIL_DEV int imin(int a, int b) { return a < b ? a : b; }
ANVIL_DEV float fsign(float a) { return a > 0 ? 1.0f : (a < 0 ? -1.0f : a); }
ANVIL_DEV int isign(int a) { return a > 0 ? 1 : (a < 0 ? -1 : 0); }
ANVIL_DEV float sigmoid(float a) { return 1.0f / (1.0f + expf(-a)); }
ANVIL_DEV int f2i(float a) { return (int)truncf(a); }

// ---------------------------------------------------------------------------- reductions
// Combine operators. Every tree below has a shape fixed by the launch geometry alone, so a kernel
// gives the same bits on every run.
struct OpSum { template <typename T> ANVIL_DEV static T id() { return (T)0; }
               template <typename T> ANVIL_DEV static T f(T a, T b) { return a + b; } };
struct OpProd { template <typename T> ANVIL_DEV static T id() { return (T)1; }
                template <typename T> ANVIL_DEV static T f(T a, T b) { return a * b; } };
struct OpMax {
    template <typename T> ANVIL_DEV static T id();
    ANVIL_DEV static float f(float a, float b) { return fmax_nan(a, b); }
    ANVIL_DEV static int f(int a, int b) { return imax(a, b); }
};
template <> ANVIL_DEV float OpMax::id<float>() { return -CUDART_INF_F; }
template <> ANVIL_DEV int OpMax::id<int>() { return (-2147483647 - 1); }
struct OpMin {
    template <typename T> ANVIL_DEV static T id();
    ANVIL_DEV static float f(float a, float b) { return fmin_nan(a, b); }
    ANVIL_DEV static int f(int a, int b) { return imin(a, b); }
};
template <> ANVIL_DEV float OpMin::id<float>() { return CUDART_INF_F; }
template <> ANVIL_DEV int OpMin::id<int>() { return 2147483647; }

template <typename Op, typename T>
ANVIL_DEV T warp_reduce(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = Op::f(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// All threads of the block get the result. `smem` holds at least 32 elements of T.
template <typename Op, typename T>
ANVIL_DEV T block_reduce(T v, T *smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_reduce<Op>(v);
    __syncthreads();                       // smem may still be in use by a previous reduction
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    T r = lane < nwarps ? smem[lane] : Op::template id<T>();
    return warp_reduce<Op>(r);
}

// Reduction over the T threads that share one row (T a power of two, 32 <= T <= 256, rows packed
// 256 / T to a CTA). Every thread of the row gets the result. Warps are combined in index order.
// `smem` holds 8 floats. Must be reached by all threads of the CTA.
template <typename Op, int T>
ANVIL_DEV float row_reduce(float v, float *smem) {
    v = warp_reduce<Op>(v);
    if (T == 32) return v;
    constexpr int WPR = T / 32;                      // warps per row
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) smem[w] = v;
    __syncthreads();
    const int w0 = (w / WPR) * WPR;
    float r = smem[w0];
#pragma unroll
    for (int i = 1; i < WPR; i++) r = Op::f(r, smem[w0 + i]);
    return r;
}

// argmax / argmin keep (value, flat reduction index); ties and equal values keep the smaller index,
// which reproduces "first index of the strict extremum" (anvil/backend/cuda.py:286-307).
template <typename T> struct Arg { T v; long i; };
template <bool IsMax, typename T>
ANVIL_DEV Arg<T> arg_pick(Arg<T> a, Arg<T> b) {
    bool take_b = IsMax ? (b.v > a.v) : (b.v < a.v);
    if (b.v == a.v) take_b = b.i < a.i;
    return take_b ? b : a;
}
template <bool IsMax, typename T>
ANVIL_DEV Arg<T> warp_arg_reduce(Arg<T> a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Arg<T> b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = arg_pick<IsMax>(a, b);
    }
    return a;
}

// Asks for the line holding *p to be brought into L2; never faults, returns nothing.
ANVIL_DEV void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
ANVIL_DEV void prefetch_l1(const void *p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

// ---------------------------------------------------------------------------- 128-bit access
ANVIL_DEV float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
ANVIL_DEV void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
ANVIL_DEV int4 ld4(const int *p) { return *reinterpret_cast<const int4 *>(p); }
ANVIL_DEV void st4(int *p, int4 v) { *reinterpret_cast<int4 *>(p) = v; }

}  // namespace anvil
