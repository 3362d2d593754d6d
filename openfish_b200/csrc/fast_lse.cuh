// fast_lse.cuh -- fp32 evaluation of the reference's five-term log-sum-exp that knows when it
// is right.
//
// The value-exact routine in exact_math.cuh costs about 63 FP64 operations per state and
// timestep.  Most of the time that effort is not needed to know which float the reference
// arithmetic produces: the result max + log(sum) is rounded to a float whose spacing grows with
// the magnitude of the scores (2^-12 once they pass 2048), while log(sum) can be had in fp32
// to about 2^-20.  So: evaluate log(sum) in fp32, widen it by a bound on every error that
// separates it from the reference's own value, add both ends of that interval to the maximum
// with one correctly rounded float addition each, and accept when both ends land on the same
// float (rounding is monotone, so the reference's result is pinned between them).  Otherwise
// the caller falls back to the value-exact routine.  Nothing is approximated in what is
// accepted.
//
// Error budget of log(sum), all relative to sum >= 1 (so also absolute in the logarithm), in
// units of 1e-7:
//   ex2.approx: 2 ulp = 2^-22 documented (2^-22.7 measured), weights sum to one        2.38
//   rounding of (v-m)*log2(e) before ex2, weighted by the term's size
//     (max a*exp(-a) = 0.37, 4 terms)                                                   0.88
//   four float additions here, each relative to a partial sum                           2.38
//   the reference's five float roundings of its running sum (decode_cpu.c:47)           2.98
//   lg2.approx on [1,8): at most 2^-21.75 absolute in log2, its own rounding included
//     (measured over every float of the interval: 2^-21.78), times ln 2                 1.96
//   rounding of the product with ln 2 and of l -+ eps (l < 2)                           1.19
// Sum 11.8 = 2^-19.7; kLseEps = 13.5 = 2^-19.5.  openfish_b200_selfcheck_arith repeats the two
// measurements on the GPU at hand and compares them with the bounds used here.
#pragma once
#include <cuda_runtime.h>

namespace ofd {

constexpr float kLseEps = 1.3487e-6f;  // 2^-19.5

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// maximum of three in one instruction (sm_100); a NaN operand loses against a number, as in fmaxf
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float max5(const float v[5]) { return max3(max3(v[0], v[1], v[2]), v[3], v[4]); }
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ln of s in [1, 8).
__device__ __forceinline__ float ln_1to8(float s) {
    const float kLn2 = 0.6931471805599453f;
    return lg2_approx(s) * kLn2;
}

// v: the five terms.  On success writes the reference-exact float to `out`.
__device__ __forceinline__ bool lse5_try_fast(const float v[5], float &out) {
    const float kLog2e = 1.4426950408889634f;
    const float m = max5(v);
    float s = ex2_approx((v[0] - m) * kLog2e);
    s += ex2_approx((v[1] - m) * kLog2e);
    s += ex2_approx((v[2] - m) * kLog2e);
    s += ex2_approx((v[3] - m) * kLog2e);
    s += ex2_approx((v[4] - m) * kLog2e);
    const float l = ln_1to8(s);
    const float lo = m + (l - kLseEps);
    const float hi = m + (l + kLseEps);
    out = lo;
    // A NaN or infinite term makes the sum NaN (an infinite maximum gives inf - inf in its own
    // term), the logarithm and both ends with it, and NaN compares unequal.
    return lo == hi;
}

}  // namespace ofd

#include "exact_math.cuh"

namespace ofd {

// K fast evaluations stage by stage.  out[k] is the certified result where ok[k], and otherwise
// the better of the two candidate floats (the one nearest to max + log(sum) as estimated), to be
// confirmed or corrected by the value-exact routine.
template <int K>
__device__ __forceinline__ void lse5_fast_guess(const float (*v)[5], float *out, bool *ok) {
    const float kLog2e = 1.4426950408889634f;
    float m[K], e[K][5], s[K], l[K];
#pragma unroll
    for (int k = 0; k < K; ++k)
        m[k] = max5(v[k]);
#pragma unroll
    for (int i = 0; i < 5; ++i)
#pragma unroll
        for (int k = 0; k < K; ++k) e[k][i] = ex2_approx((v[k][i] - m[k]) * kLog2e);
#pragma unroll
    for (int k = 0; k < K; ++k) s[k] = ((e[k][0] + e[k][1]) + (e[k][2] + e[k][3])) + e[k][4];
#pragma unroll
    for (int k = 0; k < K; ++k) {
        l[k] = ln_1to8(s[k]);
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const float lo = m[k] + (l[k] - kLseEps);
        const float hi = m[k] + (l[k] + kLseEps);
        out[k] = m[k] + l[k];
        ok[k] = lo == hi;  // (a NaN sum makes both ends NaN: never accepted)
    }
}

}  // namespace ofd
