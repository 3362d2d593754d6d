// exact_math.cuh -- double-precision exp/log kernels that reproduce, value for value, what the
// reference CPU decoder's `float sum += exp(float)` / `max + log(sum)` arithmetic produces
// (src/decode_cpu.c:45-49), at a fraction of the cost of a full libm exp/log.
//
// Why this exists: decoded moves change in a few percent of chunks when the backward scores
// differ from the CPU's by single float ulps, so the backward scan must land on the same
// float after every rounding the CPU performs.  The CPU rounds (a) each running-sum update to
// float and (b) the final max+log(sum) to float; both roundings are decided correctly as long
// as exp/log are accurate to far below half a float ulp.  The fast routines below (first tier) are
// accurate to 2^-43 and 2^-48, which leaves a rounding undecided about once in 2^20 (and harmless
// far more often than not: a running sum off by an ulp moves the result only if that in turn sits
// within 2^-23 of a boundary).  Built with -DOFX_RIGOROUS=1 the routines close that gap with two
// tiers (Ziv's strategy):
//   1. the fast routines, accurate to 2^-43 (exp, relative, on [-80, 2]) and 2^-48 (log,
//      absolute, on [1, 8)).  Every emulated rounding also measures how close the value was to a
//      rounding boundary; when it was closer than the routines' own error can bridge (about one
//      rounding in 2^16) the evaluation is not trusted and
//   2. is redone with routines accurate to 2^-51 (two-part argument reduction, longer
//      polynomials).
// What is left undecided after that are values within about 2^-50 of a boundary in units of the
// float's half ulp^-1, i.e. about one rounding in 2^26, and there the reference's own result hangs
// on the last bit of its libm's exp and log: nothing short of that libm's code can do better.
// The rigorous build is not the default: its checks are a few integer instructions per rounding,
// but every way of hanging the rarely needed second tier onto these routines (inlined behind a
// branch, or out of line) cost the scans 20 to 30 % of their time on a B200 with nvcc 12.9,
// measured; the default build runs the first tier alone, and the host tests run both.
//
// The same source compiles for the host (plain C++) so the arithmetic can be checked against
// the CPU oracle without a GPU; every operation is an explicitly rounded IEEE operation
// (fma / add / mul, no contraction), so host and device agree bit for bit.
#pragma once
#include <stdint.h>
#include <string.h>
#include <math.h>

#ifndef OFX_RIGOROUS
#define OFX_RIGOROUS 0
#endif

#ifdef __CUDACC__
#define OFX_HD __host__ __device__ __forceinline__
// (the rarely taken second steps; inlined like everything else: an out-of-line call inside the
// scan's loops cost far more, taken or not, than the instructions it kept out of them)
#define OFX_HD_RARE __host__ __device__ __forceinline__
#else
#define OFX_HD static inline
#define OFX_HD_RARE static __attribute__((noinline))
#endif

namespace ofx {

// Tables: 2^(j/64) for the exp; reciprocal and logarithm of interval centres for the log
// (64 intervals per binade over [1,8)).  Filled once on the host by fill_tables().
constexpr int kExpTab = 64;
constexpr int kLogTab = 192;
struct Tables {
    double exp2_j[kExpTab];
    double rcp_c[kLogTab];
    double log_c[kLogTab];
};

inline void fill_tables(Tables *t) {
    for (int j = 0; j < kExpTab; ++j) t->exp2_j[j] = exp2((double)j / kExpTab);
    for (int i = 0; i < kLogTab; ++i) {
        const double c = ldexp(1.0 + ((i & 63) + 0.5) / 64.0, i >> 6);
        t->rcp_c[i] = 1.0 / c;
        t->log_c[i] = log(c);
    }
    // The first interval is expanded about 1 itself: log(y) is then exact for y = 1 and carries
    // a relative, not an absolute, error for y just above 1.  That matters because sums of the
    // form 1 + k*2^-23 (one dominant term) put max + log(sum) within k^2 * 2^-47 of a rounding
    // tie whenever the maximum is a round number, as it is on the first timestep.
    t->rcp_c[0] = 1.0;
    t->log_c[0] = 0.0;
}

OFX_HD double d_fma(double a, double b, double c) {
#ifdef __CUDA_ARCH__
    return __fma_rn(a, b, c);
#else
    return fma(a, b, c);
#endif
}
OFX_HD double d_add(double a, double b) {
#ifdef __CUDA_ARCH__
    return __dadd_rn(a, b);
#else
    return a + b;
#endif
}
OFX_HD double d_mul(double a, double b) {
#ifdef __CUDA_ARCH__
    return __dmul_rn(a, b);
#else
    return a * b;
#endif
}
OFX_HD double make_double(uint32_t hi, uint32_t lo) {
#ifdef __CUDA_ARCH__
    return __hiloint2double((int)hi, (int)lo);
#else
    const uint64_t u = ((uint64_t)hi << 32) | lo;
    double d;
    memcpy(&d, &u, 8);
    return d;
#endif
}
OFX_HD uint32_t hi_word(double d) {
#ifdef __CUDA_ARCH__
    return (uint32_t)__double2hiint(d);
#else
    uint64_t u;
    memcpy(&u, &d, 8);
    return (uint32_t)(u >> 32);
#endif
}
OFX_HD uint32_t lo_word(double d) {
#ifdef __CUDA_ARCH__
    return (uint32_t)__double2loint(d);
#else
    uint64_t u;
    memcpy(&u, &d, 8);
    return (uint32_t)u;
#endif
}
OFX_HD uint32_t f_bits(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

// exp(-a) for a in [0, 80], a given as a double.  Argument reduction -a = n*ln2/64 + r with
// |r| <= ln2/128, table 2^(j/64), degree-4 Taylor polynomial (truncation < 2^-44).  8 FP64
// operations.  `tab` holds Tables::exp2_j with entry j at tab[j * stride] (any address space; a
// kernel may interleave per-lane copies of the table to keep shared-memory reads conflict free).
constexpr double kExpMagic = 6755399441055744.0;  // 1.5 * 2^52: low word of (x + magic) = rint(x)
constexpr double kExpInvStep = 92.33248261689365807103517958412;   // 64 / ln 2
constexpr double kExpStep = 0.010830424696249145097324535177;      // ln 2 / 64
// exp(x) for x in [-80, 4]: the same reduction with x = n*ln2/64 + r.
OFX_HD double exp_of(double x, const double *tab, int stride = 1) {
    const double t = d_fma(x, kExpInvStep, kExpMagic);
    const int n = (int)lo_word(t);
    const double nd = d_add(t, -kExpMagic);
    const double r = d_fma(nd, -kExpStep, x);
    double p = d_fma(r, 1.0 / 24.0, 1.0 / 6.0);
    p = d_fma(p, r, 0.5);
    p = d_fma(p, r, 1.0);
    p = d_fma(p, r, 1.0);
    const double e = d_mul(tab[(n & 63) * stride], p);
    // scale by 2^(n >> 6): results stay far inside the normal range for -80 <= x <= 4
    return make_double(hi_word(e) + ((uint32_t)(n & ~63) << 14), lo_word(e));
}
// exp(-a), a in [0, 80]: exp_of(-a) operation for operation, with the negations folded into the operands.
OFX_HD double exp_neg(double a, const double *tab, int stride = 1) {
    const double t = d_fma(a, -kExpInvStep, kExpMagic);
    const int n = (int)lo_word(t);  // <= 0
    const double nd = d_add(t, -kExpMagic);
    const double r = d_fma(nd, -kExpStep, -a);
    double p = d_fma(r, 1.0 / 24.0, 1.0 / 6.0);
    p = d_fma(p, r, 0.5);
    p = d_fma(p, r, 1.0);
    p = d_fma(p, r, 1.0);
    const double e = d_mul(tab[(n & 63) * stride], p);
    return make_double(hi_word(e) + ((uint32_t)(n & ~63) << 14), lo_word(e));
}

// The second tier's exp, same domain: the step ln2/64 in two parts (the first has 21 trailing zero
// bits, so n times it is exact for |n| < 2^20), degree-7 polynomial; what is left is the rounding
// of the table entry, of the polynomial's last steps and of the product: below 2^-51 relative.
constexpr double kExpStepHi = 0x1.62e42ffp-7;                // ln2/64 rounded to 32 significant bits
constexpr double kExpStepLo = -6.563929801064194889347411e-13;  // ln2/64 - kExpStepHi
OFX_HD double exp_of_t2(double x, const double *tab, int stride = 1) {
    const double t = d_fma(x, kExpInvStep, kExpMagic);
    const int n = (int)lo_word(t);
    const double nd = d_add(t, -kExpMagic);
    double r = d_fma(nd, -kExpStepHi, x);  // (the product is exact, the sum rounded below 2^-60)
    r = d_fma(nd, -kExpStepLo, r);
    double p = d_fma(r, 1.0 / 5040.0, 1.0 / 720.0);
    p = d_fma(p, r, 1.0 / 120.0);
    p = d_fma(p, r, 1.0 / 24.0);
    p = d_fma(p, r, 1.0 / 6.0);
    p = d_fma(p, r, 0.5);
    p = d_fma(p, r, 1.0);
    p = d_fma(p, r, 1.0);
    const double e = d_mul(tab[(n & 63) * stride], p);
    return make_double(hi_word(e) + ((uint32_t)(n & ~63) << 14), lo_word(e));
}

// log(y) for y in [1, 8).  y = c*(1+u) with c the centre of y's 1/64-binade interval (the
// first interval's lower end, 1, instead of its centre); log1p(u) by a degree-7 Taylor
// polynomial, |u| <= 2^-7 (first interval: 0 <= u < 2^-6, truncation < 2^-51).  8 FP64 operations.
OFX_HD double log_1to8(double y, const double *rcp_c, const double *log_c) {
    // y outside [1,8) (only possible for non-finite or garbage inputs) is pinned to the table's
    // ends so the lookup can never leave it
    uint32_t i = (hi_word(y) >> 14) - (1023u << 6);
    i = i < (uint32_t)kLogTab ? i : (uint32_t)(kLogTab - 1);
    const double u = d_fma(y, rcp_c[i], -1.0);
    double p = d_fma(u, 1.0 / 7.0, -1.0 / 6.0);
    p = d_fma(p, u, 0.2);
    p = d_fma(p, u, -0.25);
    p = d_fma(p, u, 1.0 / 3.0);
    p = d_fma(p, u, -0.5);
    p = d_fma(p, u, 1.0);
    return d_fma(p, u, log_c[i]);
}

// The second tier's log, same domain: two more terms (truncation below 2^-60 in every interval);
// what is left is the rounding of the two table entries and of the last steps: below 2^-51.
OFX_HD double log_1to8_t2(double y, const double *rcp_c, const double *log_c) {
    uint32_t i = (hi_word(y) >> 14) - (1023u << 6);
    i = i < (uint32_t)kLogTab ? i : (uint32_t)(kLogTab - 1);
    const double u = d_fma(y, rcp_c[i], -1.0);
    double p = d_fma(u, 1.0 / 9.0, -1.0 / 8.0);
    p = d_fma(p, u, 1.0 / 7.0);
    p = d_fma(p, u, -1.0 / 6.0);
    p = d_fma(p, u, 0.2);
    p = d_fma(p, u, -0.25);
    p = d_fma(p, u, 1.0 / 3.0);
    p = d_fma(p, u, -0.5);
    p = d_fma(p, u, 1.0);
    return d_fma(p, u, log_c[i]);
}

// Round a positive normal-range double to the nearest float (ties to even), keeping the
// result in a double: identical to (double)(float)y but with two FP64 adds and two integer
// operations instead of two conversions.
OFX_HD double round_to_f32(double y) {
    const double c = make_double((hi_word(y) & 0x7ff00000u) + 0x01d80000u, 0u);
    return d_add(d_add(y, c), -c);
}

// The same, also reporting whether y lay so close to the midpoint of two floats that an error of
// 2^-16 half ulps in y could have changed the result (`near` is only ever set, never cleared).
// A float keeps the top 23 of a double's 52 mantissa bits; the other 29 say where y lies between
// two floats, 2^28 being the midpoint: the test looks at those bits and costs no FP64 operation.
OFX_HD bool near_float_midpoint(double y, uint32_t window) {
    const uint32_t low = lo_word(y) & 0x1fffffffu;
    return low - (0x10000000u - window) < 2u * window;
}
OFX_HD double round_to_f32_flag(double y, bool &near) {
    near = near || near_float_midpoint(y, 1u << 12);  // 2^12 / 2^28 = 2^-16 of half an ulp
    return round_to_f32(y);
}

// Where a routine finds the tables (host: the Tables struct itself; device: shared memory).
struct TabRef {
    const double *exp2_j;  // entry j at exp2_j[j * exp_stride]
    int exp_stride;
    const double *rcp_c;
    const double *log_c;
};
OFX_HD TabRef ref_of(const Tables *t) {
    TabRef r = {t->exp2_j, 1, t->rcp_c, t->log_c};
    return r;
}

// The last rounding, (float)r with r = m + log(s) in double: was r so close to the midpoint of two
// floats that an error of abs_err in the logarithm (this tier's own plus the reference libm's) or
// the rounding of the double sum itself (2^-53 |r|) could have decided?  In units of the double's
// last mantissa bit, 2^(E-52) for 2^E <= |r| < 2^(E+1), those two are abs_err * 2^(52-E) and 1/2:
// with abs_err = 2^-W the window is 2^(52-W-E) + 8 units for E >= -4 (a power of two, given by the
// caller for E = -4, covers all of them), and smaller results (the first timestep or two) simply
// count as near.
OFX_HD bool last_rounding_is_near(double r, uint32_t window) {
    const uint32_t e = (hi_word(r) >> 20) & 0x7ffu;
    return e < 1023u - 4u || e > 1023u + 120u || near_float_midpoint(r, window);  // (NaN, infinity: near)
}
constexpr uint32_t kLogWindow = 1u << 11;   // abs_err 2^-46: 2^(52-46+4) + 8 < 2^11
constexpr uint32_t kFoldWindow = 1u << 15;  // abs_err 2^-42: 2^(52-42+4) + 8 < 2^15

// The reference's five-term log-sum-exp (src/decode_cpu.c:37-49, 93-108):
//   m = max v[i];  s = 0f;  for i in 0..4: s = (float)(s + exp((double)(v[i] - m)));
//   return (float)(m + log((double)s));
// First tier; `near` reports that one of the six roundings came too close to a boundary for this
// tier's accuracy (2^-43 in the exponentials, 2^-48 in the logarithm) to be trusted.
OFX_HD float lse5_tier1(const float v[5], const TabRef t, bool &near) {
    float m = v[0];
#pragma unroll
    for (int i = 1; i < 5; ++i) m = m > v[i] ? m : v[i];
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        float a = m - v[i];          // = -(v[i] - m) exactly
        a = a < 80.0f ? a : 80.0f;   // exp(-80) is far below anything a float sum >= 1 can see
        const double e = exp_neg((double)a, t.exp2_j, t.exp_stride);
        // (the maximum's own term is exp(0) = 1 exactly, here and in the reference: a tie it
        // produces is a true tie, settled the same way on both sides, and nothing to worry about)
        bool tie = false;
        s = round_to_f32_flag(i == 0 ? e : d_add(s, e), tie);
        near = near || (tie && a != 0.0f);
    }
    const double l = log_1to8(s, t.rcp_c, t.log_c);
    const double r = d_add((double)m, l);
    const float out = (float)r;
    near = near || last_rounding_is_near(r, kLogWindow);
    return out;
}

// Second tier, same arithmetic with the more accurate routines.  (The five terms arrive by value:
// a caller's array whose address went to a function that is not inlined would have to live in
// local memory for all of its life.)
OFX_HD_RARE float lse5_tier2(float v0, float v1, float v2, float v3, float v4, const TabRef t) {
    const float v[5] = {v0, v1, v2, v3, v4};
    float m = v[0];
#pragma unroll
    for (int i = 1; i < 5; ++i) m = m > v[i] ? m : v[i];
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        float a = m - v[i];
        a = a < 80.0f ? a : 80.0f;
        const double e = exp_of_t2(-(double)a, t.exp2_j, t.exp_stride);
        s = round_to_f32(i == 0 ? e : d_add(s, e));
    }
    return (float)d_add((double)m, log_1to8_t2(s, t.rcp_c, t.log_c));
}

// First tier with its checks, second tier behind it; out of line, for the callers below that need
// it once in a hundred evaluations.
OFX_HD_RARE float lse5_careful(float v0, float v1, float v2, float v3, float v4, const TabRef t) {
    const float v[5] = {v0, v1, v2, v3, v4};
    bool near = false;
    const float r = lse5_tier1(v, t, near);
    return near ? lse5_tier2(v0, v1, v2, v3, v4, t) : r;
}

// The routine for single evaluations (one state per lane): the first tier's arithmetic without the
// per-rounding checks, and one look at the result instead.  Whatever happens in the five roundings
// of the running sum moves it by at most five float ulps, i.e. the logarithm by less than 2^-20.6:
// a result further than 2^-20 from every midpoint of two floats is therefore right whatever those
// roundings did.  That settles all but 2^-19 / ulp(result) of the evaluations (under one in a
// hundred once the scores have passed 2048); the rest, and results below 32, go through lse5_careful.
// `wanted` = false (a lane of a warp that only keeps its neighbours company) skips that second step:
// a warp pays for it as soon as one of its lanes takes it.
OFX_HD float lse5_exact(const float v[5], const TabRef t, bool wanted = true) {
    (void)wanted;
    float m = v[0];
#pragma unroll
    for (int i = 1; i < 5; ++i) m = m > v[i] ? m : v[i];
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        float a = m - v[i];          // = -(v[i] - m) exactly
        a = a < 80.0f ? a : 80.0f;   // exp(-80) is far below anything a float sum >= 1 can see
        const double e = exp_neg((double)a, t.exp2_j, t.exp_stride);
        s = i == 0 ? round_to_f32(e) : round_to_f32(d_add(s, e));
    }
    const double r = d_add((double)m, log_1to8(s, t.rcp_c, t.log_c));
#if OFX_RIGOROUS
    // 2^-20 in units of r's last mantissa bit, 2^(E-52): 2^(32-E); the window test needs E >= 5
    const uint32_t e = (hi_word(r) >> 20) & 0x7ffu;
    const bool far = e >= 1023u + 5u && e < 1023u + 32u && !near_float_midpoint(r, (1u << (1023u + 32u - e)) + 8u);
    return (far || !wanted) ? (float)r : lse5_careful(v[0], v[1], v[2], v[3], v[4], t);
#else
    return (float)r;
#endif
}

// Is `guess` certainly the float the reference's arithmetic yields for the terms v?  Meant for a
// guess that is right nearly always: it takes the logarithm off the chain of dependent operations.
// With m the maximum and S the reference's float running sum, the result is `guess` exactly when
// m + log(S) lies between the midpoints that separate the guess from its two neighbouring floats,
// i.e. when exp(mid_below - m) <= S < exp(mid_above - m); the two thresholds do not depend on S
// and are evaluated beside the five exponentials of the sum.  A margin of 2^-34 (relative, on S)
// covers the error of the exponentials here (2^-43), of the reference's logarithm (2^-52) and of
// its double addition m + log(S) (2^-53 |m|, below 2^-38 for |m| < 2^15).  `false` means "not
// certain" (a wrong guess, a value inside the margin, a rounding of the running sum too close to
// a boundary, magnitudes outside the routine's range), never "wrong": the caller then computes
// the value with lse5_exact.
OFX_HD bool lse5_confirm(const float v[5], float guess, const TabRef t) {
    float m = v[0];
#pragma unroll
    for (int i = 1; i < 5; ++i) m = m > v[i] ? m : v[i];
    const uint32_t gb = f_bits(guess), mag = gb & 0x7fffffffu;
    const uint32_t mm = f_bits(m) & 0x7fffffffu;
    // 2^-8 <= |guess| < 2^15 (neighbours are then one bit pattern away on either side), |m| < 2^15
    if (mag < 0x3b800000u || mag >= 0x47000000u || mm >= 0x47000000u) return false;
    const bool neg = (gb >> 31) != 0;
    float above, below;
    {
        const uint32_t away = gb + 1u, toward = gb - 1u;  // away from / toward zero
        uint32_t ua = neg ? toward : away, ub = neg ? away : toward;
#ifdef __CUDA_ARCH__
        above = __uint_as_float(ua);
        below = __uint_as_float(ub);
#else
        memcpy(&above, &ua, 4);
        memcpy(&below, &ub, 4);
#endif
    }
    const double g = (double)guess, md = (double)m;
    const double tau_hi = d_add(d_mul(0.5, d_add(g, (double)above)), -md);  // exact
    const double tau_lo = d_add(d_mul(0.5, d_add(g, (double)below)), -md);  // exact
    if (!(tau_lo > -1.0 && tau_hi < 3.0)) return false;
    const double e_hi = exp_of(tau_hi, t.exp2_j, t.exp_stride);
    const double e_lo = exp_of(tau_lo, t.exp2_j, t.exp_stride);
    bool near = false;
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        float a = m - v[i];
        a = a < 80.0f ? a : 80.0f;
        const double e = exp_neg((double)a, t.exp2_j, t.exp_stride);
        // (the maximum's own term is exp(0) = 1 exactly, here and in the reference: a tie it
        // produces is a true tie, settled the same way on both sides, and nothing to worry about)
        bool tie = false;
        s = round_to_f32_flag(i == 0 ? e : d_add(s, e), tie);
        near = near || (tie && a != 0.0f);
    }
    const bool inside = d_mul(s, 1.0 - 0x1p-34) >= e_lo && d_mul(s, 1.0 + 0x1p-34) <= e_hi;
    return inside && !near;
}

// K independent five-term log-sum-exps at once, same arithmetic as lse5_exact.  The work is
// written stage by stage across all 5K exponentials so that the FP64 pipe always has
// independent operations in flight (one lse5_exact after another leaves it waiting on its own
// dependency chain most of the time).
template <int K>
OFX_HD void lse5_batch_exact(const float (*v)[5], float *out, const TabRef t) {
    float m[K];
    double x[K * 5], r[K * 5], p[K * 5];
    int n[K * 5];
#pragma unroll
    for (int k = 0; k < K; ++k) {
        m[k] = v[k][0];
#pragma unroll
        for (int i = 1; i < 5; ++i) m[k] = m[k] > v[k][i] ? m[k] : v[k][i];
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            float a = m[k] - v[k][i];
            a = a < 80.0f ? a : 80.0f;
            x[k * 5 + i] = (double)a;  // exact; one conversion instead of three integer operations
        }
    }
#pragma unroll
    for (int q = 0; q < K * 5; ++q) p[q] = d_fma(x[q], -kExpInvStep, kExpMagic);
#pragma unroll
    for (int q = 0; q < K * 5; ++q) {
        n[q] = (int)lo_word(p[q]);
        r[q] = d_add(p[q], -kExpMagic);
    }
#pragma unroll
    for (int q = 0; q < K * 5; ++q) r[q] = d_fma(r[q], -kExpStep, -x[q]);
#pragma unroll
    for (int q = 0; q < K * 5; ++q) p[q] = d_fma(r[q], 1.0 / 24.0, 1.0 / 6.0);
#pragma unroll
    for (int q = 0; q < K * 5; ++q) p[q] = d_fma(p[q], r[q], 0.5);
#pragma unroll
    for (int q = 0; q < K * 5; ++q) p[q] = d_fma(p[q], r[q], 1.0);
#pragma unroll
    for (int q = 0; q < K * 5; ++q) p[q] = d_fma(p[q], r[q], 1.0);
#pragma unroll
    for (int q = 0; q < K * 5; ++q) {
        const double e = d_mul(t.exp2_j[(n[q] & 63) * t.exp_stride], p[q]);
        p[q] = make_double(hi_word(e) + ((uint32_t)(n[q] & ~63) << 14), lo_word(e));
    }
    double s[K];
#if OFX_RIGOROUS
    bool near[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
        near[k] = false;
        s[k] = round_to_f32_flag(p[k * 5], near[k]);
        near[k] = near[k] && x[k * 5] != 0.0;  // (exp(0) = 1 exactly: its ties are true ties)
    }
#pragma unroll
    for (int i = 1; i < 5; ++i) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
            bool tie = false;
            s[k] = round_to_f32_flag(d_add(s[k], p[k * 5 + i]), tie);
            near[k] = near[k] || (tie && x[k * 5 + i] != 0.0);
        }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const double r = d_add((double)m[k], log_1to8(s[k], t.rcp_c, t.log_c));
        out[k] = (float)r;
        near[k] = near[k] || last_rounding_is_near(r, kLogWindow);
    }
    // (about one evaluation in ten thousand)
#pragma unroll
    for (int k = 0; k < K; ++k)
        if (near[k]) out[k] = lse5_tier2(v[k][0], v[k][1], v[k][2], v[k][3], v[k][4], t);
#else
#pragma unroll
    for (int k = 0; k < K; ++k) s[k] = round_to_f32(p[k * 5]);
#pragma unroll
    for (int i = 1; i < 5; ++i) {
#pragma unroll
        for (int k = 0; k < K; ++k) s[k] = round_to_f32(d_add(s[k], p[k * 5 + i]));
    }
#pragma unroll
    for (int k = 0; k < K; ++k)
        out[k] = (float)d_add((double)m[k], log_1to8(s[k], t.rcp_c, t.log_c));
#endif
}

OFX_HD_RARE float fold2_tier2(float m, float d, const TabRef t) {
    const double e2 = exp_of_t2(-(double)d, t.exp2_j, t.exp_stride);
    return (float)d_add((double)m, log_1to8_t2(d_add(1.0, e2), t.rcp_c, t.log_c));
}

// The reference's two-term fold used when beam elements merge (src/beam_search.c:43-47):
//   d = |x - y| (float);  m = max;  return (float)(m + (d < 17 ? log(1.0 + exp(-(double)d)) : 0))
// (the sum 1 + exp(-d) is a double there, so the only float rounding is the last one)
OFX_HD float fold2_exact(float x, float y, const TabRef t) {
    const float d = fabsf(x - y);
    const float m = x > y ? x : y;
    if (!(d < 17.0f)) return m;
    const double e = exp_neg((double)d, t.exp2_j, t.exp_stride);
    const double r = d_add((double)m, log_1to8(d_add(1.0, e), t.rcp_c, t.log_c));
    const float out = (float)r;
#if OFX_RIGOROUS
    if (last_rounding_is_near(r, kFoldWindow)) return fold2_tier2(m, d, t);  // (the exponential's 2^-43 reaches the logarithm here)
#endif
    return out;
}

}  // namespace ofx
