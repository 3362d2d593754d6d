// exact_math.cuh -- double-precision exp/log kernels that reproduce, value for value, what the
// reference CPU decoder's `float sum += exp(float)` / `max + log(sum)` arithmetic produces
// (src/decode_cpu.c:45-49), at a fraction of the cost of a full libm exp/log.
//
// Why this exists: decoded moves change in a few percent of chunks when the backward scores
// differ from the CPU's by single float ulps, so the backward scan must land on the same
// float after every rounding the CPU performs.  The CPU rounds (a) each running-sum update to
// float and (b) the final max+log(sum) to float; both roundings are decided correctly as long
// as exp/log are accurate to far below half a float ulp.  The routines here are accurate to
// about 2^-44 absolute on their domains (exp on [-80,0], log on [1,8)), which leaves a
// mismatch probability per rounding of about 2^-22.
//
// The same source compiles for the host (plain C++) so the arithmetic can be checked against
// the CPU oracle without a GPU; every operation is an explicitly rounded IEEE operation
// (fma / add / mul, no contraction), so host and device agree bit for bit.
#pragma once
#include <stdint.h>
#include <string.h>
#include <math.h>

#ifdef __CUDACC__
#define OFX_HD __host__ __device__ __forceinline__
#else
#define OFX_HD static inline
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
    // scale by 2^(n >> 6): results stay far inside the normal range for a <= 80
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

// Round a positive normal-range double to the nearest float (ties to even), keeping the
// result in a double: identical to (double)(float)y but with two FP64 adds and two integer
// operations instead of two conversions.
OFX_HD double round_to_f32(double y) {
    const double c = make_double((hi_word(y) & 0x7ff00000u) + 0x01d80000u, 0u);
    return d_add(d_add(y, c), -c);
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

// The reference's five-term log-sum-exp (src/decode_cpu.c:37-49, 93-108):
//   m = max v[i];  s = 0f;  for i in 0..4: s = (float)(s + exp((double)(v[i] - m)));
//   return (float)(m + log((double)s));
OFX_HD float lse5_exact(const float v[5], const TabRef t) {
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
    return (float)r;
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
}

// The reference's two-term fold used when beam elements merge (src/beam_search.c:43-47):
//   d = |x - y| (float);  m = max;  return (float)(m + (d < 17 ? log(1.0 + exp(-(double)d)) : 0))
OFX_HD float fold2_exact(float x, float y, const TabRef t) {
    const float d = fabsf(x - y);
    const float m = x > y ? x : y;
    if (!(d < 17.0f)) return m;
    const double e = exp_neg((double)d, t.exp2_j, t.exp_stride);
    const double l = log_1to8(d_add(1.0, e), t.rcp_c, t.log_c);
    return (float)d_add((double)m, l);
}

}  // namespace ofx
