// Host build of the arithmetic the CUDA backward scan runs (openfish_b200/csrc/exact_math.cuh
// compiles for the host too), so its agreement with the CPU oracle can be checked bit for bit
// without a GPU.  Test code only.
#include "../../openfish_b200/csrc/exact_math.cuh"

static ofx::Tables g_tables;
static bool g_ready = false;
static const ofx::Tables *tables() {
    if (!g_ready) {
        ofx::fill_tables(&g_tables);
        g_ready = true;
    }
    return &g_tables;
}

// Same recursion as the kernel (and src/decode_cpu.c:13-52), one chunk.
extern "C" void host_backward_scan(const float *scores, float *bwd, int chunk, int T, int N, int ns) {
    const ofx::TabRef tr = ofx::ref_of(tables());
    const size_t row = (size_t)ns * 4;
    const float *cs = scores + (size_t)chunk * row;
    float *out = bwd + (size_t)chunk * (T + 1) * ns;
    for (int s = 0; s < ns; ++s) out[(size_t)T * ns + s] = 0.f;
    for (int t = T - 1; t >= 0; --t) {
        const float *sc = cs + (size_t)N * row * t;
        const float *nxt = out + (size_t)(t + 1) * ns;
        float *cur = out + (size_t)t * ns;
        // states are taken four at a time through the batched routine the kernel uses, and
        // every fourth group also through the one-at-a-time routine: both must agree
        for (int s0 = 0; s0 < ns; s0 += 4) {
            float v[4][5], res[4];
            for (int k = 0; k < 4; ++k) {
                const int s = s0 + k;
                const int u0 = (s * 4) % ns, col = u0 * 4 + (s * 4) / ns;
                v[k][0] = nxt[s] + 2.0f;
                for (int b = 0; b < 4; ++b) v[k][b + 1] = nxt[u0 + b] + sc[col + 4 * b];
            }
            ofx::lse5_batch_exact<4>(v, res, tr);
            for (int k = 0; k < 4; ++k) {
                if ((s0 & 12) == 0 && ofx::lse5_exact(v[k], tr) != res[k]) res[k] = -1.0f;
                cur[s0 + k] = res[k];
            }
        }
    }
}
extern "C" float host_fold2(float x, float y) { return ofx::fold2_exact(x, y, ofx::ref_of(tables())); }
extern "C" double host_exp_neg(double a) { return ofx::exp_neg(a, tables()->exp2_j); }
extern "C" double host_log_1to8(double y) { return ofx::log_1to8(y, tables()->rcp_c, tables()->log_c); }
extern "C" double host_round_to_f32(double y) { return ofx::round_to_f32(y); }

// single evaluations: the two-tier routine, its tiers on their own, the confirmation shortcut
extern "C" float host_lse5(const float *v) { return ofx::lse5_exact(v, ofx::ref_of(tables())); }
extern "C" float host_lse5_tier1(const float *v, int *near) {
    bool n = false;
    const float r = ofx::lse5_tier1(v, ofx::ref_of(tables()), n);
    *near = n;
    return r;
}
extern "C" float host_lse5_tier2(const float *v) { return ofx::lse5_tier2(v[0], v[1], v[2], v[3], v[4], ofx::ref_of(tables())); }
extern "C" int host_lse5_confirm(const float *v, float guess) { return ofx::lse5_confirm(v, guess, ofx::ref_of(tables())); }
extern "C" double host_exp_of(double x) { return ofx::exp_of(x, tables()->exp2_j); }
extern "C" double host_exp_of_t2(double x) { return ofx::exp_of_t2(x, tables()->exp2_j); }
extern "C" double host_log_1to8_t2(double y) { return ofx::log_1to8_t2(y, tables()->rcp_c, tables()->log_c); }
// many evaluations at once: out[i] = two-tier result, flags[i] = first tier asked for the second,
// confirmed[i] = the shortcut confirmed guess[i]
extern "C" void host_lse5_many(const float *v, const float *guess, int n, float *out, unsigned char *flags,
                               unsigned char *confirmed) {
    const ofx::TabRef tr = ofx::ref_of(tables());
    for (int i = 0; i < n; ++i) {
        bool near = false;
        const float r1 = ofx::lse5_tier1(v + 5 * i, tr, near);
        const float *w = v + 5 * i;
        out[i] = near ? ofx::lse5_tier2(w[0], w[1], w[2], w[3], w[4], tr) : r1;
        flags[i] = near;
        confirmed[i] = ofx::lse5_confirm(v + 5 * i, guess[i], tr);
    }
}
