/*
 * crf_oracle.c -- CPU restatement of openfish's CRF-CTC decode and rotary embedding.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests, the smoke test and the
 * CPU-baseline leg of the benchmark compare the CUDA path against.  Nothing in the product
 * library links, loads or calls it, and the product has no CPU fallback.
 *
 * Parity status: PINNED.  The restatement is checked (tests/test_oracle.py) against
 *   - the reference's own golden vector (test/data/{scores,moves,sequence,qstring}.blob, the
 *     case test/test.sh:26-40 runs), stored as tests/golden/ref_fast_chunk.npz, and
 *   - outputs of the unmodified reference CPU decoder compiled from its own sources
 *     (oracle/Makefile -> oracle/_ref/), stored as tests/golden/synth_*.npz and re-checked
 *     live whenever oracle/_ref/ is present.
 *
 * Every function names the reference lines whose arithmetic it restates.  The arithmetic
 * (operand order, where a value is a float and where it is a double) follows the reference
 * exactly because decoded moves are sensitive to single-ulp changes of the backward scores.
 *
 * Layouts (the reference's):
 *   scores  [T][N][C]   float (the GPU path's fp16 values widened), the scans stride a
 *                       timestep by N*4*ns and a chunk by 4*ns regardless of C
 *                       (src/decode_cpu.c:16-18,27,59-62,80), the beam search strides a
 *                       timestep by N*C (src/decode_cpu.c:204,216)
 *   bwd/fwd/post [N][T+1][ns]  float
 *   moves/sequence/qstring [N][T], states [N][T] int32, qual [N][T][4]
 */
#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define OR_BASES 4
#define OR_BEAM 32
#define OR_CAND (5 * OR_BEAM)
#define OR_MAX_STATES 1024
#define OR_CRC_SEED 0x12345678u

typedef struct {
    uint64_t beam_width; /* ignored, like the reference (src/decode.h:49 fixes 32) */
    float beam_cut;
    float blank_score;
    float q_shift;
    float q_scale;
    float temperature; /* ignored by oracle_decode (src/decode_cpu.c:216 passes 1.0f); see oracle_decode_ex */
    uint8_t move_pad;  /* ignored */
} oracle_opt_t;

/* ---------------------------------------------------------------------------------------- */
/* scans                                                                                     */

/* Five-term log-sum-exp exactly as src/decode_cpu.c:37-49 and :93-108 compute it: float
 * differences, double exp, a float running sum that is rounded after every addition (terms
 * taken in index order), double log, one final rounding to float. */
static float lse5(const float v[5]) {
    float top = v[0];
    for (int i = 1; i < 5; ++i) top = top > v[i] ? top : v[i];
    float acc = 0.0f;
    for (int i = 0; i < 5; ++i) acc += exp(v[i] - top);
    return top + log(acc);
}

/* exported for the arithmetic checks of the CUDA path's log-sum-exp: n evaluations, v[5n] */
void oracle_lse5_many(const float *v, int n, float *out) {
    for (int i = 0; i < n; ++i) out[i] = lse5(v + 5 * i);
}

/* Backward scores of one chunk.  src/decode_cpu.c:13-52.  Row T is zero; row t is built from
 * row t+1.  State s can stay (fixed score 2.0f, :14) or move to u = (4s mod ns) + b; that
 * transition's score sits at column 4u + (4s div ns) of timestep t (:33-35,41-42).
 * The _stay variants take the stay score as an argument: the reference's CUDA launcher hands
 * its scans options->blank_score (src/decode_cuda.cu:115) where the CPU scans hard-code 2.0f. */
void oracle_backward_scan_stay(const float *scores, float *bwd, int chunk, int T, int N, int ns,
                               float stay) {
    const size_t row = (size_t)ns * OR_BASES;
    const float *cs = scores + (size_t)chunk * row;
    float *out = bwd + (size_t)chunk * (T + 1) * ns;
    for (int s = 0; s < ns; ++s) out[(size_t)T * ns + s] = 0.0f;
    for (int t = T - 1; t >= 0; --t) {
        const float *sc = cs + (size_t)N * row * t;
        const float *nxt = out + (size_t)(t + 1) * ns;
        float *cur = out + (size_t)t * ns;
        for (int s = 0; s < ns; ++s) {
            const int u0 = (s * OR_BASES) % ns;
            const int col = u0 * OR_BASES + (s * OR_BASES) / ns;
            float v[5];
            v[0] = nxt[s] + stay;
            for (int b = 0; b < OR_BASES; ++b) v[b + 1] = nxt[u0 + b] + sc[col + b * OR_BASES];
            cur[s] = lse5(v);
        }
    }
}
void oracle_backward_scan(const float *scores, float *bwd, int chunk, int T, int N, int ns) {
    oracle_backward_scan_stay(scores, bwd, chunk, T, N, ns, 2.0f);
}

/* Forward scan of one chunk fused with the fwd+bwd sum.  src/decode_cpu.c:54-119.  It runs
 * T+1 steps; step t writes out[t][s] = fwd[t][s] + bwd[t][s] (float add, :115-116) and builds
 * fwd[t+1]; scores at step T count as zero (:99).  Predecessors of s are (s div 4) + b*ns/4
 * with score column 4s + b (:91-92,101). */
void oracle_forward_scan_stay(const float *scores, const float *bwd, float *fwdbwd, int chunk, int T,
                              int N, int ns, float stay) {
    const int msb = ns / OR_BASES;
    const size_t row = (size_t)ns * OR_BASES;
    const float *cs = scores + (size_t)chunk * row;
    float ping[2][OR_MAX_STATES];
    for (int s = 0; s < ns; ++s) ping[0][s] = 0.0f;
    for (int t = 0; t <= T; ++t) {
        const float *sc = cs + (size_t)N * row * t;
        const float *in = ping[t & 1];
        float *nx = ping[(t & 1) ^ 1];
        const size_t base = ((size_t)chunk * (T + 1) + t) * ns;
        for (int s = 0; s < ns; ++s) {
            float v[5];
            v[0] = in[s] + stay;
            for (int b = 0; b < OR_BASES; ++b) {
                const float x = t < T ? sc[s * OR_BASES + b] : 0.0f;
                v[b + 1] = in[s / OR_BASES + b * msb] + x;
            }
            nx[s] = lse5(v);
            fwdbwd[base + s] = in[s] + bwd[base + s];
        }
    }
}
void oracle_forward_scan(const float *scores, const float *bwd, float *fwdbwd, int chunk, int T,
                         int N, int ns) {
    oracle_forward_scan_stay(scores, bwd, fwdbwd, chunk, T, N, ns, 2.0f);
}

/* Posterior = softmax over states of fwd+bwd, row by row.  src/decode_cpu.c:121-147: float
 * max, exp in double rounded to float, float running sum in state order, float division. */
void oracle_softmax(const float *fwdbwd, float *post, int chunk, int T, int ns) {
    float e[OR_MAX_STATES];
    for (int t = 0; t <= T; ++t) {
        const size_t base = ((size_t)chunk * (T + 1) + t) * ns;
        float top = fwdbwd[base];
        for (int s = 0; s < ns; ++s) top = top > fwdbwd[base + s] ? top : fwdbwd[base + s];
        float acc = 0;
        for (int s = 0; s < ns; ++s) {
            const float x = exp(fwdbwd[base + s] - top);
            e[s] = x;
            acc += x;
        }
        for (int s = 0; s < ns; ++s) post[base + s] = (float)(e[s] / acc);
    }
}

/* ---------------------------------------------------------------------------------------- */
/* beam search                                                                               */

/* CRC32C (reversed polynomial 0x82f63b78) fed `nbits` bits, LSB first.
 * src/beam_search.c:103-115. */
uint32_t oracle_crc32c(uint32_t crc, uint32_t bits, int nbits) {
    for (int i = 0; i < nbits; ++i) {
        const uint32_t lsb = (bits ^ crc) & 1u;
        crc >>= 1;
        if (lsb) crc ^= 0x82f63b78u;
        bits >>= 1;
    }
    return crc;
}

/* src/beam_search.c:43-47: float |x-y|, double log(1+exp(-d)) when d < 17, sum rounded once. */
static float fold_scores(float x, float y) {
    const float d = fabs(x - y);
    const float m = x > y ? x : y;
    return m + ((d < 17.0f) ? log(1.0 + exp(-d)) : 0.0f);
}

/* exported for the arithmetic checks of the CUDA path's two-term fold */
float oracle_fold_scores(float x, float y) { return fold_scores(x, y); }

static int cmp_desc(const void *a, const void *b) {
    const float x = *(const float *)a, y = *(const float *)b;
    return (x < y) - (x > y);
}

/* The value the reference's quick-select returns (src/beam_search.c:13-41,151-163): the
 * 32nd largest of the first backward row, duplicates counted. */
static float kth_largest_32(const float *v, int n) {
    float tmp[OR_MAX_STATES];
    memcpy(tmp, v, sizeof(float) * n);
    qsort(tmp, n, sizeof(float), cmp_desc);
    return tmp[OR_BEAM - 1];
}

static size_t count_at_least(const float *v, size_t n, float cut) {
    size_t c = 0;
    for (size_t i = 0; i < n; ++i) c += v[i] >= cut;
    return c;
}

/* One chunk of beam search + traceback + per-timestep quality.  src/beam_search.c:117-497.
 * bp receives one {state, prev, stay} triple per kept element and timestep, laid out
 * [T+1][32] like the reference's beam_vector.  score_scale multiplies every transition score
 * (:233) and posts_scale every posterior (:452,483); the reference's decoder passes 1.0f for
 * both (src/decode_cpu.c:216).  On return states[t] is the base (k-mer mod 4) of the path at
 * timestep t, as the reference leaves it (:446). */
void oracle_beam_search(const float *scores, size_t t_stride, const float *bwd, const float *post,
                        int state_bits, int T, float beam_cut, float stay_score, int32_t *states,
                        uint8_t *moves, float *qual, int32_t *bp_state, uint8_t *bp_prev,
                        uint8_t *bp_stay, float score_scale, float posts_scale) {
    const int ns = 1 << state_bits;
    const int32_t mask = ns - 1;
    const float log_cut = beam_cut > 0.0f ? logf(beam_cut) : FLT_MAX; /* :135 */

    uint32_t c_hash[OR_CAND], p_hash[OR_CAND];
    int32_t c_state[OR_CAND], p_state[OR_CAND];
    uint8_t c_prev[OR_CAND], p_prev[OR_CAND], c_stay[OR_CAND], p_stay[OR_CAND];
    float c_score[OR_CAND], p_score[OR_CAND];

    /* initial beam: the first <=32 states, in state order, whose bwd[0] reaches the 32nd
     * largest value (:151-175) */
    float thr = -FLT_MAX;
    if (OR_BEAM < ns) thr = kth_largest_32(bwd, ns);
    size_t width = 0;
    for (int s = 0; s < ns && width < OR_BEAM; ++s) {
        if (bwd[s] >= thr) {
            p_hash[width] = oracle_crc32c(OR_CRC_SEED, (uint32_t)s, 32);
            p_state[width] = s;
            p_prev[width] = 0;
            p_stay[width] = 0;
            p_score[width] = 0.0f;
            ++width;
        }
    }
    width = OR_BEAM < ns ? OR_BEAM : ns; /* :178 */
    for (size_t i = 0; i < width; ++i) {
        bp_state[i] = p_state[i];
        bp_prev[i] = p_prev[i];
        bp_stay[i] = p_stay[i];
    }

    for (int t = 0; t < T; ++t) {
        const float *sc = scores + (size_t)t * t_stride;
        const float *back = bwd + ((size_t)(t + 1) << state_bits);
        float best = -FLT_MAX;
        size_t n = 0;

        /* 4 step candidates per element, element-major (:205-256) */
        for (size_t i = 0; i < width; ++i) {
            for (int b = 0; b < OR_BASES; ++b) {
                const int32_t ns_ = ((p_state[i] << 2) & mask) | b;
                const int32_t col = (ns_ << 2) + ((p_state[i] << 2) >> state_bits);
                const float x = sc[col] * score_scale; /* :233 */
                const float v = p_score[i] + x + back[ns_];
                c_hash[n] = oracle_crc32c(p_hash[i], (uint32_t)b, 2);
                c_state[n] = ns_;
                c_prev[n] = (uint8_t)i;
                c_stay[n] = 0;
                c_score[n] = v;
                best = best > v ? best : v;
                ++n;
            }
        }
        /* 1 stay candidate per element; a stay whose hash equals the hash of a step that
         * appends the stay's last base is the same sequence: fold the two scores into the
         * better one and retire the other (:258-318).  The reference gates the comparison with
         * a one-hash Bloom filter that has no false negatives, so comparing always is
         * equivalent. */
        for (size_t i = 0; i < width; ++i) {
            const size_t si = (width << 2) + i;
            const float v = p_score[i] + stay_score + back[p_state[i]];
            c_hash[si] = p_hash[i];
            c_state[si] = p_state[i];
            c_prev[si] = (uint8_t)i;
            c_stay[si] = 1;
            c_score[si] = v;
            best = best > v ? best : v;
            const int last = p_state[i] & 3;
            for (size_t j = 0; j < width; ++j) {
                const size_t sj = (j << 2) | (size_t)last;
                if (c_hash[si] != c_hash[sj]) continue;
                const float f = fold_scores(c_score[si], c_score[sj]);
                if (c_score[si] > c_score[sj]) {
                    c_score[si] = f;
                    c_score[sj] = -FLT_MAX;
                } else {
                    c_score[sj] = f;
                    c_score[si] = -FLT_MAX;
                }
                best = f > best ? f : best;
            }
            ++n;
        }

        /* pruning threshold: best - ln(beam_cut); when more than 32 pass, bisect between it
         * and best for at most 9 further guesses aiming at 25..32 survivors; reaching the
         * guess limit takes the upper bracket (:320-381) */
        float cut = best - log_cut;
        size_t kept = count_at_least(c_score, n, cut);
        if (kept > OR_BEAM) {
            const size_t floor_w = (OR_BEAM * 8) / 10;
            float lo = cut, hi = best;
            int guesses = 1;
            while ((kept > OR_BEAM || kept < floor_w) && guesses < 10) {
                if (kept > OR_BEAM) {
                    lo = cut;
                    cut = (cut + hi) / 2.0f;
                } else {
                    hi = cut;
                    cut = (cut + lo) / 2.0f;
                }
                kept = count_at_least(c_score, n, cut);
                ++guesses;
            }
            if (guesses == 10) {
                cut = hi;
                kept = count_at_least(c_score, n, cut);
            }
            if (kept > OR_BEAM) kept = OR_BEAM;
        }
        /* survivors keep candidate order; at most 32 (:383-394) */
        size_t w = 0;
        for (size_t r = 0; r < n && w < OR_BEAM; ++r) {
            if (c_score[r] >= cut) {
                p_hash[w] = c_hash[r];
                p_state[w] = c_state[r];
                p_prev[w] = c_prev[r];
                p_stay[w] = c_stay[r];
                p_score[w] = c_score[r];
                ++w;
            }
        }
        /* last timestep: best survivor swaps into slot 0 (:398-414) */
        if (t == T - 1) {
            float top = -FLT_MAX;
            size_t at = 0;
            for (size_t i = 0; i < kept; ++i)
                if (p_score[i] > top) {
                    top = p_score[i];
                    at = i;
                }
            uint32_t h = p_hash[0]; p_hash[0] = p_hash[at]; p_hash[at] = h;
            int32_t s = p_state[0]; p_state[0] = p_state[at]; p_state[at] = s;
            uint8_t q = p_prev[0]; p_prev[0] = p_prev[at]; p_prev[at] = q;
            q = p_stay[0]; p_stay[0] = p_stay[at]; p_stay[at] = q;
            float f = p_score[0]; p_score[0] = p_score[at]; p_score[at] = f;
        }
        /* strip the backward contribution, record back-pointers (:416-427) */
        const size_t off = (size_t)(t + 1) * OR_BEAM;
        for (size_t i = 0; i < kept; ++i) {
            p_score[i] -= back[p_state[i]];
            bp_state[off + i] = p_state[i];
            bp_prev[off + i] = p_prev[i];
            bp_stay[off + i] = p_stay[i];
        }
        width = kept;
    }

    /* traceback from slot 0 (:430-439) */
    uint8_t at = 0;
    for (int t = T; t != 0; --t) {
        const size_t a = (size_t)t * OR_BEAM + at;
        states[t - 1] = bp_state[a];
        moves[t - 1] = bp_stay[a] ? 0 : 1;
        at = bp_prev[a];
    }
    moves[0] = 1;

    /* per-timestep quality (:441-496): posterior of the path k-mer plus its distinct left-
     * and right-shifted neighbours at row t+1, clamped, raised to 0.4 */
    const int msb = ns >> 2;
    for (int t = 0; t < T; ++t) {
        const int st = states[t];
        const int base = st % OR_BASES;
        states[t] = base;
        const float *p = post + ((size_t)(t + 1) << state_bits);
        float prob = p[st] * posts_scale; /* :452 */
        int nb[8];
        for (int b = 0; b < OR_BASES; ++b) {
            nb[2 * b] = (st >> 2) + msb * b;
            nb[2 * b + 1] = ((st << 2) % ns) + b;
        }
        for (int k = 0; k < 8; ++k) {
            int fresh = nb[k] != st;
            for (int m = 0; fresh && m < k; ++m) fresh = nb[m] != nb[k];
            if (fresh) prob += p[nb[k]] * posts_scale; /* :483 */
        }
        if (prob > 1.0f) prob = 1.0f;
        else if (prob < 0.0f) prob = 0.0f;
        prob = powf(prob, 0.4f);
        const float other = (1.0f - prob) / 3.0f;
        for (int b = 0; b < OR_BASES; ++b) qual[t * OR_BASES + b] = b == base ? prob : other;
    }
}

/* Bases and quality string of one chunk.  src/beam_search.c:49-99 with the zeroing of
 * src/decode_cpu.c:218-223.  A timestep's quality adds to the base it steps to or stays on;
 * q = clamp(-10*log10f(1 - base/total)*scale + shift, 1, 50); character = 33.5f + q truncated. */
void oracle_generate_sequence(const uint8_t *moves, const int32_t *bases, const float *qual,
                              float shift, float scale, int T, float *base_probs,
                              float *total_probs, char *sequence, char *qstring) {
    size_t len = 0;
    for (int t = 0; t < T; ++t) {
        len += moves[t];
        base_probs[t] = 0;
        total_probs[t] = 0;
    }
    size_t pos = 0;
    for (int t = 0; t < T; ++t) {
        const int b = bases[t] & 3;
        const int mv = moves[t];
        const size_t at = pos + (t == 0 ? 0 : mv - 1);
        base_probs[at] += qual[t * OR_BASES + b];
        for (int k = 0; k < OR_BASES; ++k) total_probs[at] += qual[t * OR_BASES + k];
        if (t == 0 || mv) sequence[pos++] = (char)b;
    }
    for (size_t i = 0; i < len; ++i) {
        sequence[i] = "ACGT"[(int)sequence[i]];
        base_probs[i] = 1.0f - (base_probs[i] / total_probs[i]);
        base_probs[i] = -10.0f * log10f(base_probs[i]);
        float q = base_probs[i] * scale + shift;
        if (q > 50.0f) q = 50.0f;
        if (q < 1.0f) q = 1.0f;
        qstring[i] = (char)(33.5f + q);
    }
}

/* ---------------------------------------------------------------------------------------- */
/* whole decode, threaded over contiguous chunk ranges like src/decode_cpu.c:278-332         */

typedef struct {
    const float *scores;
    int T, N, C, state_len, lo, hi;
    float scan_stay, score_scale;
    const oracle_opt_t *opt;
    float *bwd, *fwdbwd, *post, *qual, *base_probs, *total_probs;
    int32_t *states, *bp_state;
    uint8_t *moves, *bp_prev, *bp_stay;
    char *sequence, *qstring;
} job_t;

static void *run_range(void *arg) {
    job_t *j = (job_t *)arg;
    const int bits = 2 * j->state_len;
    const int ns = 1 << bits;
    const int T = j->T;
    for (int c = j->lo; c < j->hi; ++c) {
        oracle_backward_scan_stay(j->scores, j->bwd, c, T, j->N, ns, j->scan_stay);
        oracle_forward_scan_stay(j->scores, j->bwd, j->fwdbwd, c, T, j->N, ns, j->scan_stay);
        oracle_softmax(j->fwdbwd, j->post, c, T, ns);
        const size_t cs = (size_t)c * ns * (T + 1);
        const size_t bo = (size_t)c * OR_BEAM * (T + 1);
        oracle_beam_search(j->scores + (size_t)c * ns * OR_BASES, (size_t)j->N * j->C, j->bwd + cs,
                           j->post + cs, bits, T, j->opt->beam_cut, j->opt->blank_score,
                           j->states + (size_t)c * T, j->moves + (size_t)c * T,
                           j->qual + (size_t)c * T * OR_BASES, j->bp_state + bo, j->bp_prev + bo,
                           j->bp_stay + bo, j->score_scale, 1.0f);
        oracle_generate_sequence(j->moves + (size_t)c * T, j->states + (size_t)c * T,
                                 j->qual + (size_t)c * T * OR_BASES, j->opt->q_shift,
                                 j->opt->q_scale, T, j->base_probs + (size_t)c * T,
                                 j->total_probs + (size_t)c * T, j->sequence + (size_t)c * T,
                                 j->qstring + (size_t)c * T);
    }
    return NULL;
}

/* Decode N chunks.  moves/sequence/qstring must hold N*T bytes (zeroed here, as the reference
 * callocs them, src/decode_cpu.c:252-259).  The tensor outputs (bwd, fwdbwd, post:
 * N*(T+1)*ns floats; qual: N*T*4; base_probs,total_probs: N*T) may each be NULL, in which case
 * scratch is allocated and dropped.  Returns 0, or -1 on allocation failure. */
/* flags for oracle_decode_ex */
#define OR_FLAG_SCAN_STAY_FROM_OPTIONS 1 /* scans use opt->blank_score, as src/decode_cuda.cu:115 does */
#define OR_FLAG_TEMPERATURE_SCALES_SCORES 2 /* beam search's score_scale (:233) = opt->temperature */

/* states_out (may be NULL): N*T int32, the base of the decoded path at every timestep, i.e. the
 * contents of the reference's `states` buffer after beam_search_cpu (src/beam_search.c:446). */
int oracle_decode_ex(int T, int N, int C, int nthreads, const float *scores, int state_len,
                     const oracle_opt_t *opt, uint8_t *moves, char *sequence, char *qstring,
                     float *bwd, float *fwdbwd, float *post, float *qual, float *base_probs,
                     float *total_probs, int32_t *states_out, int flags) {
    const int ns = 1 << (2 * state_len);
    const size_t tens = (size_t)N * (T + 1) * ns;
    float *own[6] = {0};
    float **slot[6] = {&bwd, &fwdbwd, &post, &qual, &base_probs, &total_probs};
    const size_t need[6] = {tens, tens, tens, (size_t)N * T * 4, (size_t)N * T, (size_t)N * T};
    int rc = 0;
    for (int i = 0; i < 6; ++i)
        if (!*slot[i]) {
            own[i] = (float *)calloc(need[i], sizeof(float));
            if (!own[i]) rc = -1;
            *slot[i] = own[i];
        }
    int32_t *states = (int32_t *)malloc(sizeof(int32_t) * N * T);
    int32_t *bp_state = (int32_t *)malloc(sizeof(int32_t) * N * OR_BEAM * (T + 1));
    uint8_t *bp_prev = (uint8_t *)malloc((size_t)N * OR_BEAM * (T + 1));
    uint8_t *bp_stay = (uint8_t *)malloc((size_t)N * OR_BEAM * (T + 1));
    if (!states || !bp_state || !bp_prev || !bp_stay) rc = -1;
    if (rc == 0) {
        memset(moves, 0, (size_t)N * T);
        memset(sequence, 0, (size_t)N * T);
        memset(qstring, 0, (size_t)N * T);
        if (nthreads > N) nthreads = N;
        if (nthreads < 1) nthreads = 1;
        pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * nthreads);
        job_t *jobs = (job_t *)malloc(sizeof(job_t) * nthreads);
        const int each = N / nthreads, extra = N % nthreads;
        int lo = 0;
        for (int k = 0; k < nthreads; ++k) {
            job_t j = {scores, T, N, C, state_len, lo, lo + each + (k < extra),
                       (flags & OR_FLAG_SCAN_STAY_FROM_OPTIONS) ? opt->blank_score : 2.0f,
                       (flags & OR_FLAG_TEMPERATURE_SCALES_SCORES) ? opt->temperature : 1.0f, opt,
                       bwd, fwdbwd, post, qual, base_probs, total_probs,
                       states, bp_state, moves, bp_prev, bp_stay, sequence, qstring};
            lo = j.hi;
            jobs[k] = j;
            pthread_create(&tid[k], NULL, run_range, &jobs[k]);
        }
        for (int k = 0; k < nthreads; ++k) pthread_join(tid[k], NULL);
        free(tid);
        free(jobs);
    }
    if (rc == 0 && states_out) memcpy(states_out, states, sizeof(int32_t) * N * T);
    free(states);
    free(bp_state);
    free(bp_prev);
    free(bp_stay);
    for (int i = 0; i < 6; ++i) free(own[i]);
    return rc;
}

/* The reference decoder's behaviour: stay score 2.0f in the scans, temperature ignored. */
int oracle_decode(int T, int N, int C, int nthreads, const float *scores, int state_len,
                  const oracle_opt_t *opt, uint8_t *moves, char *sequence, char *qstring,
                  float *bwd, float *fwdbwd, float *post, float *qual, float *base_probs,
                  float *total_probs) {
    return oracle_decode_ex(T, N, C, nthreads, scores, state_len, opt, moves, sequence, qstring, bwd,
                            fwdbwd, post, qual, base_probs, total_probs, NULL, 0);
}

/* ---------------------------------------------------------------------------------------- */
/* rotary embedding, src/nn_cpu.c:10-39: in-place rotation of the pairs (i, i+rotary_half) of
 * every head vector by the angle whose cos/sin sit at [seq][i]; fp32 throughout.             */
void oracle_rotary_emb(float *x, const float *sin_buf, const float *cos_buf, int batch, int seqlen,
                       int nheads, int rotary_half, long stride_batch, long stride_seq,
                       long stride_head) {
    for (int b = 0; b < batch; ++b)
        for (int h = 0; h < nheads; ++h)
            for (int t = 0; t < seqlen; ++t) {
                float *v = x + b * stride_batch + t * stride_seq + h * stride_head;
                for (int i = 0; i < rotary_half; ++i) {
                    const float c = cos_buf[(size_t)t * rotary_half + i];
                    const float s = sin_buf[(size_t)t * rotary_half + i];
                    const float x0 = v[i], x1 = v[i + rotary_half];
                    v[i] = x0 * c - x1 * s;
                    v[i + rotary_half] = x0 * s + x1 * c;
                }
            }
}
