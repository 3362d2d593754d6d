/* openfish_api.c -- the C host layer: the openfish entry points, argument checking, the
 * reference's error convention and its log level.
 *
 * Counterpart of the reference's src/openfish.c (dispatch), src/error.c (log level) and the
 * host half of src/decode_cuda.cu (result buffers).  All CUDA work happens behind the C ABI in
 * backend.h. */
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "backend.h"
#include "openfish_b200.h"

static enum openfish_log_level_opt g_log_level = OPENFISH_LOG_VERB; /* reference src/error.c:33 */
static int g_keep_running = 0;
static __thread int t_status = OPENFISH_B200_OK;
static __thread char t_text[600] = "";

enum openfish_log_level_opt get_openfish_log_level(void) { return g_log_level; }
void set_openfish_log_level(enum openfish_log_level_opt level) { g_log_level = level; }

void openfish_b200_set_error_mode(int keep_running) { g_keep_running = keep_running != 0; }
int openfish_b200_get_error_mode(void) { return g_keep_running; }
int openfish_b200_last_status(void) { return t_status; }
const char *openfish_b200_error_text(void) { return t_text; }

static void trace(const char *func, const char *fmt, ...) {
    if (g_log_level < OPENFISH_LOG_TRAC) return;
    va_list ap;
    va_start(ap, fmt);
    fprintf(stderr, "[OPENFISH_DEBUG] %s: ", func);
    vfprintf(stderr, fmt, ap);
    fputc('\n', stderr);
    va_end(ap);
}

/* Record a failure; terminate like the reference unless the caller asked to keep running. */
static void raise_error(const char *func, int code, const char *text) {
    t_status = code;
    snprintf(t_text, sizeof(t_text), "%s: %s", func, text);
    if (g_log_level >= OPENFISH_LOG_ERR)
        fprintf(stderr, "[%s::OPENFISH_ERROR]\033[1;31m %s\033[0m\n", func, text);
    if (!g_keep_running) exit(EXIT_FAILURE);
}
static void clear_error(void) {
    t_status = OPENFISH_B200_OK;
    t_text[0] = '\0';
}
static int backend_failed(const char *func, int rc) {
    if (rc == OPENFISH_B200_OK) return 0;
    raise_error(func, rc, ofb_error_text());
    return 1;
}

static int states_of(int state_len) { return 1 << (2 * state_len); }

/* Argument checks shared by every decode flavour. */
static int check_decode_args(const char *func, int T, int N, int C, const void *scores,
                             int state_len, const openfish_opt_t *options,
                             const openfish_gpubuf_t *gpubuf) {
    char msg[256];
    if (!scores || !options) {
        raise_error(func, OPENFISH_B200_ERR_ARGUMENT, "scores_TNC and options must not be NULL");
        return 1;
    }
    if (state_len < 3 || state_len > 5) {
        snprintf(msg, sizeof(msg), "state_len %d not supported (3, 4 or 5)", state_len);
        raise_error(func, OPENFISH_B200_ERR_ARGUMENT, msg);
        return 1;
    }
    if (T < 1 || N < 1) {
        snprintf(msg, sizeof(msg), "T=%d and N=%d must be at least 1", T, N);
        raise_error(func, OPENFISH_B200_ERR_ARGUMENT, msg);
        return 1;
    }
    if (T > 16384) {
        snprintf(msg, sizeof(msg), "T=%d exceeds the 16384 timesteps one block can trace back", T);
        raise_error(func, OPENFISH_B200_ERR_TOO_LONG, msg);
        return 1;
    }
    if (C < 4 * states_of(state_len) || C % 8 != 0) {
        snprintf(msg, sizeof(msg), "C=%d must be a multiple of 8 and at least 4*4^state_len=%d", C,
                 4 * states_of(state_len));
        raise_error(func, OPENFISH_B200_ERR_LAYOUT, msg);
        return 1;
    }
    if (((size_t)scores & 15u) != 0) {
        raise_error(func, OPENFISH_B200_ERR_LAYOUT, "scores_TNC must be 16-byte aligned");
        return 1;
    }
    if (options->beam_width != 32) {
        snprintf(msg, sizeof(msg), "beam_width %zu not supported: the beam is 32 wide", options->beam_width);
        raise_error(func, OPENFISH_B200_ERR_OPTION, msg);
        return 1;
    }
    return backend_failed(func, ofb_gpubuf_check(gpubuf, T, N, state_len));
}

openfish_gpubuf_t *openfish_gpubuf_init(const int T, const int N, const int state_len) {
    clear_error();
    if (state_len < 3 || state_len > 5 || T < 1 || N < 1) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "need T >= 1, N >= 1 and state_len 3, 4 or 5");
        return NULL;
    }
    openfish_gpubuf_t *g = NULL;
    trace(__func__, "allocating device buffers for T=%d N=%d state_len=%d", T, N, state_len);
    if (backend_failed(__func__, ofb_gpubuf_create(T, N, state_len, &g))) return NULL;
    return g;
}

void openfish_gpubuf_free(openfish_gpubuf_t *gpubuf) {
    clear_error();
    backend_failed(__func__, ofb_gpubuf_destroy(gpubuf));
}

static void submit(const char *func, int on_stream, void *cuda_stream, int T, int N, int C,
                   const void *scores_TNC, int state_len, const openfish_opt_t *options,
                   const openfish_gpubuf_t *gpubuf, uint8_t *moves, char *sequence, char *qstring) {
    clear_error();
    if (!moves || !sequence || !qstring) {
        raise_error(func, OPENFISH_B200_ERR_ARGUMENT, "result buffers must not be NULL");
        return;
    }
    if (check_decode_args(func, T, N, C, scores_TNC, state_len, options, gpubuf)) return;
    trace(func, "scores tensor dim: %d, %d, %d", T, N, C);
    const ofb_decode_params_t params = {options->beam_cut, options->blank_score, options->q_shift,
                                        options->q_scale, options->temperature, on_stream, cuda_stream};
    backend_failed(func, ofb_decode_submit(T, N, C, scores_TNC, state_len, &params, gpubuf, moves,
                                           sequence, qstring));
}

void openfish_b200_decode_submit(int T, int N, int C, const void *scores_TNC, int state_len,
                                 const openfish_opt_t *options, const openfish_gpubuf_t *gpubuf,
                                 uint8_t *moves, char *sequence, char *qstring) {
    submit(__func__, 0, NULL, T, N, C, scores_TNC, state_len, options, gpubuf, moves, sequence, qstring);
}

void openfish_b200_decode_submit_on(void *cuda_stream, int T, int N, int C, const void *scores_TNC,
                                    int state_len, const openfish_opt_t *options,
                                    const openfish_gpubuf_t *gpubuf, uint8_t *moves, char *sequence,
                                    char *qstring) {
    submit(__func__, 1, cuda_stream, T, N, C, scores_TNC, state_len, options, gpubuf, moves, sequence, qstring);
}

void openfish_b200_decode_submit_5wide(void *cuda_stream, int T, int N, const void *scores_TN5, int state_len,
                                       const openfish_opt_t *options, float clamp,
                                       const openfish_gpubuf_t *gpubuf, uint8_t *moves, char *sequence,
                                       char *qstring) {
    clear_error();
    if (!moves || !sequence || !qstring) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "result buffers must not be NULL");
        return;
    }
    /* same checks as the 4-wide calls, on the 4-wide shape the scores are stripped to */
    if (state_len < 3 || state_len > 5) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "state_len not supported (3, 4 or 5)");
        return;
    }
    if (check_decode_args(__func__, T, N, 4 * states_of(state_len), scores_TN5, state_len, options, gpubuf)) return;
    if (!(clamp >= 0.0f)) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "clamp must be zero (off) or positive");
        return;
    }
    const ofb_decode_params_t params = {options->beam_cut, options->blank_score, options->q_shift,
                                        options->q_scale, options->temperature, cuda_stream != NULL, cuda_stream};
    backend_failed(__func__, ofb_decode_submit_5wide(T, N, scores_TN5, state_len, clamp, &params, gpubuf, moves,
                                                     sequence, qstring));
}

void openfish_b200_stream_wait_decode(void *cuda_stream, const openfish_gpubuf_t *gpubuf) {
    clear_error();
    if (!gpubuf) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "gpubuf is NULL");
        return;
    }
    if (backend_failed(__func__, ofb_gpubuf_check_owner(gpubuf))) return;
    backend_failed(__func__, ofb_stream_wait_decode(cuda_stream, gpubuf));
}

int openfish_b200_selfcheck_wait(const openfish_gpubuf_t *gpubuf, unsigned limit_us) {
    if (!gpubuf || ofb_gpubuf_check_owner(gpubuf) != OPENFISH_B200_OK) return OPENFISH_B200_ERR_ARGUMENT;
    return ofb_selfcheck_wait(gpubuf, limit_us);
}

void openfish_b200_decode_wait(const openfish_gpubuf_t *gpubuf) {
    clear_error();
    if (!gpubuf) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "gpubuf is NULL");
        return;
    }
    backend_failed(__func__, ofb_decode_wait(gpubuf));
}

void openfish_b200_decode_into(int T, int N, int C, const void *scores_TNC, int state_len,
                               const openfish_opt_t *options, const openfish_gpubuf_t *gpubuf,
                               uint8_t *moves, char *sequence, char *qstring) {
    openfish_b200_decode_submit(T, N, C, scores_TNC, state_len, options, gpubuf, moves, sequence, qstring);
    if (t_status != OPENFISH_B200_OK) return;
    openfish_b200_decode_wait(gpubuf);
}

void openfish_decode_gpu(const int T, const int N, const int C, void *scores_TNC,
                         const int state_len, const openfish_opt_t *options,
                         const openfish_gpubuf_t *gpubuf, uint8_t **moves, char **sequence,
                         char **qstring) {
    clear_error();
    if (!moves || !sequence || !qstring) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "moves, sequence and qstring must not be NULL");
        return;
    }
    *moves = NULL;
    *sequence = NULL;
    *qstring = NULL;
    if (check_decode_args(__func__, T, N, C, scores_TNC, state_len, options, gpubuf)) return;
    /* the caller frees these with free(), reference src/decode_cuda.cu:118-123 */
    const size_t nt = (size_t)N * (size_t)T;
    uint8_t *m = (uint8_t *)malloc(nt);
    char *s = (char *)malloc(nt);
    char *q = (char *)malloc(nt);
    if (!m || !s || !q) {
        free(m); free(s); free(q);
        raise_error(__func__, OPENFISH_B200_ERR_ALLOC, "could not allocate the result buffers");
        return;
    }
    openfish_b200_decode_submit(T, N, C, scores_TNC, state_len, options, gpubuf, m, s, q);
    if (t_status == OPENFISH_B200_OK) {
        /* Fresh allocations of this size are untouched pages: writing to them for the first time
         * costs a page fault per 4 KB (a quarter of a millisecond for a 512-chunk batch).  That
         * is paid here, while the GPU is busy, instead of in the copy after the wait. */
        memset(m, 0, nt);
        memset(s, 0, nt);
        memset(q, 0, nt);
        openfish_b200_decode_wait(gpubuf);
    }
    if (t_status != OPENFISH_B200_OK) {
        free(m); free(s); free(q);
        return;
    }
    *moves = m;
    *sequence = s;
    *qstring = q;
}

void openfish_b200_last_decode_ms(const openfish_gpubuf_t *gpubuf, float ms[4]) {
    clear_error();
    if (!gpubuf || !ms) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "gpubuf and ms must not be NULL");
        return;
    }
    float all[8];
    ofb_last_decode_ms(gpubuf, all);
    memcpy(ms, all, 4 * sizeof(float));
}

void openfish_b200_last_decode_detail_ms(const openfish_gpubuf_t *gpubuf, float ms[8]) {
    clear_error();
    if (!gpubuf || !ms) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "gpubuf and ms must not be NULL");
        return;
    }
    ofb_last_decode_ms(gpubuf, ms);
}

int openfish_b200_kernels_per_decode(void) { return 4; }

void openfish_rotary_emb_gpu(void *x_gpu, void *sin_gpu, void *cos_gpu, int batch_size, int seqlen,
                             int nheads, int head_dim, int rotary_half, int stride_batch,
                             int stride_seq, int stride_head) {
    (void)head_dim; /* unused by the reference as well, src/nn_cuda.cu:18 */
    clear_error();
    if (!x_gpu || !sin_gpu || !cos_gpu) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "x_gpu, sin_gpu and cos_gpu must not be NULL");
        return;
    }
    if (batch_size < 0 || seqlen < 0 || nheads < 0 || rotary_half < 0) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "negative extent");
        return;
    }
    backend_failed(__func__, ofb_rotary(x_gpu, sin_gpu, cos_gpu, batch_size, seqlen, nheads,
                                        rotary_half, stride_batch, stride_seq, stride_head));
}

float openfish_b200_last_rotary_ms(void) { return ofb_last_rotary_ms(); }

int openfish_b200_selfcheck_arith(double err[2]) {
    const int rc = ofb_selfcheck_arith(err);
    if (rc != OPENFISH_B200_OK) return rc;
    return (err[0] <= OPENFISH_B200_EX2_REL_BOUND && err[1] <= OPENFISH_B200_LG2_ABS_BOUND) ? OPENFISH_B200_OK
                                                                                           : OPENFISH_B200_ERR_ARITH;
}

void openfish_decode_cpu(const int T, const int N, const int C, int nthreads, void *scores_TNC,
                         const int state_len, const openfish_opt_t *options, uint8_t **moves,
                         char **sequence, char **qstring) {
    (void)T; (void)N; (void)C; (void)nthreads; (void)scores_TNC; (void)state_len; (void)options;
    clear_error();
    if (moves) *moves = NULL;
    if (sequence) *sequence = NULL;
    if (qstring) *qstring = NULL;
    raise_error(__func__, OPENFISH_B200_ERR_NO_CPU_PATH, "this library has no CPU decode path");
}

void openfish_rotary_emb_cpu(void *x, void *sin_buf, void *cos_buf, int batch_size, int seqlen,
                             int nheads, int head_dim, int rotary_half, int stride_batch,
                             int stride_seq, int stride_head, int nthreads) {
    (void)x; (void)sin_buf; (void)cos_buf; (void)batch_size; (void)seqlen; (void)nheads;
    (void)head_dim; (void)rotary_half; (void)stride_batch; (void)stride_seq; (void)stride_head;
    (void)nthreads;
    clear_error();
    raise_error(__func__, OPENFISH_B200_ERR_NO_CPU_PATH, "this library has no CPU rotary path");
}

/* ---- what the reference's test driver calls besides the public API (src/decode_cuda.h:35-55,
 * src/decode_cuda.cu:214-343): device selection, score upload, and a dump of the gpubuf's
 * tensors into the current directory. */
void set_device_cuda(int device) {
    clear_error();
    backend_failed(__func__, ofb_set_device(device));
}

void *upload_scores_to_cuda(const int T, const int N, const int C, const void *scores_TNC) {
    clear_error();
    if (!scores_TNC || T < 0 || N < 0 || C < 0) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "scores_TNC must not be NULL, extents not negative");
        return NULL;
    }
    void *d = NULL;
    if (backend_failed(__func__, ofb_device_upload(scores_TNC, (size_t)T * N * C * 2u, &d))) return NULL;
    return d;
}

void free_scores_cuda(void *scores_TNC_gpu) {
    clear_error();
    backend_failed(__func__, ofb_device_free(scores_TNC_gpu));
}

/* One device tensor to a file, through a bounce buffer (the tensors reach gigabytes). */
static int dump_tensor(const char *func, const char *path, const void *device, size_t bytes, void *bounce,
                       size_t bounce_bytes) {
    FILE *fp = fopen(path, "w");
    if (!fp) {
        char msg[300];
        snprintf(msg, sizeof(msg), "cannot open %s for writing", path);
        raise_error(func, OPENFISH_B200_ERR_ARGUMENT, msg);
        return 1;
    }
    for (size_t off = 0; off < bytes; off += bounce_bytes) {
        const size_t n = bytes - off < bounce_bytes ? bytes - off : bounce_bytes;
        if (backend_failed(func, ofb_device_download(bounce, (const char *)device + off, n))) {
            fclose(fp);
            return 1;
        }
        if (fwrite(bounce, 1, n, fp) != n) {
            char msg[300];
            snprintf(msg, sizeof(msg), "short write to %s", path);
            fclose(fp);
            raise_error(func, OPENFISH_B200_ERR_ARGUMENT, msg);
            return 1;
        }
    }
    fclose(fp);
    return 0;
}

void write_gpubuf_cuda(const uint64_t T, const uint64_t N, const int state_len, const openfish_gpubuf_t *gpubuf) {
    clear_error();
    if (!gpubuf || state_len < 3 || state_len > 5) {
        raise_error(__func__, OPENFISH_B200_ERR_ARGUMENT, "gpubuf must not be NULL, state_len 3..5");
        return;
    }
    if (backend_failed(__func__, ofb_gpubuf_check(gpubuf, (int)T, (int)N, state_len))) return;
    const size_t ns = (size_t)states_of(state_len), bounce_bytes = (size_t)32 << 20;
    void *bounce = malloc(bounce_bytes);
    if (!bounce) {
        raise_error(__func__, OPENFISH_B200_ERR_ALLOC, "out of host memory");
        return;
    }
    const struct { const char *path; const void *dev; size_t bytes; } out[] = {
        {"bwd_NTC.blob", gpubuf->bwd_NTC, N * (T + 1) * ns * sizeof(float)},
        {"post_NTC.blob", gpubuf->post_NTC, N * (T + 1) * ns * sizeof(float)},
        {"qual_data.blob", gpubuf->qual_data, N * T * 4 * sizeof(float)},
        {"base_probs.blob", gpubuf->base_probs, N * T * sizeof(float)},
        {"total_probs.blob", gpubuf->total_probs, N * T * sizeof(float)},
    };
    for (size_t i = 0; i < sizeof(out) / sizeof(out[0]); ++i)
        if (dump_tensor(__func__, out[i].path, out[i].dev, out[i].bytes, bounce, bounce_bytes)) break;
    free(bounce);
}

