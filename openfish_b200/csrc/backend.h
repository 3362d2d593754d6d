/* backend.h -- the thin C ABI between the C host layer (openfish_api.c) and the CUDA side
 * (decode_b200.cu).  Plain C types only.  Every function returns an openfish_b200_status
 * value and, on failure, leaves a description retrievable with ofb_error_text(). */
#ifndef OFB_BACKEND_H
#define OFB_BACKEND_H

#include <stddef.h>
#include <stdint.h>

#include "openfish/openfish.h"

#ifdef __cplusplus
extern "C" {
#endif

int ofb_gpubuf_create(int T, int N, int state_len, openfish_gpubuf_t **out);
int ofb_gpubuf_destroy(openfish_gpubuf_t *gpubuf);
/* Checks that gpubuf came from ofb_gpubuf_create (whatever its shape). */
int ofb_gpubuf_check_owner(const openfish_gpubuf_t *gpubuf);
/* Checks that gpubuf came from ofb_gpubuf_create with this shape. */
int ofb_gpubuf_check(const openfish_gpubuf_t *gpubuf, int T, int N, int state_len);

/* What a decode takes from openfish_opt_t, plus where to run it. */
typedef struct {
    float beam_cut, blank_score, q_shift, q_scale;
    float score_scale;   /* options->temperature: the beam search's score_scale (src/beam_search.c:233) */
    int on_caller_stream;/* 0: order after the legacy default stream (the reference's behaviour) */
    void *caller_stream; /* cudaStream_t the scores were produced on, when on_caller_stream */
} ofb_decode_params_t;

/* Enqueue one decode and the copies of moves/sequence/qstring into the three host buffers. */
int ofb_decode_submit(int T, int N, int C, const void *scores, int state_len,
                      const ofb_decode_params_t *params, const openfish_gpubuf_t *gpubuf,
                      uint8_t *moves, char *sequence, char *qstring);
/* The same for scores laid out [T][N][5*4^state_len], every state's stay score in front of its four
 * transition scores: they are stripped (and clamped to +-clamp when clamp > 0) into a 4-wide copy the
 * gpubuf owns (allocated on the first such call), which is then decoded. */
int ofb_decode_submit_5wide(int T, int N, const void *scores5, int state_len, float clamp,
                            const ofb_decode_params_t *params, const openfish_gpubuf_t *gpubuf,
                            uint8_t *moves, char *sequence, char *qstring);
/* Wait for the gpubuf's decode in flight; returns its status (device-side status included). */
int ofb_decode_wait(const openfish_gpubuf_t *gpubuf);
int ofb_last_decode_ms(const openfish_gpubuf_t *gpubuf, float ms[8]);
/* Makes `stream` (a cudaStream_t) wait, on the device, for the gpubuf's decode in flight. */
int ofb_stream_wait_decode(void *stream, const openfish_gpubuf_t *gpubuf);
/* Runs, on the gpubuf's stream and status word, a one-block kernel whose only act is a bounded wait
 * (limit_us microseconds) on a barrier nothing will ever complete, then reads the status the way a
 * decode's completion does.  Returns OPENFISH_B200_ERR_DEVICE_WAIT when the machinery works. */
int ofb_selfcheck_wait(const openfish_gpubuf_t *gpubuf, unsigned limit_us);

int ofb_rotary(void *x, const void *sin_t, const void *cos_t, int batch, int seqlen, int nheads,
               int rotary_half, long long stride_batch, long long stride_seq,
               long long stride_head);

/* Measured error of the two hardware approximations the certified fp32 arithmetic relies on:
 * err[0] ex2.approx (relative, arguments in [-126, 0]), err[1] lg2.approx (absolute, [1, 8)). */
int ofb_selfcheck_arith(double err[2]);

/* Device time of the calling thread's last ofb_rotary call, in milliseconds. */
float ofb_last_rotary_ms(void);

/* Device selection and plain copies for driver programs (no CUDA headers needed on their side). */
int ofb_set_device(int device);
int ofb_device_upload(const void *host, size_t bytes, void **out);
int ofb_device_free(void *device);
int ofb_device_download(void *host, const void *device, size_t bytes);

const char *ofb_error_text(void);

#ifdef __cplusplus
}
#endif
#endif
