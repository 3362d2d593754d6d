/*
 * openfish_b200.h -- entry points this library adds next to the openfish C API.
 *
 * Nothing here exists in the reference; a program written against the reference never needs
 * this header.  It offers (a) error reporting that does not terminate the process, (b) decode
 * calls that write into caller-owned host buffers instead of malloc'ing new ones on every
 * call, split into submit and wait so that the caller can overlap the decode of one batch with
 * other work (the reference's synchronous malloc + pageable copy, src/decode_cuda.cu:118-123
 * and :206-211, costs as much as the kernels themselves at B200 speeds), and (c) the device
 * times of the last decode for benchmarking.
 */
#ifndef OPENFISH_B200_H
#define OPENFISH_B200_H

#include "openfish/openfish.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Status of the calling thread's most recent library call. */
enum openfish_b200_status {
    OPENFISH_B200_OK = 0,
    OPENFISH_B200_ERR_ARGUMENT = 1,    /* NULL pointer, unsupported state_len, T or N < 1, ... */
    OPENFISH_B200_ERR_LAYOUT = 2,      /* C < 4*4^state_len, C % 8 != 0, misaligned pointer */
    OPENFISH_B200_ERR_SHAPE = 3,       /* T, N or state_len differ from the gpubuf's */
    OPENFISH_B200_ERR_OPTION = 4,      /* beam_width != 32 */
    OPENFISH_B200_ERR_ALLOC = 5,       /* host or device allocation failed */
    OPENFISH_B200_ERR_CUDA = 6,        /* a CUDA call failed; see openfish_b200_error_text */
    OPENFISH_B200_ERR_DEVICE_WAIT = 7, /* a kernel gave up waiting for an asynchronous copy */
    OPENFISH_B200_ERR_NO_CPU_PATH = 8, /* openfish_decode_cpu / openfish_rotary_emb_cpu called */
    OPENFISH_B200_ERR_TOO_LONG = 9,    /* T beyond what one block's shared memory can trace back */
    OPENFISH_B200_ERR_SCRATCH_LIMIT = 10, /* shape needs more than the static scratch array holds */
    OPENFISH_B200_ERR_ARITH = 11       /* this GPU's ex2/lg2 approximations exceed the assumed error bounds */
};

/* 0 (default): behave like the reference -- print the error and exit(EXIT_FAILURE).
 * 1: print the error (subject to the log level), record it, and return to the caller; output
 *    pointers are set to NULL and openfish_gpubuf_init returns NULL.  Process-wide. */
void openfish_b200_set_error_mode(int keep_running);
int openfish_b200_get_error_mode(void);

/* Status of the calling thread's last call into the library, and a description of it. */
int openfish_b200_last_status(void);
const char *openfish_b200_error_text(void);

/* Same work as openfish_decode_gpu, but the results land in buffers the caller owns: three host
 * buffers of N*T bytes each (page-locked memory avoids a staging copy; pageable memory works
 * too).  Nothing is malloc'ed. */
void openfish_b200_decode_into(int T, int N, int C, const void *scores_TNC, int state_len,
                               const openfish_opt_t *options, const openfish_gpubuf_t *gpubuf,
                               uint8_t *moves, char *sequence, char *qstring);

/* The same split in two: submit enqueues the kernels and the device-to-host copies on the
 * gpubuf's stream and returns at once; wait blocks until they are done and reports the status.
 * One decode may be in flight per gpubuf.  The three host buffers must be page-locked for the
 * copies to be asynchronous. */
void openfish_b200_decode_submit(int T, int N, int C, const void *scores_TNC, int state_len,
                                 const openfish_opt_t *options, const openfish_gpubuf_t *gpubuf,
                                 uint8_t *moves, char *sequence, char *qstring);
void openfish_b200_decode_wait(const openfish_gpubuf_t *gpubuf);

/* Submit for callers that produce the scores on a CUDA stream of their own.  The calls above run
 * on a stream that is ordered after the legacy default stream only (where the reference does all
 * its work): scores written by a kernel on any other stream -- a non-blocking one in particular,
 * as every side stream of a deep-learning framework is -- are not waited for unless the caller
 * synchronises first.  This variant takes that stream (a cudaStream_t, passed as void * so that
 * this header needs no CUDA header) and makes the decode wait, on the device, for everything
 * queued on it so far; the host does not wait.  No counterpart in the reference, which
 * synchronises the whole device around every kernel (reference src/decode_cuda.cu:152-211). */
void openfish_b200_decode_submit_on(void *cuda_stream, int T, int N, int C, const void *scores_TNC,
                                    int state_len, const openfish_opt_t *options,
                                    const openfish_gpubuf_t *gpubuf, uint8_t *moves, char *sequence,
                                    char *qstring);

/* The other direction: makes cuda_stream wait, on the device, for the gpubuf's decode in flight
 * (a no-op when there is none).  Work queued on that stream afterwards -- overwriting the scores
 * with the next batch, reading the gpubuf's tensors -- then runs after the decode.  The results
 * in the host buffers still need openfish_b200_decode_wait. */
void openfish_b200_stream_wait_decode(void *cuda_stream, const openfish_gpubuf_t *gpubuf);

/* Submit for scores that carry the blank column: [T][N][5*4^state_len] fp16, five consecutive
 * entries per state, its stay ("blank") score first and then its four transition scores in the
 * order of the 4-wide layout (the layout of bonito-style CRF heads).  The reference has no such
 * entry point -- its driver only ever builds 4*4^state_len columns (reference src/main.c:221) and
 * its decoders take the stay score from options->blank_score -- so what this call does is this
 * library's own definition: every state's first entry is dropped, the other four are clamped to
 * [-clamp, +clamp] when clamp > 0 (such heads bound their scores, usually at 5; 0 = no clamp),
 * the result goes into a 4-wide copy that the gpubuf allocates on the first such call
 * (T*N*4*4^state_len*2 bytes, released with the gpubuf), and that copy is decoded exactly as by
 * openfish_b200_decode_submit, stay score = options->blank_score.  The extra pass is bound by HBM
 * (it reads 1.25 and writes 1 times the size of the 4-wide tensor).  cuda_stream: the stream the
 * scores were produced on, as in openfish_b200_decode_submit_on, or NULL for the legacy default
 * stream.  scores_TN5 must be 16-byte aligned.  Finish with openfish_b200_decode_wait. */
void openfish_b200_decode_submit_5wide(void *cuda_stream, int T, int N, const void *scores_TN5, int state_len,
                                       const openfish_opt_t *options, float clamp,
                                       const openfish_gpubuf_t *gpubuf, uint8_t *moves, char *sequence,
                                       char *qstring);

/* Device time, in milliseconds, of the gpubuf's last completed decode, measured with CUDA
 * events on the streams the kernels ran on: ms[0] backward scan kernel, ms[1] everything between
 * it and the copies (the beam search kernel with the forward scan kernel beside it on a second
 * stream, then the posterior + traceback + sequence kernel), ms[2] device-to-host copies, ms[3]
 * all of it. */
void openfish_b200_last_decode_ms(const openfish_gpubuf_t *gpubuf, float ms[4]);

/* The same four numbers followed by: ms[4] beam search kernel, ms[5] forward scan kernel, ms[6]
 * posterior + traceback + sequence kernel, ms[7] the blank-column strip in front of a decode
 * submitted through openfish_b200_decode_submit_5wide (0 otherwise; not part of ms[3]). */
void openfish_b200_last_decode_detail_ms(const openfish_gpubuf_t *gpubuf, float ms[8]);

/* Device time, in milliseconds, of the calling thread's last openfish_rotary_emb_gpu call (CUDA
 * events on the legacy default stream around the kernel). */
float openfish_b200_last_rotary_ms(void);

/* Self-check of the arithmetic the scans rely on.  Backward scores are made bit-identical to the
 * reference CPU decoder's by an fp32 evaluation that certifies its own result, with an exact FP64
 * routine behind it; the certificate rests on error bounds of two hardware approximations.  This
 * call measures them on the current GPU over their whole domains (about a second): err[0] = largest
 * relative error of ex2.approx.ftz.f32 on [-126, 0], err[1] = largest absolute error of
 * lg2.approx.ftz.f32 on [1, 8).  Returns OK when both are within the bounds below, ERR_ARITH when
 * not (results could then differ from the reference's in the last bit), ERR_CUDA/ERR_ALLOC on
 * failure.  Does not touch openfish_b200_last_status().  No counterpart in the reference. */
#define OPENFISH_B200_EX2_REL_BOUND 2.384185791015625e-07 /* 2^-22 */
#define OPENFISH_B200_LG2_ABS_BOUND 2.828e-07             /* 2^-21.75 */
int openfish_b200_selfcheck_arith(double err[2]);

/* Self-check of the path by which a kernel reports that a wait ran out.  Every wait of a kernel
 * for an asynchronous copy is bounded (two seconds); when one runs out the kernel raises a status
 * word, ends normally, and the decode's completion reports OPENFISH_B200_ERR_DEVICE_WAIT.  This
 * call runs, on the gpubuf's stream and status word, a one-block kernel whose only act is such a
 * wait, limit_us microseconds long, on a barrier that nothing will ever complete (no copy is
 * issued), and then reads the status exactly as openfish_b200_decode_wait does.  It returns
 * OPENFISH_B200_ERR_DEVICE_WAIT when the machinery works (and has cleared the status word again,
 * so the gpubuf decodes normally afterwards), OPENFISH_B200_OK if the wait did not run out.
 * Nothing faults, traps or hangs.  Does not touch openfish_b200_last_status().  No counterpart in
 * the reference, whose kernels do not wait. */
int openfish_b200_selfcheck_wait(const openfish_gpubuf_t *gpubuf, unsigned limit_us);

/* Number of kernels one decode call launches (for benchmark bookkeeping). */
int openfish_b200_kernels_per_decode(void);

/* Decode without allocating anything, for callers that cannot let a library allocate once they
 * are running: a serving process that has handed all free device memory to its own arena (a
 * later cudaMalloc from here would fail or fragment it), or a steady-state pipeline that must
 * not run into the device-wide synchronisation cudaMalloc / cudaFree imply.  This entry point has
 * no counterpart in the reference.
 *
 * Same decode, same options and same requirements on scores_TNC as openfish_decode_gpu, but no
 * gpubuf: every intermediate lives in one fixed device array of
 * OPENFISH_B200_STATIC_SCRATCH_BYTES that the library carries (each GPU on which the library's
 * code gets loaded holds it until the process exits).  moves_gpu, sequence_gpu and qstring_gpu
 * are DEVICE buffers of N*T bytes each, owned by the caller.  The work runs on the legacy default
 * stream; the call returns when it is done.  It calls no cudaMalloc, cudaFree, cudaMallocHost,
 * malloc or other allocating routine.
 *
 *   - Shapes whose intermediates do not fit are refused with OPENFISH_B200_ERR_SCRATCH_LIMIT:
 *     needed = k*N*(T+1)*4^state_len*4 + N*(T+1)*32 + N*T*28 bytes (+ 5 KB) with k = 2 tensors
 *     for state_len 4 and 5 (backward scores and posteriors) and 3 for state_len 3 (forward
 *     scores as well), e.g. at T=1666 fast up to N=36, hac up to N=14, sup up to N=3.
 *   - All calls on one GPU share the array.  It keeps what the previous call left (the call
 *     clears what has to start from zero itself); two calls that overlap on the same GPU race,
 *     so serialise them.
 *   - The first call on each device resolves the array's device address and uploads 4 KB of
 *     tables: make that call before any stream capture begins.
 *
 * Returns an openfish_b200_status value (0 = OK); errors are also printed subject to the log
 * level.  It never terminates the process and does not touch openfish_b200_last_status(). */
#define OPENFISH_B200_STATIC_SCRATCH_BYTES (48u << 20)
int openfish_b200_decode_static(int T, int N, int C, const void *scores_TNC, int state_len,
                                const openfish_opt_t *options, uint8_t *moves_gpu,
                                char *sequence_gpu, char *qstring_gpu);

/* The four helpers the reference's test driver (src/main.c:207-252,337-351) calls next to the
 * public API; the reference declares them in an internal header (src/decode_cuda.h:35-55).
 * Same names, arguments and behaviour, so that a driver written against the reference links
 * against this library: select the calling thread's device; copy T*N*C fp16 scores from the
 * host into a new device buffer / release it; write the gpubuf's bwd_NTC, post_NTC, qual_data,
 * base_probs and total_probs as raw little-endian blobs of those names into the current
 * directory (src/decode_cuda.cu:242-343).  Errors follow the library's error mode. */
void set_device_cuda(int device);
void *upload_scores_to_cuda(const int T, const int N, const int C, const void *scores_TNC);
void free_scores_cuda(void *scores_TNC_gpu);
void write_gpubuf_cuda(const uint64_t T, const uint64_t N, const int state_len,
                       const openfish_gpubuf_t *gpubuf);

#ifdef __cplusplus
}
#endif

#endif /* OPENFISH_B200_H */
