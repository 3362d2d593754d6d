/*
 * openfish/openfish.h -- CRF-CTC decode for nanopore basecalling on NVIDIA B200 (sm_100a).
 *
 * This header is a binary-compatible drop-in for the reference's include/openfish/openfish.h:
 * the two structs, DECODER_INIT and every function signature match it declaration for
 * declaration, so code written against the reference recompiles and relinks unchanged.
 * What differs is behind it: the GPU entry points are implemented by hand-written sm_100a
 * kernels whose results follow the reference's CPU decoder, and the CPU entry points are not
 * implemented (this library has no CPU path; they report an error exactly like the reference
 * built without a GPU back end reports for its GPU entry points, reference src/openfish.c:24-26).
 *
 * Error behaviour (same as the reference, src/cuda_utils.cuh:5-13, src/error.h:44-49): the
 * functions return nothing; on a CUDA failure, an allocation failure or an argument the
 * library cannot handle they print to stderr and terminate the process.  A caller that wants
 * to stay alive instead can switch that off with openfish_b200_set_error_mode(), see
 * openfish_b200.h.
 */
#ifndef OPENFISH_H
#define OPENFISH_H

#include <stdbool.h>
#include <stdint.h>
#include <stdlib.h>

#include "openfish_error.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Default decoder options: beam_width 32, beam_cut 100, blank_score 2, q_shift 0, q_scale 1,
 * temperature 1, move_pad false.  (reference include/openfish/openfish.h:14) */
#define DECODER_INIT {32, 100.0, 2.0, 0.0, 1.0, 1.0, false}

/* Device buffers a decode needs, allocated once for a fixed (T, N, state_len) by
 * openfish_gpubuf_init and reused by every decode call of that shape.  All members are device
 * pointers.  (reference include/openfish/openfish.h:16-27; sizes reference
 * src/decode_cuda.cu:22-45)
 *
 * After openfish_decode_gpu returns they hold, for chunk n:
 *   bwd_NTC      float [N][T+1][4^state_len]  backward scores
 *   post_NTC     float [N][T+1][4^state_len]  posterior state probabilities
 *   moves        uint8 [N][T]                 1 where a base is emitted
 *   sequence     char  [N][T]                 bases, zero padded
 *   qstring      char  [N][T]                 Phred+33 qualities, zero padded
 *   beam_vector  opaque: this library keeps one packed byte per beam slot and timestep,
 *                [N][T+1][32] (previous slot | stay << 5 | base << 6), in the first
 *                N*(T+1)*32 bytes of the reference-sized allocation
 *   states       int32 [N][T]                 base (0..3) of the path element at each timestep
 *   qual_data    float [N][T][4]              per-timestep base probabilities
 *   base_probs   float [N][T]                 -10*log10(1 - p_base/p_total) per base
 *   total_probs  float [N][T]                 p_total per base
 */
typedef struct openfish_gpubuf {
    float *bwd_NTC;
    float *post_NTC;
    uint8_t *moves;
    char *sequence;
    char *qstring;
    void *beam_vector;
    void *states;
    float *qual_data;
    float *base_probs;
    float *total_probs;
} openfish_gpubuf_t;

/* Decoder options (reference include/openfish/openfish.h:29-37).  Like the reference, the
 * decoder reads beam_cut, blank_score, q_shift and q_scale (reference
 * src/decode_cuda.cu:133-136); the beam width is fixed at 32 (reference src/decode.h:49) and a
 * beam_width other than 32 is reported as an error instead of being silently ignored; move_pad
 * is not used.
 *
 * Two fields reach further here than in the reference's CPU decoder, the decoder whose results
 * this library otherwise reproduces.  At their DECODER_INIT values nothing differs.
 *   blank_score  is also the stay score of the two scans, as in the reference's CUDA launcher
 *                (reference src/decode_cuda.cu:115); the reference's CPU scans use the literal
 *                2.0 whatever the option says (reference src/decode_cpu.c:14,56).  Results equal
 *                the CPU decoder's at blank_score = 2.0 only.
 *   temperature  multiplies every transition score inside the beam search: it is handed to the
 *                search as the score_scale argument the reference's beam_search_cpu has
 *                (reference src/beam_search.c:129,233) and that the reference's decoders always
 *                pass as 1.0 (reference src/decode_cpu.c:216, src/decode_cuda.cu:165), ignoring
 *                the option.  The scans are not scaled.  Results equal the reference's at
 *                temperature = 1.0 only. */
typedef struct openfish_opt {
    size_t beam_width;
    float beam_cut;
    float blank_score;
    float q_shift;
    float q_scale;
    float temperature;
    bool move_pad;
} openfish_opt_t;

/* Not implemented by this library (no CPU path): logs an error and terminates, or, in the
 * non-terminating error mode, records OPENFISH_B200_ERR_NO_CPU_PATH and returns with the output
 * pointers set to NULL.  (reference declaration include/openfish/openfish.h:39-50) */
void openfish_decode_cpu(const int T, const int N, const int C, int nthreads, void *scores_TNC,
                         const int state_len, const openfish_opt_t *options, uint8_t **moves,
                         char **sequence, char **qstring);

/* Not implemented by this library, as above.  (reference include/openfish/openfish.h:52-65) */
void openfish_rotary_emb_cpu(void *x, void *sin_buf, void *cos_buf, int batch_size, int seqlen,
                             int nheads, int head_dim, int rotary_half, int stride_batch,
                             int stride_seq, int stride_head, int nthreads);

/* Decode N chunks of T timesteps on the calling thread's current CUDA device.
 * (reference include/openfish/openfish.h:67-78, src/decode_cuda.cu:79-212)
 *
 *   scores_TNC  device pointer, fp16, laid out [T][N][C], 16-byte aligned, read only.
 *               C must be at least 4*4^state_len and a multiple of 8.  As in the reference the
 *               scans address the tensor as [T][N][4*4^state_len] whatever C is, while the
 *               beam search strides timesteps by N*C; the two agree when C = 4*4^state_len,
 *               the layout the reference's driver uses (reference src/main.c:221).
 *   state_len   3, 4 or 5 (64, 256 or 1024 states).
 *   gpubuf      from openfish_gpubuf_init with the same T, N and state_len.
 *   moves, sequence, qstring
 *               out: each receives a malloc'ed buffer of N*T bytes that the caller frees;
 *               chunk n starts at offset n*T; sequence and qstring are zero filled beyond the
 *               chunk's sequence length (the sum of its moves).
 * The call returns when the results are in host memory. */
void openfish_decode_gpu(const int T, const int N, const int C, void *scores_TNC,
                         const int state_len, const openfish_opt_t *options,
                         const openfish_gpubuf_t *gpubuf, uint8_t **moves, char **sequence,
                         char **qstring);

/* Allocate the device buffers for decodes of shape (T, N, state_len) on the current device.
 * (reference include/openfish/openfish.h:80-84, src/decode_cuda.cu:11-48) */
openfish_gpubuf_t *openfish_gpubuf_init(const int T, const int N, const int state_len);

/* Release what openfish_gpubuf_init allocated.
 * (reference include/openfish/openfish.h:86-88, src/decode_cuda.cu:50-77) */
void openfish_gpubuf_free(openfish_gpubuf_t *gpubuf);

/* Rotary position embedding, in place, on fp16 device data: for every batch element, position
 * and head, the pairs (i, i + rotary_half) of the head vector are rotated by the angle whose
 * sine and cosine are sin_gpu[position][i] and cos_gpu[position][i] (fp32 device tables of
 * shape [seqlen][rotary_half]).  Strides are in elements.  head_dim is accepted and unused,
 * as in the reference.  Returns when the kernel has finished.
 * (reference include/openfish/openfish.h:90-102, src/nn_cuda.cu:10-40) */
void openfish_rotary_emb_gpu(void *x_gpu, void *sin_gpu, void *cos_gpu, int batch_size, int seqlen,
                             int nheads, int head_dim, int rotary_half, int stride_batch,
                             int stride_seq, int stride_head);

#ifdef __cplusplus
}
#endif

#endif /* OPENFISH_H */
