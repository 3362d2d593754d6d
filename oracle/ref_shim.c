/*
 * ref_shim.c -- exposes the reference CPU decoder's file-local scan routines.
 *
 * TEST INFRASTRUCTURE ONLY.  This translation unit contains no reference code: it textually
 * includes the reference's own src/decode_cpu.c from the reference checkout (found through
 * the -I flag oracle/Makefile passes) so that its static backward_scan / forward_scan /
 * softmax (src/decode_cpu.c:13-147) can be called on their own, which is what the tensor-
 * level parity checks of the CPU restatement need.  The product never links it.
 */
#include "decode_cpu.c"

/* bwd, fwdbwd, post: [N][T+1][4^state_len] floats, all three filled for every chunk. */
void ref_scan_tensors(const float *scores, int T, int N, int state_len, float *bwd, float *fwdbwd,
                      float *post) {
    const uint64_t ns = 1ull << (2 * state_len);
    for (int c = 0; c < N; ++c) {
        backward_scan(scores, bwd, c, T, N, ns);
        forward_scan(scores, bwd, fwdbwd, c, T, N, ns);
        softmax(fwdbwd, post, c, T, ns);
    }
}

/* Beam search, traceback and per-timestep quality of one chunk through the reference's
 * beam_search_cpu (src/beam_search.c:117); beam_vector must hold 32*(T+1) 8-byte elements. */
void ref_beam_search(const float *scores, size_t t_stride, const float *bwd, const float *post,
                     int state_bits, int T, float beam_cut, float stay_score, int32_t *states,
                     uint8_t *moves, float *qual, void *beam_vector) {
    beam_search_cpu(scores, t_stride, bwd, post, state_bits, T, beam_cut, stay_score, states, moves,
                    qual, 1.0f, 1.0f, (beam_element_t *)beam_vector);
}

/* The same with the reference's two scale arguments exposed (src/beam_search.c:129-130: score_scale
 * multiplies every transition score, :233; posts_scale every posterior, :452,483), which its own
 * decoder always passes as 1.0f (src/decode_cpu.c:216). */
void ref_beam_search_scaled(const float *scores, size_t t_stride, const float *bwd, const float *post,
                            int state_bits, int T, float beam_cut, float stay_score, int32_t *states,
                            uint8_t *moves, float *qual, float score_scale, float posts_scale,
                            void *beam_vector) {
    beam_search_cpu(scores, t_stride, bwd, post, state_bits, T, beam_cut, stay_score, states, moves,
                    qual, score_scale, posts_scale, (beam_element_t *)beam_vector);
}

/* Sequence and quality string of one chunk through the reference's generate_sequence_cpu
 * (src/beam_search.c:49-99); base_probs and total_probs must arrive zeroed, as the reference's
 * decoder hands them over (src/decode_cpu.c:218-223). */
void ref_generate_sequence(const uint8_t *moves, const int32_t *states, const float *qual, float shift,
                           float scale, size_t T, size_t seq_len, float *base_probs, float *total_probs,
                           char *sequence, char *qstring) {
    generate_sequence_cpu(moves, states, qual, shift, scale, T, seq_len, base_probs, total_probs,
                          sequence, qstring);
}
