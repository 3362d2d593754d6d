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
