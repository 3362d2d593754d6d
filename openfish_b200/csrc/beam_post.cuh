// beam_post.cuh -- launchers of the beam search kernel (beam_search.cu) and of the posterior +
// traceback + sequence kernel (posterior_seq.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
namespace ofx { struct Tables; }

struct OfDecodeArgs {
    const __half *scores;      // [T][N][C] fp16, 16-byte aligned, C % 8 == 0, C >= 4*ns
    const float *bwd;          // [N][T+1][ns], from the backward scan
    const float *fwd;          // [N][T+1][ns], from the forward scan (posterior kernel only); null when
                               // the forward scan has already written the posterior into `post`
    float *post;               // [N][T+1][ns] out
    unsigned char *bp;         // [N][T+1][32] packed back-pointers: beam search -> traceback
    int *init_kmers;           // [N][32] k-mers of the initial beam: beam search -> traceback
    uint8_t *moves;            // [N][T] out
    char *sequence;            // [N][T] out
    char *qstring;             // [N][T] out
    int *states;               // [N][T] out (base per timestep)
    float *qual;               // [N][T][4] out
    float *base_probs;         // [N][T] out
    float *total_probs;        // [N][T] out
    const ofx::Tables *tables;
    int *status;
    uint64_t wait_ns;          // how long a kernel waits for an asynchronous copy before raising *status
    int T, N, C, state_len;
    float stay, log_beam_cut, q_shift, q_scale;
    float score_scale;         // multiplies every transition score in the beam search (src/beam_search.c:233)
};

// needs scores, bwd; writes bp, init_kmers
cudaError_t of_launch_beam_search(const OfDecodeArgs &a, cudaStream_t stream);
// needs bwd, fwd, bp, init_kmers; writes post and every output
cudaError_t of_launch_posterior_seq(const OfDecodeArgs &a, cudaStream_t stream);
