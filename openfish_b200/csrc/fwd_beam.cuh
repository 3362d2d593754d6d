// fwd_beam.cuh -- launcher of the fused posterior + beam search + sequence kernel
// (see fwd_beam.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
namespace ofx { struct Tables; }

struct OfFusedLaunch {
    const void *scores_fp16;   // [T][N][C] fp16, 16-byte aligned, C % 8 == 0, C >= 4*ns
    const float *bwd;          // [N][T+1][ns], from the backward scan
    const float *fwd;          // [N][T+1][ns], from the forward scan
    float *post;               // [N][T+1][ns] out
    unsigned char *bp;         // [N][T+1][32] out, packed back-pointers
    uint8_t *moves;            // [N][T] out
    char *sequence;            // [N][T] out
    char *qstring;             // [N][T] out
    int *states;               // [N][T] out (base per timestep)
    float *qual;               // [N][T][4] out
    float *base_probs;         // [N][T] out
    float *total_probs;        // [N][T] out
    const ofx::Tables *tables;
    int *status;
    int T, N, C, state_len;
    float stay, log_beam_cut, q_shift, q_scale;
};

cudaError_t of_launch_fwd_beam(const OfFusedLaunch &l, cudaStream_t stream);
size_t of_fwd_beam_max_T(int state_len);
