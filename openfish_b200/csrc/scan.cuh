// scan.cuh -- launcher of the backward + forward scan kernel (see scan.cu).
#pragma once
#include <cuda_runtime.h>
namespace ofx { struct Tables; }

// scores_fp16: [T][N][>=4*ns] fp16, 16-byte aligned; bwd, fwd: [N][T+1][ns] fp32 out, either may
// be null (that direction is then not scanned); tables: device copy of ofx::Tables; status: device int raised on a
// bounded-wait timeout.
cudaError_t of_launch_scans(const void *scores_fp16, float *bwd, float *fwd, int T, int N,
                            int state_len, float stay, const ofx::Tables *tables, int *status,
                            cudaStream_t stream);

// Forward scan and posterior in one kernel, for the models that have it (of_forward_posterior_fused):
// reads the finished backward scores, writes post = softmax_s(fwd + bwd) [N][T+1][ns]; the forward
// scores themselves never leave the chip.
bool of_forward_posterior_fused(int state_len);
cudaError_t of_launch_forward_posterior(const void *scores_fp16, const float *bwd, float *post, int T,
                                        int N, int state_len, float stay, const ofx::Tables *tables,
                                        int *status, cudaStream_t stream);
