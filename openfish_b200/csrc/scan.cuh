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
