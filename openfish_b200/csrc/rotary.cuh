// rotary.cuh -- launcher of the rotary-embedding kernels (see rotary.cu).
#pragma once
#include <cuda_runtime.h>

// x: fp16, rotated in place; sin_t / cos_t: fp32 [seqlen][rotary_half]; strides in elements.
cudaError_t of_launch_rotary(void *x, const void *sin_t, const void *cos_t, int batch, int seqlen,
                             int nheads, int rotary_half, long long stride_batch,
                             long long stride_seq, long long stride_head, int sm_count,
                             cudaStream_t stream);
