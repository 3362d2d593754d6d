// scan.cuh -- launcher of the backward + forward scan kernel (see scan.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
namespace ofx { struct Tables; }

// scores_fp16: [T][N][>=4*ns] fp16, 16-byte aligned; bwd, fwd: [N][T+1][ns] fp32 out, either may
// be null (that direction is then not scanned); tables: device copy of ofx::Tables; status: device int raised when a
// wait for an asynchronous copy runs out, which it does after wait_ns nanoseconds.
cudaError_t of_launch_scans(const void *scores_fp16, float *bwd, float *fwd, int T, int N,
                            int state_len, float stay, const ofx::Tables *tables, int *status,
                            uint64_t wait_ns, cudaStream_t stream);

// Forward scan and posterior in one kernel, for the models that have it (of_forward_posterior_fused):
// reads the finished backward scores, writes post = softmax_s(fwd + bwd) [N][T+1][ns]; the forward
// scores themselves never leave the chip.
bool of_forward_posterior_fused(int state_len);

// Scores with every state's stay score in front of its four transition scores, [rows][5*ns] fp16,
// to the [rows][4*ns] layout the decode reads (adaptor.cu); clamp > 0 also bounds the values.
cudaError_t of_launch_strip_blank(const void *in, void *out, long long rows, int state_len, float clamp, int sms,
                                  cudaStream_t stream);

// One block, one bounded wait of wait_ns nanoseconds on a barrier that nothing completes (no copy is
// issued at all); the wait runs out, *status becomes ofd::kStatusWaitTimeout and the kernel returns.
// Exists so that the path from a kernel's timeout to the host's error can be exercised without anything
// being wrong.  (selfcheck.cu)
cudaError_t of_launch_wait_that_runs_out(int *status, uint64_t wait_ns, cudaStream_t stream);
cudaError_t of_launch_forward_posterior(const void *scores_fp16, const float *bwd, float *post, int T,
                                        int N, int state_len, float stay, const ofx::Tables *tables,
                                        int *status, uint64_t wait_ns, cudaStream_t stream);
