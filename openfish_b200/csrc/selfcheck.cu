// selfcheck.cu -- measures, on the GPU at hand, the two hardware approximations whose error bounds
// the certified fp32 log-sum-exp (fast_lse.cuh) builds on: ex2.approx.ftz.f32 over every float in
// [-126, 0] (relative error) and lg2.approx.ftz.f32 over every float in [1, 8) (absolute error),
// each against the correctly rounded double-precision function.  About a second of work.
#include <cuda_runtime.h>
#include <math.h>

#include "backend.h"
#include "fast_lse.cuh"
#include "of_device.cuh"
#include "openfish_b200.h"
#include "scan.cuh"

namespace {

__device__ void atomic_max_double(double *at, double v) {
    unsigned long long *p = reinterpret_cast<unsigned long long *>(at);
    unsigned long long seen = *p;
    while (__longlong_as_double((long long)seen) < v) {
        const unsigned long long prev = atomicCAS(p, seen, (unsigned long long)__double_as_longlong(v));
        if (prev == seen) break;
        seen = prev;
    }
}

// bit patterns first .. last (inclusive) are consecutive floats of one sign
__global__ void ex2_error_kernel(double *out, unsigned first, unsigned last) {
    double worst = 0.0;
    for (unsigned long long b = first + blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; b <= last;
         b += (unsigned long long)gridDim.x * blockDim.x) {
        const float x = __uint_as_float((unsigned)b);
        const double exact = exp2((double)x);
        if (exact < 1.1754943508222875e-38) continue;  // results the instruction flushes to zero
        worst = fmax(worst, fabs((double)ofd::ex2_approx(x) - exact) / exact);
    }
    atomic_max_double(out, worst);
}

__global__ void lg2_error_kernel(double *out, unsigned first, unsigned last) {
    double worst = 0.0;
    for (unsigned long long b = first + blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; b <= last;
         b += (unsigned long long)gridDim.x * blockDim.x) {
        const float s = __uint_as_float((unsigned)b);
        worst = fmax(worst, fabs((double)ofd::lg2_approx(s) - log2((double)s)));
    }
    atomic_max_double(out, worst);
}

// A bounded wait on a barrier for which nothing was ever issued: it has to run out.
__global__ void wait_that_runs_out_kernel(int *status, uint64_t wait_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ofd::mbar_init(&bar, 1);
        ofd::mbar_fence_init();
        ofd::mbar_wait_bounded(&bar, 0u, &abort_flag, status, wait_ns);
    }
}

}  // namespace

cudaError_t of_launch_wait_that_runs_out(int *status, uint64_t wait_ns, cudaStream_t stream) {
    wait_that_runs_out_kernel<<<1, 32, 0, stream>>>(status, wait_ns);
    return cudaGetLastError();
}

extern "C" int ofb_selfcheck_arith(double err[2]) {
    double *d = nullptr;
    if (cudaMalloc(&d, 2 * sizeof(double)) != cudaSuccess) return OPENFISH_B200_ERR_ALLOC;
    cudaError_t e = cudaMemset(d, 0, 2 * sizeof(double));
    if (e == cudaSuccess) {
        ex2_error_kernel<<<148 * 8, 256>>>(d, 0x80000000u, 0xC2FC0000u);      // -0 .. -126
        lg2_error_kernel<<<148 * 8, 256>>>(d + 1, 0x3f800000u, 0x40ffffffu);  // 1 .. just below 8
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpy(err, d, 2 * sizeof(double), cudaMemcpyDeviceToHost);
    cudaFree(d);
    return e == cudaSuccess ? OPENFISH_B200_OK : OPENFISH_B200_ERR_CUDA;
}
