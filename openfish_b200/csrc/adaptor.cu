// adaptor.cu -- scores with the blank column inside ("5-wide") to the layout the decode reads.
//
// The reference decodes [T][N][4*ns] scores only (src/main.c:221; the stay score is the scalar
// option blank_score); CRF heads in the bonito style emit [T][N][5*ns], five consecutive entries per
// state: its stay ("blank") score first, then its four transition scores in the 4-wide order.
// There is nothing in the reference to follow here: this kernel drops every state's first entry,
// optionally clamps the other four to [-clamp, +clamp] (such heads bound their outputs, usually at 5),
// and writes the 4-wide tensor the scans and the beam search take.  One pass, bound by HBM:
// it reads 10*ns and writes 8*ns bytes per chunk and timestep.
//
// A row goes through shared memory so that both the global loads and the global stores are whole
// 16-byte pieces of consecutive threads.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

// rows a block of 256 threads takes per pass: some 20 KB of input, i.e. five 16-byte loads in flight
// per thread -- a streaming kernel reaches the memory's bandwidth only with enough bytes under way
template <int NS>
struct RowsPerPass { static constexpr int value = 20480 / (NS * 10); };

template <int NS>
__global__ void __launch_bounds__(256) strip_blank_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out,
                                                          long long rows, float clamp) {
    constexpr int IN16 = NS * 10 / 16;   // 16-byte pieces of a 5-wide row
    constexpr int OUT16 = NS * 8 / 16;   // 16-byte pieces of a 4-wide row
    constexpr int RPB = RowsPerPass<NS>::value;
    __shared__ uint4 stage[RPB][IN16];
    const __half2 lo2 = __float2half2_rn(-clamp), hi2 = __float2half2_rn(clamp);
    for (long long row0 = (long long)blockIdx.x * RPB; row0 < rows; row0 += (long long)gridDim.x * RPB) {
        // the rows of a pass are consecutive in memory: one flat range of 16-byte pieces
        const long long left = (rows - row0) * IN16;
        const int pieces = left < RPB * IN16 ? (int)left : RPB * IN16;
        const uint4 *src = in + row0 * IN16;
        uint4 *flat = &stage[0][0];
#pragma unroll
        for (int k = 0; k < (RPB * IN16 + 255) / 256; ++k) {
            const int i = threadIdx.x + 256 * k;
            if (i < pieces) flat[i] = __ldcs(src + i);  // read once: streaming
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < (RPB * OUT16 + 255) / 256; ++k) {
            const int i = threadIdx.x + 256 * k;
            const int r = i / OUT16, c = i % OUT16;
            if (i >= RPB * OUT16 || row0 + r >= rows) continue;
            // output piece c holds states 2c and 2c+1: input halfs 10c+1..10c+4 and 10c+6..10c+9
            const __half *h = reinterpret_cast<const __half *>(&stage[r][0]) + 10 * c;
            __half2 p[4] = {__halves2half2(h[1], h[2]), __halves2half2(h[3], h[4]),
                            __halves2half2(h[6], h[7]), __halves2half2(h[8], h[9])};
            if (clamp > 0.f) {
#pragma unroll
                for (int k = 0; k < 4; ++k) p[k] = __hmin2(__hmax2(p[k], lo2), hi2);
            }
            uint4 v;
            v.x = *reinterpret_cast<uint32_t *>(&p[0]);
            v.y = *reinterpret_cast<uint32_t *>(&p[1]);
            v.z = *reinterpret_cast<uint32_t *>(&p[2]);
            v.w = *reinterpret_cast<uint32_t *>(&p[3]);
            out[(row0 + r) * OUT16 + c] = v;
        }
        __syncthreads();
    }
}

template <int NS>
cudaError_t launch(const void *in, void *out, long long rows, float clamp, int sms, cudaStream_t stream) {
    const long long want = (rows + RowsPerPass<NS>::value - 1) / RowsPerPass<NS>::value;
    const int grid = (int)(want < (long long)sms * 8 ? want : (long long)sms * 8);
    strip_blank_kernel<NS><<<grid, 256, 0, stream>>>(static_cast<const uint4 *>(in), static_cast<uint4 *>(out), rows, clamp);
    return cudaGetLastError();
}

}  // namespace

// in: [rows][5*ns] fp16, out: [rows][4*ns] fp16, both 16-byte aligned; rows = T*N.
cudaError_t of_launch_strip_blank(const void *in, void *out, long long rows, int state_len, float clamp, int sms,
                                  cudaStream_t stream) {
    switch (state_len) {
        case 3: return launch<64>(in, out, rows, clamp, sms, stream);
        case 4: return launch<256>(in, out, rows, clamp, sms, stream);
        case 5: return launch<1024>(in, out, rows, clamp, sms, stream);
        default: return cudaErrorInvalidValue;
    }
}
