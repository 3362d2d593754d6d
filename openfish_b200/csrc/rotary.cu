// rotary.cu -- in-place rotary position embedding on fp16 activations for sm_100a.
//
// Replaces rotary_emb_cuda / rotary_emb (src/nn_cuda.cu:10-40, src/rotary_emb_cuda.cuh:35-69):
// for every (batch, position, head) the pairs (i, i + rotary_half) of the head vector are
// rotated by the angle whose cosine/sine sit at [position][i] of two fp32 tables:
//   o0 = x0*cos - x1*sin,  o1 = x0*sin + x1*cos   (fp32 math, fp16 storage).
// The op is pure HBM streaming (read + write of the rotated part of x), so the kernel moves
// 16 bytes per access: one thread rotates eight consecutive pairs of two heads with the same
// eight angles, a grid-stride loop over positions keeps every SM busy whatever the shape.  Shapes or pointers that do not allow 16-byte accesses use
// a scalar kernel with the same arithmetic.
#include <cuda_fp16.h>
#include <stdint.h>

#include "rotary.cuh"

namespace {

struct RotArgs {
    __half *x;
    const float *cos_t;
    const float *sin_t;
    long long stride_batch, stride_seq, stride_head;
    int batch, seqlen, nheads, rotary_half;
};

__device__ __forceinline__ void rotate(float x0, float x1, float c, float s, float &o0, float &o1) {
    // same operation order as the CPU routine (src/nn_cpu.c:36-37), no fused multiply-add
    o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    o1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

// blockDim.x threads cover one position's (head group, pair group) items, blockDim.y positions
// per block; the grid strides over positions.  A thread keeps its pair group and its HPT heads for
// the whole launch, so the index arithmetic per position is one division, and the eight cosines
// and sines it loads serve HPT heads.  All 2*HPT 16-byte loads of a position are issued before
// the first is used.
template <int HPT>
__global__ void __launch_bounds__(256) rotary_vec8_kernel(const RotArgs a) {
    const int groups = a.rotary_half >> 3;  // eight pairs per item
    const int head_sets = a.nheads / HPT;
    const int per_pos = head_sets * groups;
    const long long positions = (long long)a.batch * a.seqlen;
    const long long hop = (long long)head_sets * a.stride_head;
    for (int r = threadIdx.x; r < per_pos; r += blockDim.x) {
        const int g = r % groups;
        const int h0 = r / groups;  // this thread's heads: h0, h0 + head_sets, ... (neighbours in a warp
                                    // take neighbouring heads, so each load instruction covers whole lines)
        for (long long pos = (long long)blockIdx.x * blockDim.y + threadIdx.y; pos < positions;
             pos += (long long)gridDim.x * blockDim.y) {
            const int t = (int)(pos % a.seqlen);
            const long long b = pos / a.seqlen;
            __half *base = a.x + b * a.stride_batch + (long long)t * a.stride_seq + h0 * a.stride_head + 8 * g;
            const float4 *cp = reinterpret_cast<const float4 *>(a.cos_t + (long long)t * a.rotary_half + 8 * g);
            const float4 *sp = reinterpret_cast<const float4 *>(a.sin_t + (long long)t * a.rotary_half + 8 * g);
            uint4 v0[HPT], v1[HPT];
#pragma unroll
            for (int k = 0; k < HPT; ++k) {
                v0[k] = *reinterpret_cast<const uint4 *>(base + k * hop);
                v1[k] = *reinterpret_cast<const uint4 *>(base + k * hop + a.rotary_half);
            }
            const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int k = 0; k < HPT; ++k) {
                __half2 *x0 = reinterpret_cast<__half2 *>(&v0[k]);
                __half2 *x1 = reinterpret_cast<__half2 *>(&v1[k]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 a0 = __half22float2(x0[i]);
                    const float2 a1 = __half22float2(x1[i]);
                    float o00, o10, o01, o11;
                    rotate(a0.x, a1.x, c[2 * i], s[2 * i], o00, o10);
                    rotate(a0.y, a1.y, c[2 * i + 1], s[2 * i + 1], o01, o11);
                    x0[i] = __floats2half2_rn(o00, o01);
                    x1[i] = __floats2half2_rn(o10, o11);
                }
                *reinterpret_cast<uint4 *>(base + k * hop) = v0[k];
                *reinterpret_cast<uint4 *>(base + k * hop + a.rotary_half) = v1[k];
            }
        }
    }
}

__global__ void __launch_bounds__(256) rotary_scalar_kernel(const RotArgs a) {
    const long long per_pos = (long long)a.nheads * a.rotary_half;
    const long long total = (long long)a.batch * a.seqlen * per_pos;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total;
         w += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(w % a.rotary_half);
        const int h = (int)((w / a.rotary_half) % a.nheads);
        const long long bt = w / per_pos;
        const int t = (int)(bt % a.seqlen);
        const long long b = bt / a.seqlen;
        __half *p0 = a.x + b * a.stride_batch + (long long)t * a.stride_seq + h * a.stride_head + i;
        __half *p1 = p0 + a.rotary_half;
        float o0, o1;
        rotate(__half2float(*p0), __half2float(*p1), a.cos_t[(long long)t * a.rotary_half + i],
               a.sin_t[(long long)t * a.rotary_half + i], o0, o1);
        *p0 = __float2half_rn(o0);
        *p1 = __float2half_rn(o1);
    }
}

}  // namespace

cudaError_t of_launch_rotary(void *x, const void *sin_t, const void *cos_t, int batch, int seqlen,
                             int nheads, int rotary_half, long long stride_batch,
                             long long stride_seq, long long stride_head, int sm_count,
                             cudaStream_t stream) {
    RotArgs a;
    a.x = static_cast<__half *>(x);
    a.cos_t = static_cast<const float *>(cos_t);
    a.sin_t = static_cast<const float *>(sin_t);
    a.stride_batch = stride_batch; a.stride_seq = stride_seq; a.stride_head = stride_head;
    a.batch = batch; a.seqlen = seqlen; a.nheads = nheads; a.rotary_half = rotary_half;
    const bool vec = (rotary_half % 8 == 0) && (stride_batch % 8 == 0) && (stride_seq % 8 == 0) &&
                     (stride_head % 8 == 0) && ((uintptr_t)x % 16 == 0) &&
                     ((uintptr_t)sin_t % 16 == 0) && ((uintptr_t)cos_t % 16 == 0);
    if ((long long)batch * seqlen * nheads * rotary_half <= 0) return cudaSuccess;
    if (vec) {
        const int hpt = nheads % 2 == 0 ? 2 : 1;  // (four heads per thread measured slower than two)
        const int per_pos = (nheads / hpt) * (rotary_half / 8);
        int bx = 1;
        while (bx < per_pos && bx < 256) bx <<= 1;  // 1..256 threads across one position
        const dim3 block(bx, 256 / bx);
        const long long positions = (long long)batch * seqlen;
        long long blocks = (positions + block.y - 1) / block.y;
        const long long cap = (long long)sm_count * 16;  // two waves of eight resident 256-thread blocks per SM
        if (blocks > cap) blocks = cap;
        if (hpt == 2) rotary_vec8_kernel<2><<<(unsigned)blocks, block, 0, stream>>>(a);
        else rotary_vec8_kernel<1><<<(unsigned)blocks, block, 0, stream>>>(a);
    } else {
        const long long items = (long long)batch * seqlen * nheads * rotary_half;
        long long blocks = (items + 255) / 256;
        const long long cap = (long long)sm_count * 8;
        if (blocks > cap) blocks = cap;
        rotary_scalar_kernel<<<(unsigned)blocks, 256, 0, stream>>>(a);
    }
    return cudaGetLastError();
}
