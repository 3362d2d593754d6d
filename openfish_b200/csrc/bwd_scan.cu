// bwd_scan.cu -- backward scan of the CRF-CTC decode for sm_100a.
//
// Replaces the reference kernel bwd_scan (src/scan_cuda.cu:8-57) and reproduces the CPU
// routine backward_scan (src/decode_cpu.c:13-52) bit for bit (see exact_math.cuh):
//   bwd[n][T][s] = 0
//   bwd[n][t][s] = LSE5( bwd[n][t+1][s] + stay,
//                        bwd[n][t+1][u+b] + score[t][n][4(u+b) + k] , b = 0..3 )
//   with s = j + k*ns/4 (j < ns/4), u = 4j.
//
// Shape of the kernel.  One thread owns the four states {j + k*ns/4}: they share the four
// successors u..u+3 (one 16-byte read of the previous row) and their 16 transition scores are
// one contiguous 32-byte piece of the score row, so nothing is read twice and nothing is
// strided.  A block runs CPB chunks side by side (ns/4 threads each).  The previous row lives
// in shared memory (ping-pong, one block barrier per timestep); score rows arrive through a
// ring of 1-D bulk asynchronous copies tracked by mbarriers, issued a ring length ahead by one
// thread, newest timestep first because the scan runs backwards in time.  Output rows go
// straight to HBM as coalesced 4-byte stores.
//
// The scan is bound by the FP64 pipe (about 68 FP64 operations per state and timestep), not
// by HBM: it moves T*4ns*2 + (T+1)*ns*4 bytes per chunk.
#include "bwd_scan.cuh"
#include "exact_math.cuh"
#include "of_device.cuh"

namespace {

constexpr int kExpCopies = 16;  // per-half-warp-lane copies of the 2^(j/32) table

template <int NS, int CPB, int RING>
struct BwdSmem {
    static constexpr int kRowBytes = NS * 4 * 2;            // one chunk's score row (fp16)
    static constexpr int kSlotBytes = kRowBytes * CPB;      // one timestep of the block
    alignas(128) unsigned char ring[RING][kSlotBytes];
    alignas(16) float alpha[2][CPB][NS];
    alignas(16) double exp2_rep[ofx::kExpTab * kExpCopies];
    double rcp_c[ofx::kLogTab];
    double log_c[ofx::kLogTab];
    alignas(8) uint64_t full[RING];
    int abort_flag;
};

__device__ __forceinline__ float half_at(const uint4 &lo, const uint4 &hi, int i) {
    // i is a compile-time constant after unrolling
    const uint32_t w = i < 8 ? (&lo.x)[i >> 1] : (&hi.x)[(i - 8) >> 1];
    const unsigned short h = (i & 1) ? (unsigned short)(w >> 16) : (unsigned short)(w & 0xffffu);
    return __half2float(__ushort_as_half(h));
}

template <int NS, int CPB, int RING>
__global__ void __launch_bounds__((NS / 4) * CPB)
bwd_scan_kernel(const __half *__restrict__ scores, float *__restrict__ bwd, int T, int N,
                float stay, const ofx::Tables *__restrict__ tables, int *status) {
    constexpr int TPC = NS / 4;  // threads per chunk
    using Smem = BwdSmem<NS, CPB, RING>;
    extern __shared__ unsigned char smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x;
    const int cl = tid / TPC;  // chunk within the block
    const int j = tid % TPC;
    const int chunk0 = blockIdx.x * CPB;
    const int chunk = chunk0 + cl;
    const bool live = chunk < N;
    const int nlive = min(CPB, N - chunk0);
    const uint32_t slot_bytes = (uint32_t)nlive * Smem::kRowBytes;

    // tables -> shared memory (the exp table interleaved so that lane l of a half-warp reads
    // copy l: 8-byte reads then never collide on a bank)
    for (int i = tid; i < ofx::kExpTab * kExpCopies; i += blockDim.x)
        sm.exp2_rep[i] = tables->exp2_j[i / kExpCopies];
    for (int i = tid; i < ofx::kLogTab; i += blockDim.x) {
        sm.rcp_c[i] = tables->rcp_c[i];
        sm.log_c[i] = tables->log_c[i];
    }
    if (tid == 0) {
        sm.abort_flag = 0;
        for (int r = 0; r < RING; ++r) ofd::mbar_init(&sm.full[r], 1);
        ofd::mbar_fence_init();
    }
    __syncthreads();

    // the scans address scores as [T][N][4ns] whatever C is (src/decode_cpu.c:16-18,27)
    const size_t t_stride = (size_t)N * NS * 4;  // elements
    const __half *blk_scores = scores + (size_t)chunk0 * NS * 4;
    if (tid == 0) {
        for (int i = 0; i < RING && i < T; ++i) {
            ofd::mbar_arrive_expect_tx(&sm.full[i], slot_bytes);
            ofd::bulk_g2s(sm.ring[i], blk_scores + t_stride * (size_t)(T - 1 - i), slot_bytes,
                          &sm.full[i]);
        }
    }

    const ofx::TabRef tr = {sm.exp2_rep + (tid & (kExpCopies - 1)), kExpCopies, sm.rcp_c, sm.log_c};
    float *out_chunk = bwd + (size_t)(live ? chunk : 0) * (size_t)(T + 1) * NS;

    float own[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        sm.alpha[0][cl][j + k * TPC] = 0.f;
        if (live) out_chunk[(size_t)T * NS + j + k * TPC] = 0.f;
    }
    __syncthreads();

    const int sw = (j >> 2) & 1;  // read the two 16-byte halves in an order that spreads banks
    for (int i = 0; i < T; ++i) {
        const int t = T - 1 - i;
        const int slot = i % RING;
        ofd::mbar_wait_bounded(&sm.full[slot], (uint32_t)(i / RING) & 1u, &sm.abort_flag, status);

        const unsigned char *row = sm.ring[slot] + cl * Smem::kRowBytes + 32 * j;
        const uint4 p0 = *reinterpret_cast<const uint4 *>(row + 16 * sw);
        const uint4 p1 = *reinterpret_cast<const uint4 *>(row + 16 * (1 - sw));
        const uint4 lo = sw ? p1 : p0;
        const uint4 hi = sw ? p0 : p1;
        const float4 nx = *reinterpret_cast<const float4 *>(&sm.alpha[i & 1][cl][4 * j]);
        const float nxt[4] = {nx.x, nx.y, nx.z, nx.w};

        float res[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {  // a padding chunk of the last block has no data to work on
            float v[4][5];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                v[k][0] = own[k] + stay;
#pragma unroll
                for (int b = 0; b < 4; ++b) v[k][b + 1] = nxt[b] + half_at(lo, hi, 4 * b + k);
            }
            ofx::lse5_batch_exact<4>(v, res, tr);
        }
        float *arow = sm.alpha[(i & 1) ^ 1][cl];
        float *grow = out_chunk + (size_t)t * NS;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            own[k] = res[k];
            arow[j + k * TPC] = res[k];
            if (live) grow[j + k * TPC] = res[k];
        }
        __syncthreads();  // row t complete in shared memory; ring slot fully consumed
        if (tid == 0 && i + RING < T) {
            ofd::mbar_arrive_expect_tx(&sm.full[slot], slot_bytes);
            ofd::bulk_g2s(sm.ring[slot], blk_scores + t_stride * (size_t)(T - 1 - (i + RING)),
                          slot_bytes, &sm.full[slot]);
        }
    }
}

template <int NS, int CPB, int RING>
cudaError_t launch(const __half *scores, float *bwd, int T, int N, float stay,
                   const ofx::Tables *tables, int *status, cudaStream_t stream) {
    using Smem = BwdSmem<NS, CPB, RING>;
    const size_t bytes = sizeof(Smem) + 128;
    auto kern = bwd_scan_kernel<NS, CPB, RING>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    const int blocks = (N + CPB - 1) / CPB;
    kern<<<blocks, (NS / 4) * CPB, bytes, stream>>>(scores, bwd, T, N, stay, tables, status);
    return cudaGetLastError();
}

}  // namespace

cudaError_t of_launch_bwd_scan(const void *scores_fp16, float *bwd, int T, int N, int state_len,
                               float stay, const ofx::Tables *tables, int *status,
                               cudaStream_t stream) {
    const __half *s = static_cast<const __half *>(scores_fp16);
    switch (state_len) {
        case 3: return launch<64, 4, 8>(s, bwd, T, N, stay, tables, status, stream);
        case 4: return launch<256, 1, 8>(s, bwd, T, N, stay, tables, status, stream);
        case 5: return launch<1024, 1, 6>(s, bwd, T, N, stay, tables, status, stream);
        default: return cudaErrorInvalidValue;
    }
}
