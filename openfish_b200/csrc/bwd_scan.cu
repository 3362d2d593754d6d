// bwd_scan.cu -- backward scan of the CRF-CTC decode for sm_100a.
//
// Replaces the reference kernel bwd_scan (src/scan_cuda.cu:8-57) and reproduces the CPU
// routine backward_scan (src/decode_cpu.c:13-52) bit for bit (see exact_math.cuh):
//   bwd[n][T][s] = 0
//   bwd[n][t][s] = LSE5( bwd[n][t+1][s] + stay,
//                        bwd[n][t+1][u+b] + score[t][n][4(u+b) + k] , b = 0..3 )
//   with s = j + k*ns/4 (j < ns/4), u = 4j.
//
// Shape of the kernel.  The four states {j + k*ns/4} share the four successors u..u+3 (one
// 16-byte read of the previous row) and their 16 transition scores are one contiguous 32-byte
// piece of the score row, so nothing is strided.  SPT of those four states go to one thread
// (4/SPT threads share a j); fewer states per thread means more warps per chunk, which is what
// hides the FP64 latency when only three or four chunks fit on an SM.  A block runs CPB chunks
// side by side (ns/SPT threads each).  The previous row lives
// in shared memory (ping-pong, one block barrier per timestep); score rows arrive through a
// ring of 1-D bulk asynchronous copies tracked by mbarriers, issued a ring length ahead by one
// thread, newest timestep first because the scan runs backwards in time.  Output rows go
// straight to HBM as coalesced 4-byte stores.
//
// The scan is bound by the FP64 pipe (about 68 FP64 operations per state and timestep), not
// by HBM: it moves T*4ns*2 + (T+1)*ns*4 bytes per chunk.
#include "bwd_scan.cuh"
#include "exact_math.cuh"
#include "fast_lse.cuh"
#include "of_device.cuh"

namespace {

constexpr int kExpCopies = 16;  // per-half-warp-lane copies of the 2^(j/32) table

// Score of (base b, state slot k0 + k) out of a 32-byte piece held as eight 32-bit words:
// half number 4b + k0 + k.  k0 is a multiple of SPT known only at run time, k < SPT at compile time.
template <int SPT>
__device__ __forceinline__ float score_of(const uint32_t (&w)[8], int b, int k0, int k) {
    if (SPT == 4) {
        const uint32_t x = w[2 * b + (k >> 1)];
        return __half2float(__ushort_as_half((unsigned short)((k & 1) ? (x >> 16) : (x & 0xffffu))));
    }
    const uint32_t x = (k0 & 2) ? w[2 * b + 1] : w[2 * b];
    if (SPT == 2)
        return __half2float(__ushort_as_half((unsigned short)(k ? (x >> 16) : (x & 0xffffu))));
    return __half2float(__ushort_as_half((unsigned short)((x >> ((k0 & 1) * 16)) & 0xffffu)));
}

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

template <int NS, int SPT, int CPB, int RING>
__global__ void __launch_bounds__((NS / SPT) * CPB)
bwd_scan_kernel(const __half *__restrict__ scores, float *__restrict__ bwd, int T, int N,
                float stay, const ofx::Tables *__restrict__ tables, int *status) {
    constexpr int NJ = NS / 4;     // groups of four states that share successors
    constexpr int TPC = NS / SPT;  // threads per chunk
    static_assert(TPC % 32 == 0, "a warp must not straddle two chunks");
    using Smem = BwdSmem<NS, CPB, RING>;
    extern __shared__ unsigned char smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x;
    const int cl = tid / TPC;  // chunk within the block
    const int j = tid % NJ;
    const int k0 = ((tid % TPC) / NJ) * SPT;  // first of this thread's states j + k*NJ
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

    float own[SPT];
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        own[k] = 0.f;
        sm.alpha[0][cl][j + (k0 + k) * NJ] = 0.f;
        if (live) out_chunk[(size_t)T * NS + j + (k0 + k) * NJ] = 0.f;
    }
    if (tid == 0 && T > 0) ofd::mbar_wait_bounded(&sm.full[0], 0u, &sm.abort_flag, status);
    __syncthreads();

    const int sw = (j >> 2) & 1;  // read the two 16-byte halves in an order that spreads banks
    for (int i = 0; i < T; ++i) {
        const int t = T - 1 - i;
        const int slot = i % RING;

        const unsigned char *row = sm.ring[slot] + cl * Smem::kRowBytes + 32 * j;
        const uint4 p0 = *reinterpret_cast<const uint4 *>(row + 16 * sw);
        const uint4 p1 = *reinterpret_cast<const uint4 *>(row + 16 * (1 - sw));
        const uint4 lo = sw ? p1 : p0;
        const uint4 hi = sw ? p0 : p1;
        const float4 nx = *reinterpret_cast<const float4 *>(&sm.alpha[i & 1][cl][4 * j]);
        const float nxt[4] = {nx.x, nx.y, nx.z, nx.w};
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};

        float res[SPT];
#pragma unroll
        for (int k = 0; k < SPT; ++k) res[k] = 0.f;
        if (live) {  // a padding chunk of the last block has no data to work on
            float v[SPT][5];
#pragma unroll
            for (int k = 0; k < SPT; ++k) {
                v[k][0] = own[k] + stay;
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    v[k][b + 1] = nxt[b] + score_of<SPT>(w, b, k0, k);
            }
            ofd::lse5_batch<SPT>(v, res, tr);
        }
        float *arow = sm.alpha[(i & 1) ^ 1][cl];
        float *grow = out_chunk + (size_t)t * NS;
#pragma unroll
        for (int k = 0; k < SPT; ++k) {
            own[k] = res[k];
            arow[j + (k0 + k) * NJ] = res[k];
            if (live) grow[j + (k0 + k) * NJ] = res[k];
        }
        // One thread makes sure the next timestep's scores have landed; the barrier then makes
        // them (and row t) visible to everybody and tells that thread the slot just used is free.
        if (tid == 0 && i + 1 < T)
            ofd::mbar_wait_bounded(&sm.full[(i + 1) % RING], (uint32_t)((i + 1) / RING) & 1u,
                                   &sm.abort_flag, status);
        __syncthreads();
        if (tid == 0 && i + RING < T) {
            ofd::mbar_arrive_expect_tx(&sm.full[slot], slot_bytes);
            ofd::bulk_g2s(sm.ring[slot], blk_scores + t_stride * (size_t)(T - 1 - (i + RING)),
                          slot_bytes, &sm.full[slot]);
        }
    }
}

template <int NS, int SPT, int CPB, int RING>
cudaError_t launch(const __half *scores, float *bwd, int T, int N, float stay,
                   const ofx::Tables *tables, int *status, cudaStream_t stream) {
    using Smem = BwdSmem<NS, CPB, RING>;
    const size_t bytes = sizeof(Smem) + 128;
    auto kern = bwd_scan_kernel<NS, SPT, CPB, RING>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    const int blocks = (N + CPB - 1) / CPB;
    kern<<<blocks, (NS / SPT) * CPB, bytes, stream>>>(scores, bwd, T, N, stay, tables, status);
    return cudaGetLastError();
}

}  // namespace

cudaError_t of_launch_bwd_scan(const void *scores_fp16, float *bwd, int T, int N, int state_len,
                               float stay, const ofx::Tables *tables, int *status,
                               cudaStream_t stream) {
    const __half *s = static_cast<const __half *>(scores_fp16);
    switch (state_len) {
        case 3: return launch<64, 1, 2, 8>(s, bwd, T, N, stay, tables, status, stream);
        case 4: return launch<256, 4, 1, 8>(s, bwd, T, N, stay, tables, status, stream);
        case 5: return launch<1024, 2, 1, 6>(s, bwd, T, N, stay, tables, status, stream);
        default: return cudaErrorInvalidValue;
    }
}
