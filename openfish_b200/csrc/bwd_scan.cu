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
// ring of 1-D bulk asynchronous copies tracked by mbarriers, issued a ring length ahead by a
// copy warp of their own, newest timestep first because the scan runs backwards in time.  Output rows go
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
__global__ void __launch_bounds__((NS / SPT) * CPB + 32)
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
    if (tid >= TPC * CPB) {
        // ------------------------------------------------------------------ copy warp
        // Keeps the ring of score rows full and takes every mbarrier operation off the scan
        // warps: before it joins the barrier that ends timestep i it has seen row i+1 land, so
        // the barrier hands that knowledge (and the data) to everybody; after the barrier the
        // slot of row i is free and is refilled.
        const bool issuer = tid == TPC * CPB;
        if (issuer) {
            for (int i = 0; i < RING && i < T; ++i) {
                ofd::mbar_arrive_expect_tx(&sm.full[i], slot_bytes);
                ofd::bulk_g2s(sm.ring[i], blk_scores + t_stride * (size_t)(T - 1 - i), slot_bytes,
                              &sm.full[i]);
            }
            if (T > 0) ofd::mbar_wait_bounded(&sm.full[0], 0u, &sm.abort_flag, status);
        }
        __syncthreads();
        for (int i = 0; i < T; ++i) {
            if (issuer && i + 1 < T)
                ofd::mbar_wait_bounded(&sm.full[(i + 1) % RING], (uint32_t)((i + 1) / RING) & 1u,
                                       &sm.abort_flag, status);
            __syncthreads();
            if (issuer && i + RING < T) {
                const int slot = i % RING;
                ofd::mbar_arrive_expect_tx(&sm.full[slot], slot_bytes);
                ofd::bulk_g2s(sm.ring[slot], blk_scores + t_stride * (size_t)(T - 1 - (i + RING)),
                              slot_bytes, &sm.full[slot]);
            }
        }
        return;
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
        __syncthreads();  // row t complete; the copy warp has confirmed the next score row
    }
}

// ------------------------------------------------------------------------------------------
// Speculative variant (one chunk per block).
//
// In the kernel above a state whose rounding the fp32 evaluation cannot certify sends its whole
// warp through the value-exact routine before the timestep can end, and almost every timestep
// has a few such states: the exact routine's latency is paid on nearly every step.  Here the
// scan warps do not wait for it.  An uncertified state gets the likelier of its two candidate
// floats and is put on a list; while the scan warps work on the next timestep, a checker warp
// recomputes the listed states exactly.  If every guess was right (about three timesteps in
// four) nothing else happens.  If one was wrong the block pauses at the end of that next
// timestep: the checker corrects the value and recomputes exactly the five states of the next
// row that read it (the state itself and the four that have it as a successor) before anybody
// reads those, and the scan carries on.  (Letting the scan run on and chasing the consequences
// a step behind does not work: a one-ulp change of an input moves an output by one ulp with a
// probability equal to that input's weight in the sum, and the weights of a state over its five
// readers add up to about one, so corrections would breed as fast as they die.)  What reaches
// HBM is, value for value, what the exact routine alone would have produced.  Three row buffers
// rotate so that the inputs of a timestep are still there while it is being checked, and score
// rows are released one timestep late.
template <int NS, int SPT, int RING>
struct BwdSpecSmem {
    static constexpr int kRowBytes = NS * 4 * 2;
    static constexpr int NW = NS / SPT / 32;  // scan warps
    static constexpr int kPerWarp = 8;        // listed states per warp and timestep, at most
    alignas(128) unsigned char ring[RING][kRowBytes];
    alignas(16) float alpha[3][NS];
    alignas(16) double exp2_rep[ofx::kExpTab * kExpCopies];
    double rcp_c[ofx::kLogTab];
    double log_c[ofx::kLogTab];
    alignas(8) uint64_t full[RING];
    unsigned short listed[2][NW][kPerWarp];
    int n_listed[2][NW];
    int n_wrong[2];
    unsigned short wrong_state[NW * kPerWarp];
    float wrong_value[NW * kPerWarp];
    int abort_flag;
};

// The five terms of state s at the timestep whose score row is `row` and whose input row is `in`.
template <int NS>
__device__ __forceinline__ void terms_of(int s, const float *in, const unsigned char *row, float stay,
                                         float (&v)[5]) {
    constexpr int NJ = NS / 4;
    const int j = s % NJ, k = s / NJ;
    const __half *sc = reinterpret_cast<const __half *>(row) + 16 * j + k;
    v[0] = in[s] + stay;
#pragma unroll
    for (int b = 0; b < 4; ++b) v[b + 1] = in[4 * j + b] + __half2float(sc[4 * b]);
}

template <int NS, int SPT, int RING>
__global__ void __launch_bounds__(NS / SPT + 64)
bwd_scan_spec_kernel(const __half *__restrict__ scores, float *__restrict__ bwd, int T, int N,
                     float stay, const ofx::Tables *__restrict__ tables, int *status) {
    constexpr int NJ = NS / 4;
    constexpr int TPC = NS / SPT;
    using Smem = BwdSpecSmem<NS, SPT, RING>;
    constexpr int NW = Smem::NW, PER = Smem::kPerWarp;
    static_assert(TPC % 32 == 0, "scan warps must be full");
    extern __shared__ unsigned char smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x;
    for (int i = tid; i < ofx::kExpTab * kExpCopies; i += blockDim.x)
        sm.exp2_rep[i] = tables->exp2_j[i / kExpCopies];
    for (int i = tid; i < ofx::kLogTab; i += blockDim.x) {
        sm.rcp_c[i] = tables->rcp_c[i];
        sm.log_c[i] = tables->log_c[i];
    }
    for (int i = tid; i < 2 * NW; i += blockDim.x) (&sm.n_listed[0][0])[i] = 0;
    for (int i = tid; i < NS; i += blockDim.x) sm.alpha[0][i] = 0.f;
    if (tid == 0) {
        sm.abort_flag = 0;
        sm.n_wrong[0] = sm.n_wrong[1] = 0;
        for (int r = 0; r < RING; ++r) ofd::mbar_init(&sm.full[r], 1);
        ofd::mbar_fence_init();
    }
    __syncthreads();

    const size_t t_stride = (size_t)N * NS * 4;
    const __half *chunk_scores = scores + (size_t)chunk * NS * 4;
    float *out_chunk = bwd + (size_t)chunk * (size_t)(T + 1) * NS;
    const ofx::TabRef tr = {sm.exp2_rep + (tid & (kExpCopies - 1)), kExpCopies, sm.rcp_c, sm.log_c};

    if (warp == NW) {
        // ------------------------------------------------------------------ copy warp
        // A slot is refilled one timestep late: the checker still reads the scores of the
        // timestep it is checking.
        const bool issuer = lane == 0;
        if (issuer) {
            for (int i = 0; i < RING && i < T; ++i) {
                ofd::mbar_arrive_expect_tx(&sm.full[i], Smem::kRowBytes);
                ofd::bulk_g2s(sm.ring[i], chunk_scores + t_stride * (size_t)(T - 1 - i),
                              Smem::kRowBytes, &sm.full[i]);
            }
            if (T > 0) ofd::mbar_wait_bounded(&sm.full[0], 0u, &sm.abort_flag, status);
        }
        __syncthreads();
        for (int i = 0; i < T; ++i) {
            if (issuer && i + 1 < T)
                ofd::mbar_wait_bounded(&sm.full[(i + 1) % RING], (uint32_t)((i + 1) / RING) & 1u,
                                       &sm.abort_flag, status);
            __syncthreads();
            if (sm.n_wrong[i & 1]) __syncthreads();
            if (issuer && i >= 1 && i - 1 + RING < T) {
                const int slot = (i - 1) % RING;
                ofd::mbar_arrive_expect_tx(&sm.full[slot], Smem::kRowBytes);
                ofd::bulk_g2s(sm.ring[slot], chunk_scores + t_stride * (size_t)(T - 1 - (i - 1 + RING)),
                              Smem::kRowBytes, &sm.full[slot]);
            }
        }
        return;
    }

    if (warp == NW + 1) {
        // ------------------------------------------------------------------ checker warp
        __syncthreads();  // start of the scan
        for (int i = 0; i <= T; ++i) {
            // During timestep i (for i = T: after the last one) check the states listed during
            // timestep i-1: inputs alpha[(i-1)%3], scores in slot (i-1)%RING, guesses in
            // alpha[i%3] and in output row T-i.
            int nw = 0;
            if (i >= 1) {
                const int par = (i - 1) & 1;
                int total = 0;
#pragma unroll
                for (int w = 0; w < NW; ++w) total += sm.n_listed[par][w];
                for (int base = 0; base < total; base += 32) {
                    const int e = base + lane;
                    int s = 0, acc = 0;
#pragma unroll
                    for (int w = 0; w < NW; ++w) {
                        const int c = sm.n_listed[par][w];
                        if (e >= acc && e < acc + c) s = sm.listed[par][w][e - acc];
                        acc += c;
                    }
                    float v[5];
                    terms_of<NS>(s, sm.alpha[(i - 1) % 3], sm.ring[(i - 1) % RING], stay, v);
                    const float x = ofx::lse5_exact(v, tr);
                    const bool wrong = e < total && __float_as_uint(x) != __float_as_uint(sm.alpha[i % 3][s]);
                    const uint32_t wm = __ballot_sync(0xffffffffu, wrong);
                    if (wrong) {
                        const int at = nw + __popc(wm & ((1u << lane) - 1u));
                        sm.wrong_state[at] = (unsigned short)s;
                        sm.wrong_value[at] = x;
                    }
                    nw += __popc(wm);
                }
                __syncwarp();
            }
            if (i == T) {
                // the last row: nobody reads it any more, just correct it
                for (int e = lane; e < nw; e += 32) out_chunk[sm.wrong_state[e]] = sm.wrong_value[e];
                break;
            }
            if (lane == 0) sm.n_wrong[i & 1] = nw;
            __syncthreads();  // end of timestep i
            if (nw) {
                for (int e = lane; e < nw; e += 32) {
                    const int s = sm.wrong_state[e];
                    sm.alpha[i % 3][s] = sm.wrong_value[e];
                    out_chunk[(size_t)(T - i) * NS + s] = sm.wrong_value[e];
                }
                __syncwarp();
                // the five states of row T-1-i that read a corrected value
                for (int idx = lane; idx < 5 * nw; idx += 32) {
                    const int s = sm.wrong_state[idx / 5], d = idx % 5;
                    const int dep = d == 4 ? s : (s >> 2) + d * NJ;
                    float v[5];
                    terms_of<NS>(dep, sm.alpha[i % 3], sm.ring[i % RING], stay, v);
                    const float x = ofx::lse5_exact(v, tr);
                    sm.alpha[(i + 1) % 3][dep] = x;
                    out_chunk[(size_t)(T - 1 - i) * NS + dep] = x;
                }
                __syncthreads();  // corrections in place
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- scan warps
    const int j = tid % NJ;
    const int k0 = (tid / NJ) * SPT;
#pragma unroll
    for (int k = 0; k < SPT; ++k) out_chunk[(size_t)T * NS + j + (k0 + k) * NJ] = 0.f;
    __syncthreads();
    const int sw = (j >> 2) & 1;
    const uint32_t lt_mask = (1u << lane) - 1u;
    for (int i = 0; i < T; ++i) {
        const int t = T - 1 - i;
        const unsigned char *row = sm.ring[i % RING] + 32 * j;
        const uint4 p0 = *reinterpret_cast<const uint4 *>(row + 16 * sw);
        const uint4 p1 = *reinterpret_cast<const uint4 *>(row + 16 * (1 - sw));
        const uint4 lo = sw ? p1 : p0;
        const uint4 hi = sw ? p0 : p1;
        const float4 nx = *reinterpret_cast<const float4 *>(&sm.alpha[i % 3][4 * j]);
        const float nxt[4] = {nx.x, nx.y, nx.z, nx.w};
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float v[SPT][5], res[SPT];
        bool ok[SPT];
#pragma unroll
        for (int k = 0; k < SPT; ++k) {
            // (the stay term is read from the row, not kept in a register: the checker may
            // have corrected it)
            v[k][0] = sm.alpha[i % 3][j + (k0 + k) * NJ] + stay;
#pragma unroll
            for (int b = 0; b < 4; ++b) v[k][b + 1] = nxt[b] + score_of<SPT>(w, b, k0, k);
        }
        ofd::lse5_fast_guess<SPT>(v, res, ok);
        uint32_t bad[SPT];
        int total = 0;
#pragma unroll
        for (int k = 0; k < SPT; ++k) {
            bad[k] = __ballot_sync(0xffffffffu, !ok[k]);
            total += __popc(bad[k]);
        }
        if (total > PER) {
            // many uncertified states (the first few hundred timesteps, where scores are small
            // and the float grid fine): settle them here and now, nothing to check later
            ofd::lse5_batch<SPT>(v, res, tr);
            total = 0;
        } else if (total) {
            int base = 0;
#pragma unroll
            for (int k = 0; k < SPT; ++k) {
                if (!ok[k]) sm.listed[i & 1][warp][base + __popc(bad[k] & lt_mask)] = (unsigned short)(j + (k0 + k) * NJ);
                base += __popc(bad[k]);
            }
        }
        if (lane == 0) sm.n_listed[i & 1][warp] = total;
        float *arow = sm.alpha[(i + 1) % 3];
        float *grow = out_chunk + (size_t)t * NS;
#pragma unroll
        for (int k = 0; k < SPT; ++k) {
            arow[j + (k0 + k) * NJ] = res[k];
            grow[j + (k0 + k) * NJ] = res[k];
        }
        __syncthreads();
        if (sm.n_wrong[i & 1]) __syncthreads();  // the checker is correcting this row's readers
    }
}

template <int NS, int SPT, int RING>
cudaError_t launch_spec(const __half *scores, float *bwd, int T, int N, float stay,
                        const ofx::Tables *tables, int *status, cudaStream_t stream) {
    using Smem = BwdSpecSmem<NS, SPT, RING>;
    const size_t bytes = sizeof(Smem) + 128;
    auto kern = bwd_scan_spec_kernel<NS, SPT, RING>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    kern<<<N, NS / SPT + 64, bytes, stream>>>(scores, bwd, T, N, stay, tables, status);
    return cudaGetLastError();
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
    kern<<<blocks, (NS / SPT) * CPB + 32, bytes, stream>>>(scores, bwd, T, N, stay, tables, status);
    return cudaGetLastError();
}

}  // namespace

cudaError_t of_launch_bwd_scan(const void *scores_fp16, float *bwd, int T, int N, int state_len,
                               float stay, const ofx::Tables *tables, int *status,
                               cudaStream_t stream) {
    const __half *s = static_cast<const __half *>(scores_fp16);
    switch (state_len) {
        case 3: return launch<64, 1, 2, 8>(s, bwd, T, N, stay, tables, status, stream);
        case 4: return launch_spec<256, 4, 8>(s, bwd, T, N, stay, tables, status, stream);
        case 5: return launch<1024, 2, 1, 6>(s, bwd, T, N, stay, tables, status, stream);
        default: return cudaErrorInvalidValue;
    }
}
