// posterior_seq.cu -- posterior, traceback, per-base quality and sequence/qstring generation for
// one chunk per block, for sm_100a.
//
// Replaces the softmax half of the reference kernel fwd_post_scan (src/scan_cuda.cu:147-199),
// the traceback at the end of beam_search (src/beam_search_cuda.cu:517-527) and the kernels
// compute_qual_data (:530-605) and generate_sequence (:52-121); semantics are those of the CPU
// routines (src/decode_cpu.c:115,121-147; src/beam_search.c:430-496 and 49-99).
//
// First (unless the forward scan kernel has done it already: a.fwd null) the posterior =
// softmax over states of fwd + bwd: rows are independent, so each warp
// takes rows of its own and streams them straight from and to HBM (this part is bound by HBM
// bandwidth: it reads 2(T+1)ns and writes (T+1)ns floats per chunk).  No per-row maximum is
// needed: the log partition function is the same for every row, so one offset taken from row 0
// keeps every exponent in range.
// Then the whole block walks the back-pointers the beam search left in HBM (staged through
// shared memory in windows), rebuilds the k-mer of every path element from the emitted bases,
// gathers the posterior of each path k-mer and its shifted neighbours, and emits moves,
// sequence and qstring, zero-filling the unused tail of each row.
#include <float.h>

#include "beam_post.cuh"
#include "fast_lse.cuh"
#include "of_device.cuh"

namespace {

constexpr int kBeam = 32;
constexpr int kWin = 256;  // traceback window, timesteps
using ofd::ex2_approx;
constexpr float kLog2e = 1.4426950408889634f;

// SPT (1, 2 or 4) consecutive floats through one vector access.
template <int SPT>
__device__ __forceinline__ void load_floats(float (&d)[SPT], const float *p) {
    if constexpr (SPT == 4) {
        const float4 v = *reinterpret_cast<const float4 *>(p);
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    } else if constexpr (SPT == 2) {
        const float2 v = *reinterpret_cast<const float2 *>(p);
        d[0] = v.x; d[1] = v.y;
    } else {
        d[0] = *p;
    }
}
template <int SPT>
__device__ __forceinline__ void store_floats(float *p, const float (&d)[SPT]) {
    if constexpr (SPT == 4) *reinterpret_cast<float4 *>(p) = make_float4(d[0], d[1], d[2], d[3]);
    else if constexpr (SPT == 2) *reinterpret_cast<float2 *>(p) = make_float2(d[0], d[1]);
    else *p = d[0];
}
template <int NS>
struct PostSmem {
    float m0;
    int part[256];  // block-scan partials of the tail phase
    // the tail phase's arrays start here and run into the dynamic shared memory behind
    alignas(128) unsigned char tail[128];
};

constexpr int kPostThreads = 256;

template <int NS>
__global__ void __launch_bounds__(kPostThreads)
posterior_seq_kernel(const OfDecodeArgs a) {
    constexpr int BITS = (NS == 64) ? 6 : (NS == 256 ? 8 : 10);
    constexpr int SL = BITS / 2;
    constexpr int MSB = NS / 4;
    constexpr int NT = kPostThreads;
    constexpr int NWARP = NT / 32;
    using Smem = PostSmem<NS>;
    extern __shared__ unsigned char smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int chunk = blockIdx.x;
    const int T = a.T;
    const float *bwd_chunk = a.bwd + (size_t)chunk * (size_t)(T + 1) * NS;
    const float *fwd_chunk = a.fwd + (size_t)chunk * (size_t)(T + 1) * NS;
    float *post_chunk = a.post + (size_t)chunk * (size_t)(T + 1) * NS;
    const unsigned char *bp_chunk = a.bp + (size_t)chunk * (size_t)(T + 1) * kBeam;

    // ---------------------------------------------------------------------- posterior
    // Rows are independent: a warp takes a row, each lane NS/32 of its states (two lanes per
    // 16 bytes for the 64-state model), one shuffle reduction for the row sum.  The softmax
    // offset is the maximum of fwd+bwd at row 0 (= bwd row 0, fwd is zero there): the log
    // partition function is the same for every row, so every exponent stays in range.
    if (a.fwd != nullptr && warp == 0) {
        float m = -FLT_MAX;
        for (int s = lane; s < NS; s += 32) m = fmaxf(m, bwd_chunk[s]);
        m = ofd::warp_max(m);
        if (lane == 0) sm.m0 = m;
    }
    __syncthreads();
    const float m0 = sm.m0;
    constexpr int PER = NS / 32;              // states per lane: 2, 8 or 32
    constexpr int VEC = PER >= 4 ? 4 : PER;   // floats per access
    constexpr int NV = PER / VEC;
    for (int t = warp; t <= T && a.fwd != nullptr; t += NWARP) {
        const float *fr = fwd_chunk + (size_t)t * NS, *br = bwd_chunk + (size_t)t * NS;
        float e[PER];
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float fv[VEC], bv[VEC];
            load_floats<VEC>(fv, fr + (i * 32 + lane) * VEC);
            load_floats<VEC>(bv, br + (i * 32 + lane) * VEC);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                e[i * VEC + k] = ex2_approx(((fv[k] + bv[k]) - m0) * kLog2e);
                part += e[i * VEC + k];
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        const float inv = 1.0f / part;
        float *pr = post_chunk + (size_t)t * NS;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float o[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = e[i * VEC + k] * inv;
            store_floats<VEC>(pr + (i * 32 + lane) * VEC, o);
        }
    }

    // ---------------------------------------------------------------------- tail, whole block
    __syncthreads();
    // arrays laid over the rings (and the dynamic shared memory behind them)
    unsigned char *tail = sm.tail;
    const int Tp = (T + 16) & ~15;
    unsigned char *win = tail;                          // kWin * 32 bytes
    unsigned char *bexit = win + kWin * kBeam;          // [kWin/8][32] slot reached below an 8-row block
    int *bentry = reinterpret_cast<int *>(bexit + (kWin / 8) * kBeam);  // [kWin/8] slot entering each block
    unsigned char *path = reinterpret_cast<unsigned char *>(bentry + kWin / 8);  // [T+1] packed back-pointer of the path
    unsigned char *ext = path + Tp;                     // [SL + T] initial k-mer bases then steps
    unsigned short *cnt = reinterpret_cast<unsigned short *>(ext + Tp + 16);  // [T+1] steps so far
    float *qp = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(cnt) + 2 * Tp);  // [T]

    // traceback from slot 0 of the last row (src/beam_search.c:430-438), window by window.
    // Following one pointer per row is a chain of dependent shared-memory reads, so the chain is
    // shortened eightfold: for every block of 8 rows and each of the 32 slots one could enter it
    // with, all threads first work out where one leaves it (independent short walks); one thread
    // then hops block to block; finally all threads replay their block with the known entry.
    int at = 0;
    for (int hi_r = T; hi_r >= 1; hi_r -= kWin) {
        const int lo_r = max(1, hi_r - kWin + 1);
        const int rows = hi_r - lo_r + 1;
        const int nblk = (rows + 7) >> 3;
        const int n16 = rows * 2;  // 16-byte pieces
        const uint4 *src = reinterpret_cast<const uint4 *>(bp_chunk + (size_t)lo_r * kBeam);
        for (int i = tid; i < n16; i += NT) reinterpret_cast<uint4 *>(win)[i] = __ldcg(src + i);
        __syncthreads();
        for (int w = tid; w < nblk * kBeam; w += NT) {
            const int g = w >> 5;
            int e = w & 31;
            const int top_r = hi_r - 8 * g, bot_r = max(lo_r, top_r - 7);
            for (int r = top_r; r >= bot_r; --r) e = win[(r - lo_r) * kBeam + e] & 31;
            bexit[w] = (unsigned char)e;
        }
        __syncthreads();
        if (tid == 0) {
            for (int g = 0; g < nblk; ++g) {
                bentry[g] = at;
                at = bexit[g * kBeam + at];
            }
        }
        __syncthreads();
        for (int g = tid; g < nblk; g += NT) {
            int e = bentry[g];
            const int top_r = hi_r - 8 * g, bot_r = max(lo_r, top_r - 7);
            for (int r = top_r; r >= bot_r; --r) {
                const unsigned char b = win[(r - lo_r) * kBeam + e];
                path[r] = b;
                e = b & 31;
            }
        }
        __syncthreads();
    }
    if (tid == 0) {
        const int st0 = a.init_kmers[(size_t)chunk * kBeam + at];
#pragma unroll
        for (int i = 0; i < SL; ++i) ext[i] = (unsigned char)((st0 >> (2 * (SL - 1 - i))) & 3);
    }
    __syncthreads();

    // running count of true steps along the path, and the stepped bases in order
    const int seg = (T + NT - 1) / NT;
    const int r_lo = 1 + tid * seg, r_hi = min(T, r_lo + seg - 1);
    int local = 0;
    for (int r = r_lo; r <= r_hi; ++r) local += !((path[r] >> 5) & 1);
    sm.part[tid] = local;
    __syncthreads();
    int run = 0;
    for (int i = 0; i < tid; ++i) run += sm.part[i];
    for (int r = r_lo; r <= r_hi; ++r) {
        const unsigned char b = path[r];
        if (!((b >> 5) & 1)) {
            ext[SL + run] = b >> 6;
            ++run;
        }
        cnt[r] = (unsigned short)run;
    }
    if (tid == 0) cnt[0] = 0;
    __syncthreads();

    // per-timestep quality (src/beam_search.c:441-496)
    const size_t ct = (size_t)chunk * T;
    for (int t = tid; t < T; t += NT) {
        const int r = t + 1;
        const int c = cnt[r];
        int st = 0;
#pragma unroll
        for (int i = 0; i < SL; ++i) st = (st << 2) | ext[c + i];
        const int base = st & 3;
        const float *pr = post_chunk + (size_t)r * NS;
        int nb[8];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            nb[2 * b] = (st >> 2) + MSB * b;
            nb[2 * b + 1] = ((st << 2) & (NS - 1)) + b;
        }
        // all nine posteriors are fetched before any is used: one memory round trip, not nine
        float pv[8];
        float prob = __ldcg(pr + st);
#pragma unroll
        for (int k = 0; k < 8; ++k) pv[k] = __ldcg(pr + nb[k]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            bool fresh = nb[k] != st;
#pragma unroll
            for (int m = 0; m < k; ++m) fresh = fresh && (nb[m] != nb[k]);
            prob = fresh ? __fadd_rn(prob, pv[k]) : prob;
        }
        prob = prob > 1.0f ? 1.0f : (prob < 0.0f ? 0.0f : prob);
        prob = powf(prob, 0.4f);
        const float other = __fdiv_rn(__fsub_rn(1.0f, prob), 3.0f);
        qp[t] = prob;
        *reinterpret_cast<float4 *>(a.qual + (ct + t) * 4) =
            make_float4(base == 0 ? prob : other, base == 1 ? prob : other,
                        base == 2 ? prob : other, base == 3 ? prob : other);
        a.states[ct + t] = base;
        a.moves[ct + t] = (uint8_t)((t == 0) ? 1 : !((path[r] >> 5) & 1));
    }
    __syncthreads();

    // bases and quality string (src/beam_search.c:49-99).  Position of timestep t =
    // (number of moves up to and including t) - 1; move 0 is forced.
    const int forced = (T > 0 && ((path[1] >> 5) & 1)) ? 1 : 0;
    const int seq_len = T > 0 ? cnt[T] + forced : 0;
    for (int t = tid; t < T; t += NT) {
        const bool starts = (t == 0) || !((path[t + 1] >> 5) & 1);
        if (!starts) continue;
        const int pos = cnt[t + 1] + forced - 1;
        const int b_emit = path[t + 1] >> 6;
        float bsum = 0.f, tsum = 0.f;
        for (int u = t; u < T; ++u) {
            if (u > t && !((path[u + 1] >> 5) & 1)) break;
            const int b = path[u + 1] >> 6;
            const float pq = qp[u];
            const float other = __fdiv_rn(__fsub_rn(1.0f, pq), 3.0f);
            bsum = __fadd_rn(bsum, pq);
#pragma unroll
            for (int k = 0; k < 4; ++k) tsum = __fadd_rn(tsum, k == b ? pq : other);
        }
        float v = __fsub_rn(1.0f, __fdiv_rn(bsum, tsum));
        v = __fmul_rn(-10.0f, log10f(v));
        float qs = __fadd_rn(__fmul_rn(v, a.q_scale), a.q_shift);
        if (qs > 50.0f) qs = 50.0f;
        if (qs < 1.0f) qs = 1.0f;
        a.base_probs[ct + pos] = v;
        a.total_probs[ct + pos] = tsum;
        a.sequence[ct + pos] = "ACGT"[b_emit];
        a.qstring[ct + pos] = (char)(33.5f + qs);
    }
    for (int i = seq_len + tid; i < T; i += NT) {
        a.sequence[ct + i] = 0;
        a.qstring[ct + i] = 0;
        a.base_probs[ct + i] = 0.f;
        a.total_probs[ct + i] = 0.f;
    }
}

template <int NS>
cudaError_t launch_post(const OfDecodeArgs &a, cudaStream_t stream) {
    using Smem = PostSmem<NS>;
    const int Tp = (a.T + 16) & ~15;
    const size_t tail = (size_t)kWin * kBeam + (kWin / 8) * (kBeam + 4) + 8 * (size_t)Tp + 64;
    const size_t bytes = sizeof(Smem) + tail + 128;
    if (bytes > 227 * 1024) return cudaErrorInvalidValue;
    auto kern = posterior_seq_kernel<NS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    kern<<<a.N, kPostThreads, bytes, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

cudaError_t of_launch_posterior_seq(const OfDecodeArgs &a, cudaStream_t stream) {
    switch (a.state_len) {
        case 3: return launch_post<64>(a, stream);
        case 4: return launch_post<256>(a, stream);
        case 5: return launch_post<1024>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}
