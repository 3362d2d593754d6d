// scan.cu -- backward and forward scans (and the posterior) of the CRF-CTC decode for sm_100a.
//
// Replaces the reference kernel bwd_scan (src/scan_cuda.cu:8-57) and the recursion half of
// fwd_post_scan (src/scan_cuda.cu:59-146), and reproduces the CPU routines backward_scan and
// forward_scan (src/decode_cpu.c:13-52, 54-119) bit for bit (see exact_math.cuh):
//   bwd[n][T][s] = 0,  bwd[n][t][s]   = LSE5( bwd[n][t+1][s] + stay, bwd[n][t+1][4j+b] + score[t][n][4(4j+b) + k] )
//                                       for s = j + k*ns/4
//   fwd[n][0][s] = 0,  fwd[n][t+1][s] = LSE5( fwd[n][t][s] + stay,   fwd[n][t][j + b*ns/4] + score[t][n][4s + b] )
//                                       for s = 4j + k                         (b = 0..3 in both)
// The two recursions do not depend on each other (only the posterior needs both).  The launcher
// takes either or both; the decode runs the backward scan first (the beam search waits for it)
// and the forward scan beside the beam search, which leaves most issue slots free.  For the 256-
// and 1024-state models the forward scan also forms the posterior (a warp of its own per block,
// see PosteriorRow) and its scores never leave the chip; for the 64-state model they go to HBM for
// the kernel that forms the posterior.
//
// Shape of a block.  In either direction the four states that share j also share their four
// neighbour inputs, and their 16 transition scores are one contiguous 32-byte piece of the score
// row, so nothing is strided.  SPT of those four states go to one thread.  The previous row
// lives in shared memory (one block barrier per timestep); score rows arrive through a ring of
// 1-D bulk asynchronous copies tracked by mbarriers (no multicast), issued a ring length ahead
// by a copy warp of their own.  Output rows go straight to HBM.
//
// Neither scan is bound by HBM (each moves T*4ns*2 + (T+1)*ns*4 bytes per chunk); they are bound
// by the latency of one timestep's dependent arithmetic.
#include "scan.cuh"
#include "exact_math.cuh"
#include "fast_lse.cuh"
#include "of_device.cuh"

namespace {

constexpr int kExpCopies = 16;  // per-half-warp-lane copies of the 2^(j/64) table

// One fp16 out of a 32-bit word, widened.  Going through __half2 lets the conversion pick its
// half of the register directly instead of shifting it out first.
__device__ __forceinline__ float half_of(uint32_t word, int odd) {
    const __half2 h = *reinterpret_cast<const __half2 *>(&word);
    return odd ? __high2float(h) : __low2float(h);
}

// ------------------------------------------------------------------------------------------
// The two recursions differ only in which states a thread owns, which inputs they share, where
// their scores sit inside the 32-byte piece, and in the direction of time.

template <int NS>
struct BwdTopo {
    static constexpr int NJ = NS / 4;
    static constexpr bool kForward = false;
    // thread (j, slot k) owns state j + k*NJ; the four slots share the successors 4j..4j+3
    __device__ static int state(int j, int k) { return j + k * NJ; }
    __device__ static void shared_inputs(const float *in, int j, float (&x)[4]) {
        const float4 v = *reinterpret_cast<const float4 *>(in + 4 * j);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
    // score of (slot k, base b) is half number 4b + k of the piece
    __device__ static int half_index(int k, int b) { return 4 * b + k; }
    // the same out of the piece held as eight words, slot k0 + k with k0 (a multiple of SPT)
    // known only at run time: selects instead of strided shared-memory reads
    template <int SPT>
    __device__ static float score(const uint32_t (&w)[8], int k0, int k, int b) {
        if (SPT == 4) return half_of(w[2 * b + (k >> 1)], k & 1);
        const uint32_t x = (k0 & 2) ? w[2 * b + 1] : w[2 * b];
        return SPT == 2 ? half_of(x, k) : half_of(x, k0 & 1);
    }
    __device__ static int j_of(int s) { return s % NJ; }
    __device__ static int k_of(int s) { return s / NJ; }
    // the states of the next row to be computed that read state s of this row, d = 0..3
    __device__ static int reader(int s, int d) { return (s >> 2) + d * NJ; }
    // time: step i reads score row T-1-i and produces output row T-1-i; row T is the zero row
    __device__ static int score_row(int i, int T) { return T - 1 - i; }
    __device__ static int out_row(int i, int T) { return T - 1 - i; }
    __device__ static int zero_row(int T) { return T; }
};

template <int NS>
struct FwdTopo {
    static constexpr int NJ = NS / 4;
    static constexpr bool kForward = true;
    // thread (j, slot k) owns state 4j + k; the four slots share the predecessors j + b*NJ
    __device__ static int state(int j, int k) { return 4 * j + k; }
    __device__ static void shared_inputs(const float *in, int j, float (&x)[4]) {
#pragma unroll
        for (int b = 0; b < 4; ++b) x[b] = in[j + b * NJ];
    }
    __device__ static int half_index(int k, int b) { return 4 * k + b; }
    template <int SPT>
    __device__ static float score(const uint32_t (&w)[8], int k0, int k, int b) {
        const int c = b >> 1;
        if (SPT == 4) return half_of(w[2 * k + c], b & 1);
        if (SPT == 2) return half_of(k0 ? w[4 + 2 * k + c] : w[2 * k + c], b & 1);
        const uint32_t x = (k0 & 2) ? ((k0 & 1) ? w[6 + c] : w[4 + c]) : ((k0 & 1) ? w[2 + c] : w[c]);
        return half_of(x, b & 1);
    }
    __device__ static int j_of(int s) { return s >> 2; }
    __device__ static int k_of(int s) { return s & 3; }
    __device__ static int reader(int s, int d) { return 4 * (s % NJ) + d; }
    __device__ static int score_row(int i, int) { return i; }
    __device__ static int out_row(int i, int) { return i + 1; }
    __device__ static int zero_row(int) { return 0; }
};

// The five terms of state s: inputs from row `in`, scores from the chunk's score row `row`.
template <class Topo>
__device__ __forceinline__ void terms_of(int s, const float *in, const unsigned char *row, float stay,
                                         float (&v)[5]) {
    const int j = Topo::j_of(s), k = Topo::k_of(s);
    const __half *piece = reinterpret_cast<const __half *>(row) + 16 * j;
    float x[4];
    Topo::shared_inputs(in, j, x);
    v[0] = in[s] + stay;
#pragma unroll
    for (int b = 0; b < 4; ++b) v[b + 1] = x[b] + __half2float(piece[Topo::half_index(k, b)]);
}

// Terms of the SPT states (j, k0 .. k0+SPT-1) of one thread.  The 32-byte piece is read as two
// 16-byte halves (a two-way bank conflict, which costs less than the selects that avoid it: the
// kernel is short of issue slots, not of shared-memory bandwidth).
// `own`, when given, holds the thread's own states of row `in` (what it computed a timestep ago),
// which saves reading them back.
template <class Topo, int SPT>
__device__ __forceinline__ void thread_terms(const float *in, const unsigned char *row, int j, int k0,
                                             float stay, float (&v)[SPT][5], const float *own = nullptr) {
    const unsigned char *piece = row + 32 * j;
    const uint4 lo = *reinterpret_cast<const uint4 *>(piece);
    const uint4 hi = *reinterpret_cast<const uint4 *>(piece + 16);
    float x[4];
    Topo::shared_inputs(in, j, x);
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        v[k][0] = (own ? own[k] : in[Topo::state(j, k0 + k)]) + stay;
#pragma unroll
        for (int b = 0; b < 4; ++b) v[k][b + 1] = x[b] + Topo::template score<SPT>(w, k0, k, b);
    }
}

template <class Topo, int SPT>
__device__ __forceinline__ void thread_store(float *smem_row, float *gmem_row, int j, int k0,
                                             const float (&res)[SPT], bool to_gmem) {
    if constexpr (Topo::kForward && SPT == 4) {
        const float4 v = make_float4(res[0], res[1], res[2], res[3]);
        *reinterpret_cast<float4 *>(smem_row + 4 * j) = v;
        if (to_gmem) *reinterpret_cast<float4 *>(gmem_row + 4 * j) = v;
    } else if constexpr (Topo::kForward && SPT == 2) {
        const float2 v = make_float2(res[0], res[1]);
        *reinterpret_cast<float2 *>(smem_row + 4 * j + k0) = v;
        if (to_gmem) *reinterpret_cast<float2 *>(gmem_row + 4 * j + k0) = v;
    } else {
#pragma unroll
        for (int k = 0; k < SPT; ++k) {
            smem_row[Topo::state(j, k0 + k)] = res[k];
            if (to_gmem) gmem_row[Topo::state(j, k0 + k)] = res[k];
        }
    }
}

// ------------------------------------------------------------------------------------------
// One row of the posterior, softmax_s(fwd[s] + bwd[s]), by one warp: the forward row comes from
// shared memory and so does the backward row (it arrives beside the score row of the timestep
// during which it is needed; a load from HBM issued by this warp would put a microsecond of
// latency into every timestep, which is more than the scan warps take).  Lane l
// takes the states (q*32 + l)*VEC .. +VEC-1; the arithmetic and its order are those of the
// stand-alone posterior loop in posterior_seq.cu (softmax offset m0 = the maximum of row 0, where
// fwd is zero: the log partition function is the same for every row, so exponents stay in range).
template <int NS>
struct PosteriorRow {
    static constexpr int PERL = NS / 32;
    static constexpr int VEC = PERL >= 4 ? 4 : PERL;
    static constexpr int NV = PERL / VEC;

    __device__ static float row_max(const float *row, int lane) {
        float m = -3.0e38f;
        for (int st = lane; st < NS; st += 32) m = fmaxf(m, row[st]);
        return ofd::warp_max(m);
    }
    __device__ static void load(float *d, const float *p) {
        if constexpr (VEC == 4) {
            const float4 v = *reinterpret_cast<const float4 *>(p);
            d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
        } else if constexpr (VEC == 2) {
            const float2 v = *reinterpret_cast<const float2 *>(p);
            d[0] = v.x; d[1] = v.y;
        } else {
            d[0] = *p;
        }
    }
    __device__ static void emit(const float *fwd_row, const float *bwd_row, float *post_row, float m0, int lane) {
        const float kLog2e = 1.4426950408889634f;
        float e[PERL];
        float part = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) {
            float f[VEC], b[VEC];
            load(f, fwd_row + (q * 32 + lane) * VEC);
            load(b, bwd_row + (q * 32 + lane) * VEC);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                e[q * VEC + k] = ofd::ex2_approx(((f[k] + b[k]) - m0) * kLog2e);
                part += e[q * VEC + k];
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        const float inv = 1.0f / part;
#pragma unroll
        for (int q = 0; q < NV; ++q) {
            float *p = post_row + (q * 32 + lane) * VEC;
            const float *x = e + q * VEC;
            if constexpr (VEC == 4)
                *reinterpret_cast<float4 *>(p) = make_float4(x[0] * inv, x[1] * inv, x[2] * inv, x[3] * inv);
            else if constexpr (VEC == 2)
                *reinterpret_cast<float2 *>(p) = make_float2(x[0] * inv, x[1] * inv);
            else
                *p = x[0] * inv;
        }
    }
};

// ------------------------------------------------------------------------------------------
// The scan of one chunk by one block.
//
// If a state whose rounding the fp32 evaluation cannot certify sent its warp through the
// value-exact routine before the timestep could end, that routine's latency would be paid on
// nearly every step: almost every timestep has a few such states.  Here the scan warps do not
// wait for it.  An uncertified state gets the likelier of its two candidate floats and is put on
// a list, together with its five terms; while the scan warps work on the next timestep, a
// checker warp recomputes the listed states exactly.  If every guess was right (most timesteps)
// nothing else happens.  If one was wrong the block pauses at the end of that next
// timestep: the checker corrects the value and recomputes exactly the five states of the next
// row that read it (the state itself and its four readers) before anybody reads those, and the
// scan carries on.  (Letting the scan run on and chasing the consequences a step behind does
// not work: a one-ulp change of an input moves an output by one ulp with a probability equal to
// that input's weight in the sum, and the weights of a state over its five readers add up to
// about one, so corrections would breed as fast as they die.)  What reaches HBM is, value for
// value, what the exact routine alone would have produced.  Three row buffers rotate so that the
// inputs of a timestep are still there while it is being checked, and score rows are released
// one timestep late.
template <int NS, int SPT, int RING, bool POST>
struct SpecSmem {
    static constexpr int kRowBytes = NS * 4 * 2;
    static constexpr int NW = NS / SPT / 32;  // scan warps
    static constexpr int kPerWarp = 16;       // listed states per warp and timestep, at most
    alignas(128) unsigned char ring[RING][kRowBytes];
    // with the posterior: the backward row that the posterior warp needs during a timestep
    // travels with that timestep's score row (same slot, same mbarrier)
    alignas(128) float bwd_ring[POST ? RING : 1][POST ? NS : 4];
    alignas(16) float alpha[3][NS];
    alignas(16) double exp2_rep[ofx::kExpTab * kExpCopies];
    double rcp_c[ofx::kLogTab];
    double log_c[ofx::kLogTab];
    alignas(8) uint64_t full[RING];
    // A listed state is handed to the checker with all it needs: its five terms, the guess and
    // the state's number (32 bytes), so that the checker's chain starts with one round trip to
    // shared memory instead of three dependent ones (list, then state, then the state's inputs).
    alignas(16) float4 listed[2][NW][kPerWarp][2];  // {v0 v1 v2 v3} {v4 guess state -}
    int n_listed[2][NW];
    unsigned short wrong_state[NW * kPerWarp];
    float wrong_value[NW * kPerWarp];
    // settle-now path: a warp's uncertified states, dealt out to its lanes, and their exact values
    unsigned short redo_state[NW][32 * SPT];
    float redo_value[NW][32 * SPT];
    int abort_flag;
};

// The scan warps' route for a timestep with more uncertified states than the usual one handles;
// out of line on purpose.  v: the thread's terms, res: its guesses (in) and, where states were
// settled, their exact values (out); bit k of okmask: state k was certified.  Returns the number of
// states the warp put on the list, or -1 if it settled its uncertified states here (res changed).
template <class Topo, int NS, int SPT, int RING, bool POST>
__device__ __noinline__ int crowded_step(SpecSmem<NS, SPT, RING, POST> &sm, const float (*v)[5], float *res, uint32_t okmask,
                                         int par, int j, int k0, const float *in, const unsigned char *row,
                                         float stay, const ofx::TabRef tr) {
    constexpr int PER = SpecSmem<NS, SPT, RING, POST>::kPerWarp;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lt_mask = (1u << lane) - 1u;
    uint32_t bad[SPT];
    int total = 0;
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        bad[k] = __ballot_sync(0xffffffffu, !((okmask >> k) & 1u));
        total += __popc(bad[k]);
    }
    if (total > 16 * SPT) {
        // most states uncertified (the first few dozen timesteps, where scores are small and
        // the float grid fine): the exact routine for every state
        float out[SPT];
        ofx::lse5_batch_exact<SPT>(v, out, tr);
#pragma unroll
        for (int k = 0; k < SPT; ++k) res[k] = out[k];
        return -1;
    }
    if (total > PER) {
        // many uncertified states (the next hundred or two timesteps): settle them here and
        // now, nothing to check later.  They are dealt out evenly to the warp's lanes, so the
        // exact routine runs ceil(total / 32) times rather than once per state of the
        // unluckiest lane.
        int pos[SPT], base = 0;
#pragma unroll
        for (int k = 0; k < SPT; ++k) {
            pos[k] = base + __popc(bad[k] & lt_mask);
            if (!((okmask >> k) & 1u)) sm.redo_state[warp][pos[k]] = (unsigned short)Topo::state(j, k0 + k);
            base += __popc(bad[k]);
        }
        __syncwarp();
        for (int first = 0; first < total; first += 32) {
            const int e = first + lane;
            const int st = sm.redo_state[warp][e < total ? e : 0];
            float w[5];
            terms_of<Topo>(st, in, row, stay, w);
            const float x = ofx::lse5_exact(w, tr, e < total);
            if (e < total) sm.redo_value[warp][e] = x;
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < SPT; ++k)
            if (!((okmask >> k) & 1u)) res[k] = sm.redo_value[warp][pos[k]];
        return -1;
    }
    int base = 0;
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
        if (!((okmask >> k) & 1u)) {
            float4 *entry = sm.listed[par][warp][base + __popc(bad[k] & lt_mask)];
            entry[0] = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
            entry[1] = make_float4(v[k][4], res[k], __int_as_float(Topo::state(j, k0 + k)), 0.f);
        }
        base += __popc(bad[k]);
    }
    return total;
}

//
// POST (forward direction only): the rows are not written out; a fourth kind of warp turns each
// row, once it is final, into the posterior row  softmax_s(fwd[t][s] + bwd[t][s])  and writes
// that (`out` is then the posterior tensor and `bwd_in` the finished backward scores).  Row r is
// final after the barrier that ends timestep r (its guesses have been checked by then) and its
// buffer is written again during timestep r+2, so the posterior warp takes it during timestep
// r+1; the last two rows are taken after the scan.  The arithmetic is that of the stand-alone
// posterior loop in posterior_seq.cu, operation for operation.
template <class Topo, int NS, int SPT, int RING, bool POST>
__device__ __forceinline__ void spec_body(unsigned char *smem_raw, int chunk, const __half *scores,
                                          float *out, const float *bwd_in, int T, int N, float stay,
                                          const ofx::Tables *tables, int *status, uint64_t wait_ns) {
    constexpr int NJ = NS / 4;
    constexpr int TPC = NS / SPT;
    using Smem = SpecSmem<NS, SPT, RING, POST>;
    constexpr int NW = Smem::NW, PER = Smem::kPerWarp;
    static_assert(!POST || Topo::kForward, "the posterior rides on the forward scan");
    static_assert(TPC % 32 == 0, "scan warps must be full");
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
        for (int r = 0; r < RING; ++r) ofd::mbar_init(&sm.full[r], 1);
        ofd::mbar_fence_init();
    }
    __syncthreads();

    const size_t t_stride = (size_t)N * NS * 4;
    const __half *chunk_scores = scores + (size_t)chunk * NS * 4;
    float *out_chunk = out + (size_t)chunk * (size_t)(T + 1) * NS;
    const ofx::TabRef tr = {sm.exp2_rep + (tid & (kExpCopies - 1)), kExpCopies, sm.rcp_c, sm.log_c};

    if (warp == NW) {
        // ------------------------------------------------------------------ copy warp
        // A slot is refilled one timestep late: the checker still reads the scores of the
        // timestep it is checking.
        const bool issuer = lane == 0;
        int issued = 0;  // copies go out in row order; after an abort no more are issued
        auto fill = [&](int i) {
            if (sm.abort_flag) return;
            const int slot = i % RING;
            ofd::mbar_arrive_expect_tx(&sm.full[slot], Smem::kRowBytes + (POST ? NS * 4 : 0));
            ofd::bulk_g2s(sm.ring[slot], chunk_scores + t_stride * (size_t)Topo::score_row(i, T), Smem::kRowBytes,
                          &sm.full[slot]);
            // the posterior row formed during timestep i is row i-1 (row 0 during timestep 0)
            if (POST)
                ofd::bulk_g2s(sm.bwd_ring[slot], bwd_in + ((size_t)chunk * (size_t)(T + 1) + (size_t)(i ? i - 1 : 0)) * NS,
                              NS * 4, &sm.full[slot]);
            ++issued;
        };
        auto landed = [&](int i) {
            ofd::mbar_wait_bounded(&sm.full[i % RING], (uint32_t)(i / RING) & 1u, &sm.abort_flag, status, wait_ns);
        };
        if (issuer) {
            for (int i = 0; i < RING && i < T; ++i) fill(i);
            if (T > 0) landed(0);
        }
        __syncthreads();
        for (int i = 0; i < T; ++i) {
            if (issuer && i + 1 < T) landed(i + 1);
            if (__syncthreads_or(0)) __syncthreads();
            if (issuer && i >= 1 && i - 1 + RING < T) fill(i - 1 + RING);
        }
        if (POST) __syncthreads();  // the last row is final
        // after an abort the newest copies get a bounded chance to land before the block retires
        if (issuer && sm.abort_flag) ofd::mbar_drain_bounded(sm.full, RING, issued, wait_ns);
        return;
    }

    if (POST && warp == NW + 2) {
        // ------------------------------------------------------------------ posterior warp
        const float *bwd_chunk = bwd_in + (size_t)chunk * (size_t)(T + 1) * NS;
        const float m0 = PosteriorRow<NS>::row_max(bwd_chunk, lane);
        // inside the scan the backward row is in the slot of the timestep during which the
        // posterior row is formed; the last two rows take theirs from HBM
        auto emit = [&](int r, const float *bwd_row) {
            PosteriorRow<NS>::emit(sm.alpha[r % 3], bwd_row, out_chunk + (size_t)r * NS, m0, lane);
        };
        __syncthreads();  // start of the scan
        int next_row = 0;
        for (int i = 0; i < T; ++i) {
            // during timestep i the rows up to i-1 are final (and row 0 always is)
            if (next_row == 0 || next_row <= i - 1) {
                emit(next_row, sm.bwd_ring[i % RING]);  // next_row = i-1, or 0 when i = 0
                ++next_row;
            }
            if (__syncthreads_or(0)) __syncthreads();
        }
        while (next_row <= T - 1) {  // final since the last timestep's barrier
            emit(next_row, bwd_chunk + (size_t)next_row * NS);
            ++next_row;
        }
        __syncthreads();  // the last row is final
        emit(T, bwd_chunk + (size_t)T * NS);
        return;
    }

    if (warp == NW + 1) {
        // ------------------------------------------------------------------ checker warp
        __syncthreads();  // start of the scan
        for (int i = 0; i <= T; ++i) {
            // During timestep i (for i = T: after the last one) check the states listed during
            // timestep i-1; their terms and guesses come with the list, the guesses also stand in
            // alpha[i%3] and in the output row of timestep i-1.
            int nw = 0;
            if (i >= 1) {
                const int par = (i - 1) & 1;
                // An entry was written before the correction that ended its timestep, if there
                // was one: a state that read a corrected value stands on the list with the terms
                // from before.  The correction has recomputed every such state for good, so a
                // mismatch counts only if the entry's terms are still the state's terms.
                auto still_stands = [&](bool differs, const float (&v)[5], int s) {
                    if (__any_sync(0xffffffffu, differs)) {  // one timestep in seventeen
                        float now[5];
                        terms_of<Topo>(differs ? s : 0, sm.alpha[(i - 1) % 3], sm.ring[(i - 1) % RING], stay, now);
#pragma unroll
                        for (int q = 0; q < 5; ++q) differs = differs && __float_as_uint(now[q]) == __float_as_uint(v[q]);
                    }
                    return differs;
                };
                if (NW * PER <= 32) {
                    // a lane per slot: nothing to look up before the entry can be fetched
                    const int w = lane / PER, k = lane % PER;
                    const float4 a = sm.listed[par][w < NW ? w : 0][k][0], b = sm.listed[par][w < NW ? w : 0][k][1];
                    const bool mine = w < NW && k < sm.n_listed[par][w < NW ? w : 0];
                    if (__any_sync(0xffffffffu, mine)) {
                        const float v[5] = {a.x, a.y, a.z, a.w, b.x};
                        const float x = ofx::lse5_exact(v, tr, mine);
                        const bool wrong = still_stands(mine && __float_as_uint(x) != __float_as_uint(b.y), v, __float_as_int(b.z));
                        const uint32_t wm = __ballot_sync(0xffffffffu, wrong);
                        if (wrong) {
                            const int at = __popc(wm & ((1u << lane) - 1u));
                            sm.wrong_state[at] = (unsigned short)__float_as_int(b.z);
                            sm.wrong_value[at] = x;
                        }
                        nw = __popc(wm);
                    }
                } else {
                    // more slots than lanes: the filled ones are taken 32 at a time
                    int cnt[NW], total = 0;
#pragma unroll
                    for (int w = 0; w < NW; ++w) {
                        cnt[w] = sm.n_listed[par][w];
                        total += cnt[w];
                    }
                    for (int base = 0; base < total; base += 32) {
                        const int e = base + lane;
                        int at_w = 0, at_k = 0, acc = 0;
#pragma unroll
                        for (int w = 0; w < NW; ++w) {
                            if (e >= acc && e < acc + cnt[w]) {
                                at_w = w;
                                at_k = e - acc;
                            }
                            acc += cnt[w];
                        }
                        const float4 a = sm.listed[par][at_w][at_k][0], b = sm.listed[par][at_w][at_k][1];
                        const float v[5] = {a.x, a.y, a.z, a.w, b.x};
                        const float x = ofx::lse5_exact(v, tr, e < total);
                        const bool wrong = still_stands(e < total && __float_as_uint(x) != __float_as_uint(b.y), v, __float_as_int(b.z));
                        const uint32_t wm = __ballot_sync(0xffffffffu, wrong);
                        if (wrong) {
                            const int at = nw + __popc(wm & ((1u << lane) - 1u));
                            sm.wrong_state[at] = (unsigned short)__float_as_int(b.z);
                            sm.wrong_value[at] = x;
                        }
                        nw += __popc(wm);
                    }
                }
                __syncwarp();
            }
            if (i == T) {
                // the last row: no timestep reads it any more, just correct it
                if (POST) {
                    for (int e = lane; e < nw; e += 32) sm.alpha[T % 3][sm.wrong_state[e]] = sm.wrong_value[e];
                    __syncthreads();  // the last row is final
                } else {
                    float *row = out_chunk + (size_t)Topo::out_row(T - 1, T) * NS;
                    for (int e = lane; e < nw; e += 32) row[sm.wrong_state[e]] = sm.wrong_value[e];
                }
                break;
            }
            // end of timestep i; the barrier itself tells every warp whether a guess was wrong
            __syncthreads_or(nw);
            if (nw) {
                float *prev_row = out_chunk + (size_t)Topo::out_row(i - 1, T) * NS;
                for (int e = lane; e < nw; e += 32) {
                    const int s = sm.wrong_state[e];
                    sm.alpha[i % 3][s] = sm.wrong_value[e];
                    if (!POST) prev_row[s] = sm.wrong_value[e];
                }
                __syncwarp();
                // the five states of timestep i's row that read a corrected value
                float *this_row = out_chunk + (size_t)Topo::out_row(i, T) * NS;
                for (int idx = lane; idx < 5 * nw; idx += 32) {
                    const int s = sm.wrong_state[idx / 5], d = idx % 5;
                    const int dep = d == 4 ? s : Topo::reader(s, d);
                    float v[5];
                    terms_of<Topo>(dep, sm.alpha[i % 3], sm.ring[i % RING], stay, v);
                    float x;  // certified fp32 evaluation first: it settles all but about 1 in 100
                    if (!ofd::lse5_try_fast(v, x)) x = ofx::lse5_exact(v, tr, idx < 5 * nw);
                    sm.alpha[(i + 1) % 3][dep] = x;
                    if (!POST) this_row[dep] = x;
                }
                __syncthreads();  // corrections in place
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- scan warps
    const int j = tid % NJ;
    const int k0 = (tid / NJ) * SPT;
    if (!POST) {
#pragma unroll
        for (int k = 0; k < SPT; ++k) out_chunk[(size_t)Topo::zero_row(T) * NS + Topo::state(j, k0 + k)] = 0.f;
    }
    __syncthreads();
    const uint32_t lt_mask = (1u << lane) - 1u;
    float res[SPT];  // the thread's states of the current row: its stay terms for the next timestep
#pragma unroll
    for (int k = 0; k < SPT; ++k) res[k] = 0.f;
    // rotating pointers instead of i % 3 and i % RING: row i is read from `in`, row i+1 goes to `nxt`
    const float *in = sm.alpha[0];
    float *nxt = sm.alpha[1], *spare = sm.alpha[2];
    const unsigned char *row = sm.ring[0];
    float *gmem_out = out_chunk + (size_t)Topo::out_row(0, T) * NS;
    const ptrdiff_t gmem_step = Topo::kForward ? (ptrdiff_t)NS : -(ptrdiff_t)NS;
    for (int i = 0; i < T; ++i) {
        float v[SPT][5];
        bool ok[SPT];
        thread_terms<Topo, SPT>(in, row, j, k0, stay, v, res);
        ofd::lse5_fast_guess<SPT>(v, res, ok);
        // out they go at once (certified values and guesses alike), so that the stores issue in the
        // shadow of the vote below; the two routes that settle states here and now store again
        thread_store<Topo, SPT>(nxt, gmem_out, j, k0, res, !POST);
        int total = 0, mine = 0;
#pragma unroll
        for (int k = 0; k < SPT; ++k) mine += !ok[k];
        // Both votes are taken here, where the warp is converged for certain, and nothing below
        // votes or diverges on the usual route: a vote or a lane-divergent branch inside
        // conditional code costs a hundred cycles and more of re-convergence.
        const uint32_t owners = __ballot_sync(0xffffffffu, mine != 0);  // non-zero about every other timestep per warp
        const uint32_t crowded = __ballot_sync(0xffffffffu, mine > 1);
        // The usual case: a few lanes with one uncertified state each.  The first vote settles who
        // lists where, and the entry goes out through predicated stores.
        const bool few = owners != 0 && crowded == 0 && __popc(owners) <= PER;
        if (few) {
            const uint32_t entry = (uint32_t)__cvta_generic_to_shared(sm.listed[i & 1][warp][__popc(owners & lt_mask)]);
#pragma unroll
            for (int k = 0; k < SPT; ++k)
                ofd::sts_entry_if(!ok[k], entry, v[k], res[k], __int_as_float(Topo::state(j, k0 + k)));
            total = __popc(owners);
        } else if (owners) {
            // anything else (a lane with two uncertified states, more than a list takes, the first
            // few hundred timesteps where most states are uncertified) goes out of line: the
            // loop's instructions stay few and close together.  The copies live in local memory,
            // the arrays of the usual route in registers.
            float cv[SPT][5], cres[SPT];
            uint32_t okmask = 0;
#pragma unroll
            for (int k = 0; k < SPT; ++k) {
#pragma unroll
                for (int q = 0; q < 5; ++q) cv[k][q] = v[k][q];
                cres[k] = res[k];
                okmask |= (uint32_t)ok[k] << k;
            }
            total = crowded_step<Topo, NS, SPT, RING, POST>(sm, cv, cres, okmask, i & 1, j, k0, in, row, stay, tr);
#pragma unroll
            for (int k = 0; k < SPT; ++k) res[k] = cres[k];
            if (total < 0) {  // states were settled here and now: their values replace the guesses
                thread_store<Topo, SPT>(nxt, gmem_out, j, k0, res, !POST);
                total = 0;
            }
        }
        if (lane == 0) sm.n_listed[i & 1][warp] = total;
        if (__syncthreads_or(0)) {
            __syncthreads();  // the checker is correcting this row's readers
#pragma unroll
            for (int k = 0; k < SPT; ++k) res[k] = nxt[Topo::state(j, k0 + k)];  // maybe corrected
        }
        float *const was_in = const_cast<float *>(in);
        in = nxt;
        nxt = spare;
        spare = was_in;
        row = (row == sm.ring[RING - 1]) ? sm.ring[0] : row + Smem::kRowBytes;
        gmem_out += gmem_step;
    }
    if (POST) __syncthreads();  // the last row is final
}

// ------------------------------------------------------------------------------------------
// One grid for either or both directions: the first n_bwd_blocks blocks scan backwards, the
// rest forwards.

template <int NS, int SPT, int RING>
__global__ void __launch_bounds__(NS / SPT + 64, (NS <= 64 ? 8 : NS <= 256 ? 4 : 2))
scan_spec_kernel(const __half *__restrict__ scores, float *__restrict__ bwd, float *__restrict__ fwd,
                 int T, int N, int n_bwd_blocks, float stay, const ofx::Tables *__restrict__ tables,
                 int *status, uint64_t wait_ns) {
    extern __shared__ unsigned char smem_raw[];
    if ((int)blockIdx.x < n_bwd_blocks)
        spec_body<BwdTopo<NS>, NS, SPT, RING, false>(smem_raw, blockIdx.x, scores, bwd, nullptr, T, N, stay, tables,
                                                     status, wait_ns);
    else
        spec_body<FwdTopo<NS>, NS, SPT, RING, false>(smem_raw, blockIdx.x - n_bwd_blocks, scores, fwd, nullptr, T, N,
                                                     stay, tables, status, wait_ns);
}

// Forward scan with the posterior on top: one block per chunk, reads the finished backward scores.
template <int NS, int SPT, int RING>
__global__ void __launch_bounds__(NS / SPT + 96, (NS <= 256 ? 5 : 2))
scan_spec_posterior_kernel(const __half *__restrict__ scores, const float *__restrict__ bwd,
                           float *__restrict__ post, int T, int N, float stay,
                           const ofx::Tables *__restrict__ tables, int *status, uint64_t wait_ns) {
    extern __shared__ unsigned char smem_raw[];
    spec_body<FwdTopo<NS>, NS, SPT, RING, true>(smem_raw, blockIdx.x, scores, post, bwd, T, N, stay, tables, status, wait_ns);
}

template <int NS, int SPT, int RING>
cudaError_t launch_spec(const __half *scores, float *bwd, float *fwd, int T, int N, float stay,
                        const ofx::Tables *tables, int *status, uint64_t wait_ns, cudaStream_t stream) {
    using Smem = SpecSmem<NS, SPT, RING, false>;
    const size_t bytes = sizeof(Smem) + 128;
    auto kern = scan_spec_kernel<NS, SPT, RING>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    const int n_bwd = bwd ? N : 0, n_fwd = fwd ? N : 0;
    kern<<<n_bwd + n_fwd, NS / SPT + 64, bytes, stream>>>(scores, bwd, fwd, T, N, n_bwd, stay, tables, status, wait_ns);
    return cudaGetLastError();
}

template <int NS, int SPT, int RING>
cudaError_t launch_spec_posterior(const __half *scores, const float *bwd, float *post, int T, int N, float stay,
                                  const ofx::Tables *tables, int *status, uint64_t wait_ns, cudaStream_t stream) {
    using Smem = SpecSmem<NS, SPT, RING, true>;
    const size_t bytes = sizeof(Smem) + 128;
    auto kern = scan_spec_posterior_kernel<NS, SPT, RING>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    kern<<<N, NS / SPT + 96, bytes, stream>>>(scores, bwd, post, T, N, stay, tables, status, wait_ns);
    return cudaGetLastError();
}

}  // namespace

// (Not for the 64-state model: a row is too little work there for a warp-wide reduction per
// chunk and timestep to pay; its posterior is done by the stand-alone loop.)
bool of_forward_posterior_fused(int state_len) { return state_len == 4 || state_len == 5; }

cudaError_t of_launch_forward_posterior(const void *scores_fp16, const float *bwd, float *post, int T, int N,
                                        int state_len, float stay, const ofx::Tables *tables, int *status,
                                        uint64_t wait_ns, cudaStream_t stream) {
    const __half *s = static_cast<const __half *>(scores_fp16);
    if (T < 1) return cudaErrorInvalidValue;
    switch (state_len) {
        case 4: return launch_spec_posterior<256, 4, 6>(s, bwd, post, T, N, stay, tables, status, wait_ns, stream);
        case 5: return launch_spec_posterior<1024, 4, 6>(s, bwd, post, T, N, stay, tables, status, wait_ns, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t of_launch_scans(const void *scores_fp16, float *bwd, float *fwd, int T, int N,
                            int state_len, float stay, const ofx::Tables *tables, int *status,
                            uint64_t wait_ns, cudaStream_t stream) {
    const __half *s = static_cast<const __half *>(scores_fp16);
    switch (state_len) {
        case 3: return launch_spec<64, 1, 8>(s, bwd, fwd, T, N, stay, tables, status, wait_ns, stream);
        case 4: return launch_spec<256, 4, 6>(s, bwd, fwd, T, N, stay, tables, status, wait_ns, stream);
        case 5: return launch_spec<1024, 4, 6>(s, bwd, fwd, T, N, stay, tables, status, wait_ns, stream);
        default: return cudaErrorInvalidValue;
    }
}
