// fwd_beam.cu -- posterior, beam search, traceback, per-base quality and sequence/qstring
// generation for one chunk per block, fused in one sm_100a kernel.
//
// Replaces the softmax half of the reference kernel fwd_post_scan (src/scan_cuda.cu:147-199) and
// the kernels beam_search (src/beam_search_cuda.cu:139-528), compute_qual_data (:530-605) and
// generate_sequence (:52-121).  The beam search follows the reference's CPU routine
// beam_search_cpu (src/beam_search.c:117-497) -- including its bisection of the pruning
// threshold, which the reference's CUDA kernel lacks -- because output parity is defined against
// the CPU decoder.  The forward and backward scores come from the scan kernel (scan.cu).
//
// Roles inside a block (one chunk):
//   posterior warps  ns/4 threads, four consecutive states each: posterior = softmax over states
//                of fwd + bwd, row by row (src/decode_cpu.c:115,121-147).  No per-row maximum is
//                needed: the log partition function is the same for every row, so one offset
//                taken from row 0 keeps every exponent in range; the row sum is reduced across
//                warps and applied one timestep late (one named barrier per timestep).
//   beam warp    lane = beam slot (width <= 32).  Everything is warp-synchronous and, where
//                lanes differ, branch free: candidate scores, duplicate-prefix merges (CRC32C
//                hashes; a stay merges with the step whose parent hash equals the stay's hash
//                run backwards through the CRC), maximum, threshold bisection by warp
//                reductions, order-preserving compaction by ballots.  One packed back-pointer
//                byte per slot and timestep goes to HBM (prev slot 5 bits | stay 1 bit | base
//                2 bits).
//   copy warp    one lane issues 1-D bulk asynchronous copies (no multicast) of score row t (for
//                the beam search, timesteps strided by N*C as in src/decode_cpu.c:204,216),
//                backward row t and forward row t into a ring; both consumers release a ring
//                slot through an mbarrier.
// After the last timestep the block walks the back-pointers (staged through shared memory in
// windows), rebuilds the k-mer of every path element from the emitted bases, gathers the
// posterior of each path k-mer and its shifted neighbours, and emits moves, sequence and
// qstring, zero-filling the unused tail of each row.
#include <float.h>

#include "exact_math.cuh"
#include "fast_lse.cuh"
#include "fwd_beam.cuh"
#include "of_device.cuh"

namespace {

constexpr int kBeam = 32;
constexpr int kWin = 256;  // traceback window, timesteps

using ofd::ex2_approx;
constexpr float kLog2e = 1.4426950408889634f;

// Warp maximum of a float through the sm_100a float reduction instruction.
__device__ __forceinline__ float warp_max_f32(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// The reference's two-term fold (src/beam_search.c:43-47): certified fp32 evaluation first (same
// interval argument as fast_lse.cuh: log1p(exp(-d)) in fp32 is within 2^-20.5 of the reference's
// double value; if both ends of that interval round to the same float next to m, that float is
// the reference's), value-exact routine otherwise.
__device__ __forceinline__ float fold2(float x, float y, const ofx::TabRef t) {
    const float d = fabsf(x - y);
    const float m = x > y ? x : y;
    if (!(d < 17.0f)) return m;
    const float e = ofd::ex2_approx(-d * 1.4426950408889634f);
    const float l = ofd::lg2_approx(1.0f + e) * 0.6931471805599453f;
    const float eps = 6.75e-7f;  // 2^-20.5
    const float lo = m + (l - eps), hi = m + (l + eps);
    if (lo == hi && fabsf(lo) < 3.0e38f) return lo;
    return ofx::fold2_exact(x, y, t);
}

// CRC32C over two input bits, table form of src/beam_search.c:103-115:
// crc' = (crc >> 2) ^ tab[(crc ^ bits) & 3], tab = {0, 0x417B1DBC, 0x82F63B78, 0xC38D26C4}.
__device__ __forceinline__ uint32_t crc_tab2(uint32_t x) {
    return ((x & 1u) ? 0x417B1DBCu : 0u) ^ ((x & 2u) ? 0x82F63B78u : 0u);
}
__device__ __forceinline__ uint32_t crc_step2(uint32_t crc, uint32_t bits) {
    return (crc >> 2) ^ crc_tab2((crc ^ bits) & 3u);
}
// The update is a bijection for fixed input bits (the table's top two bits equal its index),
// so the parent hash that would step to `crc` by appending `bits` is unique.
__device__ __forceinline__ uint32_t crc_unstep2(uint32_t crc, uint32_t bits) {
    const uint32_t idx = crc >> 30;
    return ((crc ^ crc_tab2(idx)) << 2) | (idx ^ bits);
}
__device__ __forceinline__ uint32_t crc32c_bits(uint32_t crc, uint32_t v, int n) {
    for (int i = 0; i < n; ++i) {
        const uint32_t b = (v ^ crc) & 1u;
        crc >>= 1;
        if (b) crc ^= 0x82f63b78u;
        v >>= 1;
    }
    return crc;
}

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
template <int NW>
__device__ __forceinline__ float sum_partials(const float *p) {
    float s = 0.f;
    if constexpr (NW % 4 == 0) {
#pragma unroll
        for (int i = 0; i < NW; i += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(p + i);
            s += (v.x + v.y) + (v.z + v.w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < NW; ++i) s += p[i];
    }
    return s;
}

template <int NS, int RING>
struct FusedSmem {
    static constexpr int kScoreRow = NS * 8;  // bytes of one fp16 score row
    static constexpr int kBwdRow = NS * 4;    // bytes of one fp32 backward row
    alignas(16) float psum[2][32];
    float red[32];
    alignas(16) uint4 rec[kBeam];
    alignas(16) float cstep[kBeam * 4];
    alignas(8) uint2 slot[2 * kBeam];  // compaction (+ one spare per lane): {score, parent slot | stay << 5 | base << 6}
    unsigned char owner[8192 + 32];    // (+ one spare per lane) hash -> slot + 1 of the beam element owning it (duplicate detection)
    int init_state[kBeam];
    double exp2_j[ofx::kExpTab];
    double rcp_c[ofx::kLogTab];
    double log_c[ofx::kLogTab];
    alignas(8) uint64_t full[RING];
    alignas(8) uint64_t empty[RING];
    int abort_flag;
    int part[608];  // block-scan partials of the tail phase
    // rings last: the tail phase reuses them (and whatever dynamic shared memory follows)
    alignas(128) unsigned char score_ring[RING][kScoreRow];
    alignas(128) unsigned char bwd_ring[RING][kBwdRow];
    alignas(128) unsigned char fwd_ring[RING][kBwdRow];
};

struct FusedArgs {
    const __half *scores;  // [T][N][C] fp16
    const float *bwd;      // [N][T+1][ns]
    const float *fwd;      // [N][T+1][ns]
    float *post;           // [N][T+1][ns]
    unsigned char *bp;     // [N][T+1][32] packed back-pointers
    uint8_t *moves;        // [N][T]
    char *sequence;        // [N][T]
    char *qstring;         // [N][T]
    int *states;           // [N][T]   base of each path element
    float *qual;           // [N][T][4]
    float *base_probs;     // [N][T]
    float *total_probs;    // [N][T]
    const ofx::Tables *tables;
    int *status;
    int T, N, C;
    float stay, log_beam_cut, q_shift, q_scale;
};

template <int NS, int RING>
__global__ void __launch_bounds__((NS / 4 < 32 ? 32 : NS / 4) + 64)
fwd_beam_kernel(const FusedArgs a) {
    constexpr int SPT = 4;  // states per posterior thread
    constexpr int BITS = (NS == 64) ? 6 : (NS == 256 ? 8 : 10);
    constexpr int SL = BITS / 2;
    constexpr int MSB = NS / 4;
    constexpr int TPC = NS / SPT;               // posterior threads that own states (SPT each)
    constexpr int TPAD = TPC < 32 ? 32 : TPC;   // scan threads including idle lanes
    constexpr int NFW = TPAD / 32;              // scan warps
    constexpr int NT = TPAD + 64;
    using Smem = FusedSmem<NS, RING>;
    extern __shared__ unsigned char smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int chunk = blockIdx.x;
    const int T = a.T, N = a.N;
    for (int i = tid; i < ofx::kExpTab; i += NT) sm.exp2_j[i] = a.tables->exp2_j[i];
    for (int i = tid; i < ofx::kLogTab; i += NT) {
        sm.rcp_c[i] = a.tables->rcp_c[i];
        sm.log_c[i] = a.tables->log_c[i];
    }
    for (int i = tid; i < 2048 + 8; i += NT) reinterpret_cast<uint32_t *>(sm.owner)[i] = 0;
    for (int i = tid; i < kBeam * 4; i += NT) sm.cstep[i] = __int_as_float(0x7fc00000);  // mailbox: NaN = empty
    if (tid == 0) {
        sm.abort_flag = 0;
        for (int r = 0; r < RING; ++r) {
            ofd::mbar_init(&sm.full[r], 1);
            ofd::mbar_init(&sm.empty[r], 2);
        }
        ofd::mbar_fence_init();
    }
    __syncthreads();

    const float *bwd_chunk = a.bwd + (size_t)chunk * (size_t)(T + 1) * NS;
    float *post_chunk = a.post + (size_t)chunk * (size_t)(T + 1) * NS;
    unsigned char *bp_chunk = a.bp + (size_t)chunk * (size_t)(T + 1) * kBeam;

    if (warp == NFW + 1) {
        // ------------------------------------------------------------------ copy warp
        if (lane == 0) {
            // the beam search strides timesteps by N*C (src/decode_cpu.c:204,216)
            const __half *beam_scores = a.scores + (size_t)chunk * NS * 4;
            const size_t beam_stride = (size_t)N * a.C;
            const float *fwd_chunk = a.fwd + (size_t)chunk * (size_t)(T + 1) * NS;
            for (int t = 0; t <= T; ++t) {
                const int slot = t % RING;
                if (t >= RING)
                    ofd::mbar_wait_bounded(&sm.empty[slot], (uint32_t)(t / RING - 1) & 1u,
                                           &sm.abort_flag, a.status);
                if (sm.abort_flag) break;
                const uint32_t bytes = 2 * Smem::kBwdRow + (t < T ? Smem::kScoreRow : 0);
                ofd::mbar_arrive_expect_tx(&sm.full[slot], bytes);
                ofd::bulk_g2s(sm.bwd_ring[slot], bwd_chunk + (size_t)t * NS, Smem::kBwdRow, &sm.full[slot]);
                ofd::bulk_g2s(sm.fwd_ring[slot], fwd_chunk + (size_t)t * NS, Smem::kBwdRow, &sm.full[slot]);
                if (t < T)
                    ofd::bulk_g2s(sm.score_ring[slot], beam_scores + beam_stride * t, Smem::kScoreRow,
                                  &sm.full[slot]);
            }
        }
    } else if (warp < NFW) {
        // ------------------------------------------------------------------ scan warps
        const int u = tid;
        const bool act = u < TPC;
        const int s0 = u * SPT;  // this thread's states s0 .. s0+SPT-1
        // softmax offset: maximum of fwd+bwd at row 0 (= bwd row 0, fwd is zero there)
        ofd::mbar_wait_bounded(&sm.full[0], 0, &sm.abort_flag, a.status);
        float m0 = -FLT_MAX;
        if (act) {
            float b0[SPT];
            load_floats<SPT>(b0, reinterpret_cast<const float *>(sm.bwd_ring[0]) + s0);
#pragma unroll
            for (int k = 0; k < SPT; ++k) m0 = fmaxf(m0, b0[k]);
        }
        m0 = ofd::warp_max(m0);
        if (lane == 0) sm.red[warp] = m0;
        ofd::named_bar_sync(1, TPAD);
        m0 = sm.red[0];
#pragma unroll
        for (int w = 1; w < NFW; ++w) m0 = fmaxf(m0, sm.red[w]);

        float e_prev[SPT];
#pragma unroll
        for (int k = 0; k < SPT; ++k) e_prev[k] = 0.f;
        for (int t = 0; t <= T; ++t) {
            const int slot = t % RING;
            float e[SPT];
#pragma unroll
            for (int k = 0; k < SPT; ++k) e[k] = 0.f;
            if (act) {
                float fv[SPT], bv[SPT];
                load_floats<SPT>(fv, reinterpret_cast<const float *>(sm.fwd_ring[slot]) + s0);
                load_floats<SPT>(bv, reinterpret_cast<const float *>(sm.bwd_ring[slot]) + s0);
#pragma unroll
                for (int k = 0; k < SPT; ++k) e[k] = ex2_approx(((fv[k] + bv[k]) - m0) * kLog2e);
            }
            float part = 0.f;
#pragma unroll
            for (int k = 0; k < SPT; ++k) part += e[k];
#pragma unroll
            for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (lane == 0) sm.psum[t & 1][warp] = part;
            if (t > 0 && act) {
                const float inv = 1.0f / sum_partials<NFW>(sm.psum[(t - 1) & 1]);
                float o[SPT];
#pragma unroll
                for (int k = 0; k < SPT; ++k) o[k] = e_prev[k] * inv;
                store_floats<SPT>(post_chunk + (size_t)(t - 1) * NS + s0, o);
            }
#pragma unroll
            for (int k = 0; k < SPT; ++k) e_prev[k] = e[k];
            // one thread checks that the next row has landed; the barrier passes that on
            if (tid == 0 && t < T)
                ofd::mbar_wait_bounded(&sm.full[(t + 1) % RING], (uint32_t)((t + 1) / RING) & 1u,
                                       &sm.abort_flag, a.status);
            ofd::named_bar_sync(1, TPAD);
            if (tid == 0) ofd::mbar_arrive(&sm.empty[slot]);
        }
        if (act) {
            const float inv = 1.0f / sum_partials<NFW>(sm.psum[T & 1]);
            float o[SPT];
#pragma unroll
            for (int k = 0; k < SPT; ++k) o[k] = e_prev[k] * inv;
            store_floats<SPT>(post_chunk + (size_t)T * NS + s0, o);
        }
    } else {
        // ------------------------------------------------------------------ beam warp
        const ofx::TabRef tr = {sm.exp2_j, 1, sm.rcp_c, sm.log_c};
        const uint32_t lt_mask = (1u << lane) - 1u;
        ofd::mbar_wait_bounded(&sm.full[0], 0, &sm.abort_flag, a.status);
        // initial beam: first <= 32 states, in state order, reaching the 32nd largest bwd[0]
        // (src/beam_search.c:151-175).  Radix-select the 32nd largest key bit by bit.
        {
            const float *b0 = reinterpret_cast<const float *>(sm.bwd_ring[0]);
            constexpr int PER = NS / 32;
            uint32_t key[PER];
#pragma unroll
            for (int i = 0; i < PER; ++i)
                key[i] = (uint32_t)ofd::float_order_key(b0[lane + 32 * i]) ^ 0x80000000u;
            uint32_t thr = 0;
            for (int bit = 31; bit >= 0; --bit) {
                const uint32_t cand = thr | (1u << bit);
                int c = 0;
#pragma unroll
                for (int i = 0; i < PER; ++i) c += key[i] >= cand;
                c = __reduce_add_sync(0xffffffffu, c);
                if (c >= kBeam) thr = cand;
            }
            int filled = 0;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const bool f = key[i] >= thr;
                const uint32_t bal = __ballot_sync(0xffffffffu, f);
                const int pos = filled + __popc(bal & lt_mask);
                if (f && pos < kBeam) sm.init_state[pos] = lane + 32 * i;
                filled += __popc(bal);
            }
            __syncwarp();
        }
        int state = sm.init_state[lane];
        uint32_t hash = crc32c_bits(0x12345678u, (uint32_t)state, 32);
        float score = 0.f;
        int W = kBeam;
        bp_chunk[lane] = (unsigned char)((state & 3) << 6);

        for (int t = 0; t < T; ++t) {
            const int slot_a = t % RING, slot_b = (t + 1) % RING;
            // row t was confirmed when it served as "next row" one step ago (or before the loop)
            ofd::mbar_wait_bounded(&sm.full[slot_b], (uint32_t)((t + 1) / RING) & 1u, &sm.abort_flag, a.status);
            const __half *srow = reinterpret_cast<const __half *>(sm.score_ring[slot_a]);
            const float *brow = reinterpret_cast<const float *>(sm.bwd_ring[slot_b]);
            const bool act = lane < W;
            const int q = state & (MSB - 1);
            const int top = state >> (BITS - 2);
            const uint32_t b_own = (uint32_t)state & 3u;

            // duplicate-prefix detection (src/beam_search.c:281-316): a stay can only merge with a
            // step whose parent's hash is `need`.  Every element writes its slot number into an
            // 8192-entry owner table indexed by its hash; a stay then finds the one candidate
            // parent by a single look-up and confirms it by comparing the full hash.  If two
            // elements landed on the same table entry the table cannot be trusted for this
            // timestep and the exhaustive comparison below takes over.
            const uint32_t need = crc_unstep2(hash, b_own);
            // idle slots (lane >= W) use a private spare entry so that nothing here branches
            const uint32_t own_at = act ? (hash & 8191u) : 8192u + lane;
            sm.owner[own_at] = (unsigned char)(lane + 1);
            __syncwarp();

            // candidates: 4 steps (state' = 4q + b, column 16q + 4b + top) and the stay
            float c0, c1, c2, c3, c4;
            {
                // idle slots still hold a valid (stale) k-mer: they read like everybody else and
                // their candidates are voided afterwards
                const float4 bw = *reinterpret_cast<const float4 *>(brow + 4 * q);
                const __half *sp = srow + 16 * q + top;
                const float x0 = __half2float(sp[0]), x1 = __half2float(sp[4]);
                const float x2 = __half2float(sp[8]), x3 = __half2float(sp[12]);
                const float bs = brow[state];
                c0 = __fadd_rn(__fadd_rn(score, x0), bw.x);
                c1 = __fadd_rn(__fadd_rn(score, x1), bw.y);
                c2 = __fadd_rn(__fadd_rn(score, x2), bw.z);
                c3 = __fadd_rn(__fadd_rn(score, x3), bw.w);
                c4 = __fadd_rn(__fadd_rn(score, a.stay), bs);
                c0 = act ? c0 : -INFINITY;
                c1 = act ? c1 : -INFINITY;
                c2 = act ? c2 : -INFINITY;
                c3 = act ? c3 : -INFINITY;
                c4 = act ? c4 : -INFINITY;
            }
            const int mine_back = sm.owner[own_at];
            const int cand_raw = sm.owner[need & 8191u];
            const int cand = act ? cand_raw : 0;
            const uint32_t clash = __ballot_sync(0xffffffffu, mine_back != lane + 1);
            const uint32_t cand_hash = __shfl_sync(0xffffffffu, hash, (cand - 1) & 31);
            int mate = (cand > 0 && cand_hash == need) ? cand - 1 : -1;
            __syncwarp();
            sm.owner[own_at] = 0;

            bool conflict = false;
            if (clash) {
                // exhaustive: for every stay that the table points anywhere, compare against
                // all elements (the reference's semantics, all-pairs)
                mate = -1;
                unsigned long long claimed01 = 0ull, claimed23 = 0ull;
                for (int i = 0; i < W; ++i) {
                    const uint32_t need_i = __shfl_sync(0xffffffffu, need, i);
                    const uint32_t b_i = __shfl_sync(0xffffffffu, b_own, i);
                    const uint32_t m = __ballot_sync(0xffffffffu, act && hash == need_i);
                    if (m) {
                        if (m & (m - 1)) conflict = true;
                        const int jj = __ffs(m) - 1;
                        const unsigned long long bitpos = 1ull << (((b_i & 1u) << 5) + jj);
                        unsigned long long &cl = (b_i & 2u) ? claimed23 : claimed01;
                        if (cl & bitpos) conflict = true;
                        cl |= bitpos;
                        if (lane == i) mate = jj;
                    }
                }
            }
            if (__any_sync(0xffffffffu, mate >= 0)) {
                if (!conflict) {
                    // every stay has at most one partner and no step has two: the folds are
                    // independent.  The stay fetches its partner's step score by shuffle, folds,
                    // and posts the partner's new score in a mailbox the partner reads.
                    const int src = mate >= 0 ? mate : lane;
                    const float y0 = __shfl_sync(0xffffffffu, c0, src), y1 = __shfl_sync(0xffffffffu, c1, src);
                    const float y2 = __shfl_sync(0xffffffffu, c2, src), y3 = __shfl_sync(0xffffffffu, c3, src);
                    if (mate >= 0) {
                        const float x = c4;
                        const float y = b_own == 0 ? y0 : (b_own == 1 ? y1 : (b_own == 2 ? y2 : y3));
                        const float f = fold2(x, y, tr);
                        const bool stay_wins = x > y;
                        c4 = stay_wins ? f : -FLT_MAX;
                        sm.cstep[4 * mate + b_own] = stay_wins ? -FLT_MAX : f;
                    }
                    __syncwarp();
                    const float4 r = *reinterpret_cast<const float4 *>(&sm.cstep[4 * lane]);
                    c0 = isnan(r.x) ? c0 : r.x;
                    c1 = isnan(r.y) ? c1 : r.y;
                    c2 = isnan(r.z) ? c2 : r.z;
                    c3 = isnan(r.w) ? c3 : r.w;
                    __syncwarp();
                    if (mate >= 0) sm.cstep[4 * mate + b_own] = __int_as_float(0x7fc00000);
                } else {
                    // repeated hashes inside the beam (CRC collisions): replay the reference's
                    // nested loop, stay-major then slot-minor, on one lane
                    *reinterpret_cast<float4 *>(&sm.cstep[4 * lane]) = make_float4(c0, c1, c2, c3);
                    sm.rec[lane] = make_uint4(hash, b_own, __float_as_uint(c4), 0u);
                    __syncwarp();
                    if (lane == 0) {
                        for (int i = 0; i < W; ++i) {
                            const uint32_t h_i = sm.rec[i].x, b_i = sm.rec[i].y;
                            for (int jj = 0; jj < W; ++jj) {
                                if (h_i != crc_step2(sm.rec[jj].x, b_i)) continue;
                                const float x = __uint_as_float(sm.rec[i].z);
                                const float y = sm.cstep[4 * jj + b_i];
                                const float f = ofx::fold2_exact(x, y, tr);
                                if (x > y) {
                                    sm.rec[i].z = __float_as_uint(f);
                                    sm.cstep[4 * jj + b_i] = -FLT_MAX;
                                } else {
                                    sm.cstep[4 * jj + b_i] = f;
                                    sm.rec[i].z = __float_as_uint(-FLT_MAX);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (act) c4 = __uint_as_float(sm.rec[lane].z);
                    const float4 r = *reinterpret_cast<const float4 *>(&sm.cstep[4 * lane]);
                    c0 = r.x; c1 = r.y; c2 = r.z; c3 = r.w;
                    __syncwarp();
                    *reinterpret_cast<float4 *>(&sm.cstep[4 * lane]) =
                        make_float4(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000),
                                    __int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
                }
            }

            // pruning threshold (src/beam_search.c:320-381): best - ln(beam_cut); if more than 32
            // candidates pass, bisect towards 25..32 survivors for at most 9 further guesses
            const float best = warp_max_f32(fmaxf(fmaxf(fmaxf(c0, c1), fmaxf(c2, c3)), c4));
            float cut = __fsub_rn(best, a.log_beam_cut);
            auto count_at_least = [&](float th) {
                const int n = (c0 >= th) + (c1 >= th) + (c2 >= th) + (c3 >= th) + (c4 >= th);
                return __reduce_add_sync(0xffffffffu, n);
            };
            int kept = count_at_least(cut);
            if (kept > kBeam) {
                float lo = cut, hi = best;
                int guesses = 1;
                while ((kept > kBeam || kept < 25) && guesses < 10) {
                    if (kept > kBeam) {
                        lo = cut;
                        cut = __fmul_rn(__fadd_rn(cut, hi), 0.5f);
                    } else {
                        hi = cut;
                        cut = __fmul_rn(__fadd_rn(cut, lo), 0.5f);
                    }
                    kept = count_at_least(cut);
                    ++guesses;
                }
                if (guesses == 10) {
                    cut = hi;
                    kept = count_at_least(cut);
                }
                kept = min(kept, kBeam);
            }
            const uint32_t B0 = __ballot_sync(0xffffffffu, c0 >= cut), B1 = __ballot_sync(0xffffffffu, c1 >= cut);
            const uint32_t B2 = __ballot_sync(0xffffffffu, c2 >= cut), B3 = __ballot_sync(0xffffffffu, c3 >= cut);
            const uint32_t B4 = __ballot_sync(0xffffffffu, c4 >= cut);

            // survivors keep candidate order: steps (slot-major, base-minor), then stays.  Each
            // survivor drops {score, parent slot | stay | base} at its new slot; the new owner
            // fetches the parent's hash and k-mer by shuffle and extends them itself.
            {
                int p = (__popc(B0 & lt_mask) + __popc(B1 & lt_mask)) + (__popc(B2 & lt_mask) + __popc(B3 & lt_mask));
                const int nsteps = (__popc(B0) + __popc(B1)) + (__popc(B2) + __popc(B3));
                // a survivor beyond the 32nd, and every non-survivor, writes into a spare slot
                // of its own instead of branching around the store
                const uint32_t bit = 1u << lane;
                const int spare = kBeam + lane;
                const bool k0 = (B0 & bit) != 0, k1 = (B1 & bit) != 0, k2 = (B2 & bit) != 0, k3 = (B3 & bit) != 0;
                const int p0 = p, p1 = p0 + k0, p2 = p1 + k1, p3 = p2 + k2;
                sm.slot[(k0 && p0 < kBeam) ? p0 : spare] = make_uint2(__float_as_uint(c0), lane | (0u << 6));
                sm.slot[(k1 && p1 < kBeam) ? p1 : spare] = make_uint2(__float_as_uint(c1), lane | (1u << 6));
                sm.slot[(k2 && p2 < kBeam) ? p2 : spare] = make_uint2(__float_as_uint(c2), lane | (2u << 6));
                sm.slot[(k3 && p3 < kBeam) ? p3 : spare] = make_uint2(__float_as_uint(c3), lane | (3u << 6));
                const int ps = nsteps + __popc(B4 & lt_mask);
                sm.slot[((B4 & bit) && ps < kBeam) ? ps : spare] = make_uint2(__float_as_uint(c4), lane | 32u | (b_own << 6));
            }
            __syncwarp();
            W = kept;
            const uint2 mine = sm.slot[lane];
            uint32_t meta = lane < W ? mine.y : 0u;
            const uint32_t ph = __shfl_sync(0xffffffffu, hash, meta & 31u);
            const int pst = __shfl_sync(0xffffffffu, state, meta & 31u);
            {
                const bool live = lane < W, stayed = (meta & 32u) != 0;
                const uint32_t h_step = crc_step2(ph, meta >> 6);
                const int s_step = ((pst << 2) & (NS - 1)) | (int)(meta >> 6);
                score = live ? __uint_as_float(mine.x) : score;
                hash = live ? (stayed ? ph : h_step) : hash;
                state = live ? (stayed ? pst : s_step) : state;
            }
            if (t == T - 1) {
                // best survivor swaps into slot 0 (src/beam_search.c:398-414)
                const float sc = lane < W ? score : -INFINITY;
                const float top_s = warp_max_f32(sc);
                const uint32_t eq = __ballot_sync(0xffffffffu, lane < W && sc == top_s && sc > -FLT_MAX);
                const int at = eq ? __ffs(eq) - 1 : 0;
                const uint32_t h0 = __shfl_sync(0xffffffffu, hash, 0), ha = __shfl_sync(0xffffffffu, hash, at);
                const int s0 = __shfl_sync(0xffffffffu, state, 0), sa = __shfl_sync(0xffffffffu, state, at);
                const float v0 = __shfl_sync(0xffffffffu, score, 0), va = __shfl_sync(0xffffffffu, score, at);
                const uint32_t m0_ = __shfl_sync(0xffffffffu, meta, 0), ma = __shfl_sync(0xffffffffu, meta, at);
                if (lane == at) { hash = h0; state = s0; score = v0; meta = m0_; }
                if (lane == 0) { hash = ha; state = sa; score = va; meta = ma; }
            }
            {
                const float back = brow[state];
                score = lane < W ? __fsub_rn(score, back) : score;
            }
            bp_chunk[(size_t)(t + 1) * kBeam + lane] = (unsigned char)meta;
            __syncwarp();
            if (lane == 0) ofd::mbar_arrive(&sm.empty[slot_a]);
        }
    }

    // ---------------------------------------------------------------------- tail, whole block
    __syncthreads();
    // arrays laid over the rings (and the dynamic shared memory behind them)
    unsigned char *tail = sm.score_ring[0];
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
        const int st0 = sm.init_state[at];
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

}  // namespace

namespace {

template <int NS, int RING>
cudaError_t launch(const OfFusedLaunch &l, cudaStream_t stream) {
    using Smem = FusedSmem<NS, RING>;
    const int Tp = (l.T + 16) & ~15;
    const size_t ring_bytes = (size_t)RING * (Smem::kScoreRow + 2 * Smem::kBwdRow);
    const size_t extra = 0;
    const size_t tail = (size_t)kWin * kBeam + (kWin / 8) * (kBeam + 4) + 8 * (size_t)Tp + 64;
    size_t bytes = sizeof(Smem) + extra + 128;
    if (tail > ring_bytes + extra) bytes += tail - (ring_bytes + extra);
    if (bytes > 227 * 1024) return cudaErrorInvalidValue;
    auto kern = fwd_beam_kernel<NS, RING>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    FusedArgs a;
    a.scores = static_cast<const __half *>(l.scores_fp16);
    a.bwd = l.bwd; a.fwd = l.fwd; a.post = l.post; a.bp = l.bp; a.moves = l.moves; a.sequence = l.sequence;
    a.qstring = l.qstring; a.states = l.states; a.qual = l.qual; a.base_probs = l.base_probs;
    a.total_probs = l.total_probs; a.tables = l.tables; a.status = l.status;
    a.T = l.T; a.N = l.N; a.C = l.C; a.stay = l.stay; a.log_beam_cut = l.log_beam_cut;
    a.q_shift = l.q_shift; a.q_scale = l.q_scale;
    constexpr int NT = (NS / 4 < 32 ? 32 : NS / 4) + 64;
    kern<<<l.N, NT, bytes, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

cudaError_t of_launch_fwd_beam(const OfFusedLaunch &l, cudaStream_t stream) {
    switch (l.state_len) {
        case 3: return launch<64, 8>(l, stream);
        case 4: return launch<256, 8>(l, stream);
        case 5: return launch<1024, 6>(l, stream);
        default: return cudaErrorInvalidValue;
    }
}

size_t of_fwd_beam_max_T(int state_len) {
    // largest T whose tail arrays fit in 227 KB next to the fixed part of the block's shared memory
    (void)state_len;
    return 16384;
}
