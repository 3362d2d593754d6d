// beam_search.cu -- the beam search of the CRF-CTC decode, one warp per chunk, for sm_100a.
//
// Replaces the reference kernel beam_search (src/beam_search_cuda.cu:139-528) up to, but not
// including, its traceback.  It follows the reference's CPU routine beam_search_cpu
// (src/beam_search.c:117-428) -- including its bisection of the pruning threshold, which the
// reference's CUDA kernel lacks -- because output parity is defined against the CPU decoder.
//
// A block is one chunk: a beam warp and a copy warp.
//   beam warp    lane = beam slot (width <= 32).  Everything is warp-synchronous and, where
//                lanes differ, branch free: candidate scores, duplicate-prefix merges (CRC32C
//                hashes; a stay merges with the step whose parent hash equals the stay's hash
//                run backwards through the CRC), maximum, threshold bisection by warp
//                reductions, order-preserving compaction by ballots.  One packed back-pointer
//                byte per slot and timestep goes to HBM (prev slot 5 bits | stay 1 bit | base
//                2 bits), plus the 32 initial k-mers; the traceback happens in the kernel that
//                also needs the posterior (posterior_seq.cu).
//   copy warp    one lane issues 1-D bulk asynchronous copies (no multicast) of score row t
//                (timesteps strided by N*C as in src/decode_cpu.c:204,216) and backward row t
//                into a ring; the beam warp releases a slot through an mbarrier.
// The kernel is a chain of T dependent, latency-bound steps per chunk and leaves most issue
// slots free, which is why the forward scan runs beside it on another stream.
#include <float.h>

#include "beam_post.cuh"
#include "exact_math.cuh"
#include "fast_lse.cuh"
#include "of_device.cuh"

namespace {

constexpr int kBeam = 32;
// Threads per block: the beam warp, the copy warp and a padding warp that exits at once.  With
// two-warp blocks the warp slots of an SM fill in pairs and every beam warp lands on the same two
// of the four schedulers, where they queue behind each other; a block of three warps rotates them
// over all four (measured on the hac decode: 3.87 -> 3.58 ms; fast, with seven blocks per SM:
// 4.84 -> 4.39 ms).
constexpr int kBeamBlock = 96;


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

template <int NS, int RING>
struct BeamSmem {
    static constexpr int kScoreRow = NS * 8;  // bytes of one fp16 score row
    static constexpr int kBwdRow = NS * 4;    // bytes of one fp32 backward row
    alignas(16) uint4 rec[kBeam];
    alignas(16) float cstep[kBeam * 4];
    alignas(8) uint2 slot[2 * kBeam];  // compaction (+ one spare per lane): {score, parent slot | stay << 5 | base << 6}
    unsigned char owner[8192 + 32];    // (+ one spare per lane) hash -> slot + 1 of the beam element owning it
    int init_state[kBeam];
    double exp2_j[ofx::kExpTab];
    double rcp_c[ofx::kLogTab];
    double log_c[ofx::kLogTab];
    alignas(8) uint64_t full[RING];
    alignas(8) uint64_t empty[RING];
    int abort_flag;
    alignas(128) unsigned char score_ring[RING][kScoreRow];
    alignas(128) unsigned char bwd_ring[RING][kBwdRow];
};

template <int NS, int RING>
__global__ void __launch_bounds__(kBeamBlock)
beam_search_kernel(const OfDecodeArgs a) {
    constexpr int BITS = (NS == 64) ? 6 : (NS == 256 ? 8 : 10);
    constexpr int MSB = NS / 4;
    constexpr int NT = kBeamBlock;
    using Smem = BeamSmem<NS, RING>;
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
            ofd::mbar_init(&sm.empty[r], 1);
        }
        ofd::mbar_fence_init();
    }
    __syncthreads();

    const float *bwd_chunk = a.bwd + (size_t)chunk * (size_t)(T + 1) * NS;
    unsigned char *bp_chunk = a.bp + (size_t)chunk * (size_t)(T + 1) * kBeam;

    if (warp >= 2) return;  // the padding warp: it has helped to set shared memory up, that is all
    if (warp == 1) {
        // ------------------------------------------------------------------ copy warp
        if (lane == 0) {
            // the beam search strides timesteps by N*C (src/decode_cpu.c:204,216)
            const __half *beam_scores = a.scores + (size_t)chunk * NS * 4;
            const size_t beam_stride = (size_t)N * a.C;
            int issued = 0;
            for (int t = 0; t <= T; ++t, ++issued) {
                const int slot = t % RING;
                if (t >= RING)
                    ofd::mbar_wait_bounded(&sm.empty[slot], (uint32_t)(t / RING - 1) & 1u,
                                           &sm.abort_flag, a.status, a.wait_ns);
                if (sm.abort_flag) break;
                const uint32_t bytes = Smem::kBwdRow + (t < T ? Smem::kScoreRow : 0);
                ofd::mbar_arrive_expect_tx(&sm.full[slot], bytes);
                ofd::bulk_g2s(sm.bwd_ring[slot], bwd_chunk + (size_t)t * NS, Smem::kBwdRow, &sm.full[slot]);
                if (t < T)
                    ofd::bulk_g2s(sm.score_ring[slot], beam_scores + beam_stride * t, Smem::kScoreRow,
                                  &sm.full[slot]);
            }
            // after an abort: the newest copies get a bounded chance to land before the block retires
            if (sm.abort_flag) ofd::mbar_drain_bounded(sm.full, RING, issued, a.wait_ns);
        }
        return;
    }
    // ------------------------------------------------------------------ beam warp
    const ofx::TabRef tr = {sm.exp2_j, 1, sm.rcp_c, sm.log_c};
    const uint32_t lt_mask = (1u << lane) - 1u;
    ofd::mbar_wait_bounded(&sm.full[0], 0, &sm.abort_flag, a.status, a.wait_ns);
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
        ofd::mbar_wait_bounded(&sm.full[slot_b], (uint32_t)((t + 1) / RING) & 1u, &sm.abort_flag, a.status, a.wait_ns);
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
            // (float)score * score_scale, rounded before it is added (src/beam_search.c:233-234)
            const float x0 = __fmul_rn(__half2float(sp[0]), a.score_scale), x1 = __fmul_rn(__half2float(sp[4]), a.score_scale);
            const float x2 = __fmul_rn(__half2float(sp[8]), a.score_scale), x3 = __fmul_rn(__half2float(sp[12]), a.score_scale);
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
        const float best = warp_max_f32(ofd::max3(ofd::max3(c0, c1, c2), c3, c4));
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
    // the initial k-mers, for the traceback's benefit
    a.init_kmers[(size_t)chunk * kBeam + lane] = sm.init_state[lane];
}

template <int NS, int RING>
cudaError_t launch_beam(const OfDecodeArgs &a, cudaStream_t stream) {
    using Smem = BeamSmem<NS, RING>;
    const size_t bytes = sizeof(Smem) + 128;
    auto kern = beam_search_kernel<NS, RING>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    kern<<<a.N, kBeamBlock, bytes, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

cudaError_t of_launch_beam_search(const OfDecodeArgs &a, cudaStream_t stream) {
    switch (a.state_len) {
        case 3: return launch_beam<64, 8>(a, stream);
        case 4: return launch_beam<256, 4>(a, stream);
        case 5: return launch_beam<1024, 4>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}
