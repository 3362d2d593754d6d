// decode_static.cu -- a decode entry point that allocates nothing.
//
// Some callers cannot let a library allocate device memory once they are running: a serving
// process that hands all free device memory to its own arena at start-up (a later cudaMalloc
// from a library then fails or fragments the arena), or a pipeline that must not hit the
// device-wide synchronisation a cudaMalloc / cudaFree implies in the middle of its steady
// state.  openfish_gpubuf_init does ten cudaMallocs, a cudaMallocHost, a stream and four events,
// and openfish_decode_gpu three host mallocs per call.  The entry point below needs none of
// that: every intermediate of the decode (backward scores, posteriors, back-pointers, path
// states, per-timestep qualities, the arithmetic tables, the status word) lives in ONE
// file-scope device array of fixed size, the results go to device buffers the caller owns, the
// work runs on the legacy default stream, and the only runtime calls are kernel launches,
// cudaMemsetAsync, cudaMemcpy and cudaStreamSynchronize.
//
// Limits and rules (also in openfish_b200.h):
//   * the array is kStaticScratchBytes = 48 MiB; every GPU on which this library's module gets
//     loaded holds that much until the process exits.  Shapes that need more are refused.
//   * all calls on a device share the array: it keeps the previous call's contents (whatever
//     must start from zero is cleared by the call itself), and two calls that overlap on the
//     same GPU -- from two host threads -- race.  Serialise them.
//   * the first call on each device looks up the array's device address and uploads the tables.
//     Make that first call before starting any stream capture.
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>

#include <mutex>

#include "scan.cuh"
#include "exact_math.cuh"
#include "beam_post.cuh"
#include "of_device.cuh"
#include "openfish_b200.h"

namespace {

constexpr size_t kStaticScratchBytes = OPENFISH_B200_STATIC_SCRATCH_BYTES;
// In host code this name is only a handle for the runtime's symbol look-up, not a device
// address; kernels receive the address cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char *g_base[kMaxDevices];  // device address of the array, per device; null = not set up
std::mutex g_setup_lock;

size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

int report(int code, const char *text) {
    if (get_openfish_log_level() >= OPENFISH_LOG_ERR)
        fprintf(stderr, "[openfish_b200_decode_static::OPENFISH_ERROR]\033[1;31m %s\033[0m\n", text);
    return code;
}

// Once per device, with that device current: resolve the array's address, put the tables at its
// start.  No allocation: the tables travel from this function's stack.
int setup_device(int dev, unsigned char **base_out) {
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_base[dev]) {
        unsigned char *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_scratch);
        if (e != cudaSuccess || !p) {
            char msg[160];
            snprintf(msg, sizeof(msg), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return report(OPENFISH_B200_ERR_CUDA, msg);
        }
        ofx::Tables host_tables;
        ofx::fill_tables(&host_tables);
        e = cudaMemcpy(p, &host_tables, sizeof(host_tables), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            char msg[160];
            snprintf(msg, sizeof(msg), "uploading the tables failed: %s", cudaGetErrorString(e));
            return report(OPENFISH_B200_ERR_CUDA, msg);
        }
        g_base[dev] = p;
    }
    *base_out = g_base[dev];
    return OPENFISH_B200_OK;
}

}  // namespace

extern "C" int openfish_b200_decode_static(int T, int N, int C, const void *scores_TNC,
                                           int state_len, const openfish_opt_t *options,
                                           uint8_t *moves_gpu, char *sequence_gpu,
                                           char *qstring_gpu) {
    if (!scores_TNC || !options || !moves_gpu || !sequence_gpu || !qstring_gpu)
        return report(OPENFISH_B200_ERR_ARGUMENT, "NULL pointer argument");
    if (state_len < 3 || state_len > 5 || T < 1 || N < 1)
        return report(OPENFISH_B200_ERR_ARGUMENT, "need T >= 1, N >= 1 and state_len 3, 4 or 5");
    if (T > 16384) return report(OPENFISH_B200_ERR_TOO_LONG, "T exceeds 16384 timesteps");
    const size_t ns = (size_t)1 << (2 * state_len);
    if (C < 0 || (size_t)C < 4 * ns || C % 8 != 0 || ((size_t)scores_TNC & 15u))
        return report(OPENFISH_B200_ERR_LAYOUT,
                      "C must be a multiple of 8 and at least 4*4^state_len, scores 16-byte aligned");
    if (options->beam_width != 32)
        return report(OPENFISH_B200_ERR_OPTION, "beam_width must be 32");

    // carve the array: tables | status | bwd | fwd | post | back-pointers | states | qual | probs
    // (no forward tensor for the models whose forward scan forms the posterior itself)
    const bool fused = of_forward_posterior_fused(state_len);
    const size_t nt = (size_t)N * T, rows = (size_t)N * (T + 1);
    size_t off = 0;
    const size_t o_tables = off; off += align_up(sizeof(ofx::Tables));
    const size_t o_status = off; off += 256;
    const size_t o_bwd = off; off += align_up(rows * ns * sizeof(float));
    const size_t o_fwd = off; off += fused ? 0 : align_up(rows * ns * sizeof(float));
    const size_t o_post = off; off += align_up(rows * ns * sizeof(float));
    const size_t o_bp = off; off += align_up(rows * 32);
    const size_t o_init = off; off += align_up((size_t)N * 32 * sizeof(int));
    const size_t o_states = off; off += align_up(nt * sizeof(int));
    const size_t o_qual = off; off += align_up(nt * 4 * sizeof(float));
    const size_t o_base = off; off += align_up(nt * sizeof(float));
    const size_t o_total = off; off += align_up(nt * sizeof(float));
    if (off > kStaticScratchBytes) {
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "T=%d N=%d state_len=%d needs %zu bytes of scratch, the static array holds %zu",
                 T, N, state_len, off, kStaticScratchBytes);
        return report(OPENFISH_B200_ERR_SCRATCH_LIMIT, msg);
    }

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return report(OPENFISH_B200_ERR_CUDA, "no usable current CUDA device");
    unsigned char *base = nullptr;
    const int rc = setup_device(dev, &base);
    if (rc != OPENFISH_B200_OK) return rc;

    const ofx::Tables *tables = reinterpret_cast<const ofx::Tables *>(base + o_tables);
    int *status = reinterpret_cast<int *>(base + o_status);
    float *bwd = reinterpret_cast<float *>(base + o_bwd);
    float *fwd = fused ? nullptr : reinterpret_cast<float *>(base + o_fwd);
    float *post = reinterpret_cast<float *>(base + o_post);
    cudaStream_t stream = 0;  // legacy default stream: nothing to create
    e = cudaMemsetAsync(status, 0, sizeof(int), stream);  // the one thing that must start at zero
    if (e == cudaSuccess)
        e = of_launch_scans(scores_TNC, bwd, fwd, T, N, state_len, options->blank_score, tables,
                            status, ofd::kDefaultWaitLimitNs, stream);
    if (e == cudaSuccess && fused)
        e = of_launch_forward_posterior(scores_TNC, bwd, post, T, N, state_len, options->blank_score,
                                        tables, status, ofd::kDefaultWaitLimitNs, stream);
    if (e == cudaSuccess) {
        OfDecodeArgs a;
        a.scores = static_cast<const __half *>(scores_TNC);
        a.bwd = bwd;
        a.fwd = fwd;
        a.post = post;
        a.bp = base + o_bp;
        a.init_kmers = reinterpret_cast<int *>(base + o_init);
        a.moves = moves_gpu;
        a.sequence = sequence_gpu;
        a.qstring = qstring_gpu;
        a.states = reinterpret_cast<int *>(base + o_states);
        a.qual = reinterpret_cast<float *>(base + o_qual);
        a.base_probs = reinterpret_cast<float *>(base + o_base);
        a.total_probs = reinterpret_cast<float *>(base + o_total);
        a.tables = tables;
        a.status = status;
        a.wait_ns = ofd::kDefaultWaitLimitNs;
        a.T = T; a.N = N; a.C = C; a.state_len = state_len;
        a.stay = options->blank_score;
        a.log_beam_cut = options->beam_cut > 0.0f ? logf(options->beam_cut) : 3.402823466e+38f;
        a.q_shift = options->q_shift;
        a.q_scale = options->q_scale;
        a.score_scale = options->temperature;
        e = of_launch_beam_search(a, stream);
        if (e == cudaSuccess) e = of_launch_posterior_seq(a, stream);
    }
    int dev_status = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&dev_status, status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        char msg[200];
        snprintf(msg, sizeof(msg), "CUDA failure: %s", cudaGetErrorString(e));
        return report(OPENFISH_B200_ERR_CUDA, msg);
    }
    if (dev_status != ofd::kStatusOk)
        return report(OPENFISH_B200_ERR_DEVICE_WAIT, "a kernel gave up waiting for an asynchronous copy");
    return OPENFISH_B200_OK;
}
