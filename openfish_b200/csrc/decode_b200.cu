// decode_b200.cu -- device buffers, stream and launch orchestration of the decode path.
//
// Replaces gpubuf_init_cuda / gpubuf_free_cuda / decode_cuda (src/decode_cuda.cu:11-212).
// Differences in design: the caller-visible openfish_gpubuf_t sits at the start of a private
// record that also owns two streams, events, the arithmetic tables and a page-locked staging
// area; one decode is four kernel launches -- backward scan; beam search with the forward scan
// beside it on the second stream; posterior + traceback + sequence -- and one device-to-host
// copy, all stream
// ordered, with a single host wait at the end (the reference launches five kernels and three
// memsets with a device-wide synchronisation after each and copies with three blocking
// pageable transfers).
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "backend.h"
#include "scan.cuh"
#include "exact_math.cuh"
#include "beam_post.cuh"
#include "of_device.cuh"
#include "openfish_b200.h"
#include "rotary.cuh"

namespace {

constexpr uint32_t kMagic = 0x0F15B200u;

struct GpuBuf {
    openfish_gpubuf_t pub;  // must stay first: the public pointer is the record's address
    uint32_t magic;
    int T, N, state_len, device;
    cudaStream_t stream;   // everything but the forward scan; blocking, see ofb_gpubuf_create
    cudaStream_t stream2;  // the forward scan, ordered against `stream` by events only
    cudaEvent_t ev[9];     // 0 start, 1 bwd scan done, 2 beam search done, 3 sequence done, 4 copies done,
                           // 5 fwd scan start, 6 fwd scan done, 7 the caller's stream at submit time, 8 blank-column strip start
    uint64_t wait_ns;      // how long a kernel waits for an asynchronous copy before it raises d_status
    int *d_init_kmers;     // inside the beam_vector allocation, behind the back-pointers
    ofx::Tables *d_tables;
    float *d_fwd;              // forward scores [N][T+1][ns]: scan kernel -> posterior kernel (64-state model
                               // only; null otherwise: the forward scan kernel writes the posterior)
    int *d_status;
    void *d_scores4;           // 4-wide copy of 5-wide scores, made on the first 5-wide decode (null before)
    int sms;
    unsigned char *d_results;  // moves | sequence | qstring, N*T bytes each
    unsigned char *h_stage;    // page-locked, 3*N*T bytes + one status word
    int *h_status;
    // decode in flight
    bool pending;
    uint8_t *dst_moves;
    char *dst_sequence, *dst_qstring;
    bool via_stage;
    float ms[8];
    bool stripped = false;  // the decode in flight began with the blank-column strip
};

thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define CU(call)                                                                              \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess)                                                                \
            return fail(e_ == cudaErrorMemoryAllocation ? OPENFISH_B200_ERR_ALLOC             \
                                                        : OPENFISH_B200_ERR_CUDA,             \
                        "%s failed: %s", #call, cudaGetErrorString(e_));                      \
    } while (0)

GpuBuf *priv(const openfish_gpubuf_t *g) {
    return reinterpret_cast<GpuBuf *>(const_cast<openfish_gpubuf_t *>(g));
}

bool host_is_pinned(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeHost;
}

int destroy(GpuBuf *g) {
    if (!g) return OPENFISH_B200_OK;
    if (g->pending && g->stream) cudaStreamSynchronize(g->stream);
    if (g->pending && g->stream2) cudaStreamSynchronize(g->stream2);
    cudaFree(g->pub.bwd_NTC);
    cudaFree(g->pub.post_NTC);
    cudaFree(g->d_results);
    cudaFree(g->pub.beam_vector);
    cudaFree(g->pub.states);
    cudaFree(g->pub.qual_data);
    cudaFree(g->pub.base_probs);
    cudaFree(g->pub.total_probs);
    cudaFree(g->d_tables);
    cudaFree(g->d_fwd);
    cudaFree(g->d_status);
    cudaFree(g->d_scores4);
    if (g->h_stage) cudaFreeHost(g->h_stage);
    for (int i = 0; i < 9; ++i)
        if (g->ev[i]) cudaEventDestroy(g->ev[i]);
    if (g->stream2) cudaStreamDestroy(g->stream2);
    if (g->stream) cudaStreamDestroy(g->stream);
    g->magic = 0;
    free(g);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(OPENFISH_B200_ERR_CUDA, "releasing device buffers failed: %s", cudaGetErrorString(e));
    return OPENFISH_B200_OK;
}

}  // namespace

extern "C" const char *ofb_error_text(void) { return g_err; }

extern "C" int ofb_gpubuf_create(int T, int N, int state_len, openfish_gpubuf_t **out) {
    *out = nullptr;
    GpuBuf *g = static_cast<GpuBuf *>(calloc(1, sizeof(GpuBuf)));
    if (!g) return fail(OPENFISH_B200_ERR_ALLOC, "out of host memory");
    g->T = T; g->N = N; g->state_len = state_len;
    const size_t ns = (size_t)1 << (2 * state_len);
    const size_t nt = (size_t)N * T;
    const size_t tens = (size_t)N * (T + 1) * ns * sizeof(float);
    int rc = [&]() -> int {
        CU(cudaGetDevice(&g->device));
        CU(cudaDeviceGetAttribute(&g->sms, cudaDevAttrMultiProcessorCount, g->device));
        // a blocking stream: ordered after work the caller queued on the legacy default
        // stream (where the reference runs), so freshly written scores are seen
        CU(cudaStreamCreateWithFlags(&g->stream, cudaStreamDefault));
        CU(cudaStreamCreateWithFlags(&g->stream2, cudaStreamNonBlocking));
        for (int i = 0; i < 9; ++i) CU(cudaEventCreate(&g->ev[i]));
        g->wait_ns = ofd::kDefaultWaitLimitNs;
        // same ten buffers and sizes as the reference (src/decode_cuda.cu:22-45); the three
        // result arrays share one allocation so that one copy brings them back
        CU(cudaMalloc(&g->pub.bwd_NTC, tens));
        CU(cudaMalloc(&g->pub.post_NTC, tens));
        // (models whose forward scan writes the posterior itself need no forward tensor)
        if (!of_forward_posterior_fused(state_len)) CU(cudaMalloc(&g->d_fwd, tens));
        CU(cudaMalloc(&g->d_results, 3 * nt));
        g->pub.moves = g->d_results;
        g->pub.sequence = reinterpret_cast<char *>(g->d_results + nt);
        g->pub.qstring = reinterpret_cast<char *>(g->d_results + 2 * nt);
        // reference-sized (8 bytes per beam slot and timestep); this library uses 1 byte of the 8
        // for its packed back-pointers and 128 bytes per chunk behind them for the initial k-mers
        CU(cudaMalloc(&g->pub.beam_vector, (size_t)8 * N * 32 * (T + 1)));
        g->d_init_kmers = reinterpret_cast<int *>(static_cast<unsigned char *>(g->pub.beam_vector) +
                                                  (((size_t)N * 32 * (T + 1) + 255) & ~(size_t)255));
        CU(cudaMalloc(&g->pub.states, sizeof(int32_t) * nt));
        CU(cudaMalloc(&g->pub.qual_data, sizeof(float) * nt * 4));
        CU(cudaMalloc(&g->pub.base_probs, sizeof(float) * nt));
        CU(cudaMalloc(&g->pub.total_probs, sizeof(float) * nt));
        CU(cudaMalloc(&g->d_tables, sizeof(ofx::Tables)));
        CU(cudaMalloc(&g->d_status, sizeof(int)));
        CU(cudaMallocHost(&g->h_stage, 3 * nt + 16));
        g->h_status = reinterpret_cast<int *>(g->h_stage + ((3 * nt + 7) & ~(size_t)7));
        ofx::Tables host_tables;
        ofx::fill_tables(&host_tables);
        CU(cudaMemcpy(g->d_tables, &host_tables, sizeof(host_tables), cudaMemcpyHostToDevice));
        CU(cudaMemset(g->d_status, 0, sizeof(int)));
        return OPENFISH_B200_OK;
    }();
    if (rc != OPENFISH_B200_OK) {
        char keep[sizeof(g_err)];
        memcpy(keep, g_err, sizeof(keep));
        destroy(g);
        memcpy(g_err, keep, sizeof(keep));
        return rc;
    }
    g->magic = kMagic;
    *out = &g->pub;
    return OPENFISH_B200_OK;
}

extern "C" int ofb_gpubuf_destroy(openfish_gpubuf_t *gpubuf) {
    if (!gpubuf) return OPENFISH_B200_OK;
    GpuBuf *g = priv(gpubuf);
    if (g->magic != kMagic) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf was not created by openfish_gpubuf_init");
    return destroy(g);
}

extern "C" int ofb_gpubuf_check_owner(const openfish_gpubuf_t *gpubuf) {
    if (!gpubuf) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf is NULL");
    if (priv(gpubuf)->magic != kMagic) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf was not created by openfish_gpubuf_init");
    return OPENFISH_B200_OK;
}

extern "C" int ofb_gpubuf_check(const openfish_gpubuf_t *gpubuf, int T, int N, int state_len) {
    if (!gpubuf) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf is NULL");
    const GpuBuf *g = priv(gpubuf);
    if (g->magic != kMagic) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf was not created by openfish_gpubuf_init");
    if (g->T != T || g->N != N || g->state_len != state_len)
        return fail(OPENFISH_B200_ERR_SHAPE, "gpubuf was sized for T=%d N=%d state_len=%d, decode asked for T=%d N=%d state_len=%d",
                    g->T, g->N, g->state_len, T, N, state_len);
    return OPENFISH_B200_OK;
}

extern "C" int ofb_decode_submit(int T, int N, int C, const void *scores, int state_len,
                                 const ofb_decode_params_t *params, const openfish_gpubuf_t *gpubuf,
                                 uint8_t *moves, char *sequence, char *qstring) {
    GpuBuf *g = priv(gpubuf);
    const float beam_cut = params->beam_cut, blank_score = params->blank_score;
    const float q_shift = params->q_shift, q_scale = params->q_scale;
    if (g->pending) return fail(OPENFISH_B200_ERR_ARGUMENT, "a decode is already in flight on this gpubuf");
    int dev = -1;
    CU(cudaGetDevice(&dev));
    if (dev != g->device) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf belongs to device %d, current device is %d", g->device, dev);
    const size_t nt = (size_t)N * T;

    OfDecodeArgs a;
    a.scores = static_cast<const __half *>(scores);
    a.bwd = g->pub.bwd_NTC;
    a.fwd = g->d_fwd;
    a.post = g->pub.post_NTC;
    a.bp = static_cast<unsigned char *>(g->pub.beam_vector);
    a.init_kmers = g->d_init_kmers;
    a.moves = g->pub.moves;
    a.sequence = g->pub.sequence;
    a.qstring = g->pub.qstring;
    a.states = static_cast<int *>(g->pub.states);
    a.qual = g->pub.qual_data;
    a.base_probs = g->pub.base_probs;
    a.total_probs = g->pub.total_probs;
    a.tables = g->d_tables;
    a.status = g->d_status;
    a.wait_ns = g->wait_ns;
    a.T = T; a.N = N; a.C = C; a.state_len = state_len;
    a.stay = blank_score;
    a.log_beam_cut = beam_cut > 0.0f ? logf(beam_cut) : 3.402823466e+38f;  // src/beam_search.c:135
    a.q_shift = q_shift;
    a.q_scale = q_scale;
    a.score_scale = params->score_scale;

    // stream:  backward scan -> beam search ----------------------> posterior + sequence -> copies
    // stream2:                  forward scan (beside the beam search) --^
    // (for hac and sup the forward scan kernel also writes the posterior, and a.fwd is null)
    // Ordering against the producer of the scores: the gpubuf's main stream is a blocking one, so it
    // runs after whatever the caller queued on the legacy default stream (the reference's stream);
    // a caller that works on a stream of its own names it, and the decode waits for that stream's
    // work as of now.
    if (params->on_caller_stream) {
        cudaStream_t caller = static_cast<cudaStream_t>(params->caller_stream);
        CU(cudaEventRecord(g->ev[7], caller));
        CU(cudaStreamWaitEvent(g->stream, g->ev[7], 0));
    }
    CU(cudaEventRecord(g->ev[0], g->stream));
    CU(of_launch_scans(scores, g->pub.bwd_NTC, nullptr, T, N, state_len, blank_score, g->d_tables,
                       g->d_status, g->wait_ns, g->stream));
    CU(cudaEventRecord(g->ev[1], g->stream));
    CU(cudaStreamWaitEvent(g->stream2, g->ev[1], 0));
    CU(cudaEventRecord(g->ev[5], g->stream2));
    if (of_forward_posterior_fused(state_len))
        CU(of_launch_forward_posterior(scores, g->pub.bwd_NTC, g->pub.post_NTC, T, N, state_len, blank_score,
                                       g->d_tables, g->d_status, g->wait_ns, g->stream2));
    else
        CU(of_launch_scans(scores, nullptr, g->d_fwd, T, N, state_len, blank_score, g->d_tables,
                           g->d_status, g->wait_ns, g->stream2));
    CU(cudaEventRecord(g->ev[6], g->stream2));
    CU(of_launch_beam_search(a, g->stream));
    CU(cudaEventRecord(g->ev[2], g->stream));
    CU(cudaStreamWaitEvent(g->stream, g->ev[6], 0));
    CU(of_launch_posterior_seq(a, g->stream));
    CU(cudaEventRecord(g->ev[3], g->stream));

    // results: straight into page-locked caller memory, else through the staging area
    g->via_stage = !(host_is_pinned(moves) && host_is_pinned(sequence) && host_is_pinned(qstring));
    if (g->via_stage) {
        CU(cudaMemcpyAsync(g->h_stage, g->d_results, 3 * nt, cudaMemcpyDeviceToHost, g->stream));
    } else {
        CU(cudaMemcpyAsync(moves, g->pub.moves, nt, cudaMemcpyDeviceToHost, g->stream));
        CU(cudaMemcpyAsync(sequence, g->pub.sequence, nt, cudaMemcpyDeviceToHost, g->stream));
        CU(cudaMemcpyAsync(qstring, g->pub.qstring, nt, cudaMemcpyDeviceToHost, g->stream));
    }
    CU(cudaMemcpyAsync(g->h_status, g->d_status, sizeof(int), cudaMemcpyDeviceToHost, g->stream));
    CU(cudaEventRecord(g->ev[4], g->stream));
    g->dst_moves = moves;
    g->dst_sequence = sequence;
    g->dst_qstring = qstring;
    g->pending = true;
    return OPENFISH_B200_OK;
}

namespace {
// Waits for the gpubuf's main stream, then looks at the status word its kernels share (copied to
// the host by the last operation queued): a raised status is reported and cleared on the device.
int stream_done_and_status(GpuBuf *g) {
    CU(cudaStreamSynchronize(g->stream));
    if (*g->h_status != ofd::kStatusOk) {
        const int st = *g->h_status;
        *g->h_status = ofd::kStatusOk;
        CU(cudaMemsetAsync(g->d_status, 0, sizeof(int), g->stream));
        return fail(OPENFISH_B200_ERR_DEVICE_WAIT, "a kernel raised device status %d (an asynchronous copy did not complete in time)", st);
    }
    return OPENFISH_B200_OK;
}
}  // namespace

extern "C" int ofb_decode_submit_5wide(int T, int N, const void *scores5, int state_len, float clamp,
                                       const ofb_decode_params_t *params, const openfish_gpubuf_t *gpubuf,
                                       uint8_t *moves, char *sequence, char *qstring) {
    GpuBuf *g = priv(gpubuf);
    if (g->pending) return fail(OPENFISH_B200_ERR_ARGUMENT, "a decode is already in flight on this gpubuf");
    int dev = -1;
    CU(cudaGetDevice(&dev));
    if (dev != g->device) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf belongs to device %d, current device is %d", g->device, dev);
    const size_t ns = (size_t)1 << (2 * state_len);
    if (!g->d_scores4) CU(cudaMalloc(&g->d_scores4, (size_t)T * N * 4 * ns * sizeof(__half)));
    if (params->on_caller_stream) {
        cudaStream_t caller = static_cast<cudaStream_t>(params->caller_stream);
        CU(cudaEventRecord(g->ev[7], caller));
        CU(cudaStreamWaitEvent(g->stream, g->ev[7], 0));
    }
    CU(cudaEventRecord(g->ev[8], g->stream));
    CU(of_launch_strip_blank(scores5, g->d_scores4, (long long)T * N, state_len, clamp, g->sms, g->stream));
    g->stripped = true;
    ofb_decode_params_t p = *params;
    p.on_caller_stream = 0;  // (already ordered: the copy above runs on the gpubuf's stream)
    return ofb_decode_submit(T, N, (int)(4 * ns), g->d_scores4, state_len, &p, gpubuf, moves, sequence, qstring);
}

extern "C" int ofb_decode_wait(const openfish_gpubuf_t *gpubuf) {
    GpuBuf *g = priv(gpubuf);
    if (!g->pending) return OPENFISH_B200_OK;
    g->pending = false;
    const int rc = stream_done_and_status(g);
    if (rc != OPENFISH_B200_OK) return rc;
    const size_t nt = (size_t)g->N * g->T;
    if (g->via_stage) {
        memcpy(g->dst_moves, g->h_stage, nt);
        memcpy(g->dst_sequence, g->h_stage + nt, nt);
        memcpy(g->dst_qstring, g->h_stage + 2 * nt, nt);
    }
    // ms: 0 backward scan, 1 everything between it and the copies (beam search with the forward
    // scan beside it, then posterior + sequence), 2 copies, 3 all of it; detail: 4 beam search,
    // 5 forward scan, 6 posterior + sequence (from the later of its two inputs), 7 the blank-column
    // strip in front of a 5-wide decode (0 otherwise)
    cudaEventElapsedTime(&g->ms[0], g->ev[0], g->ev[1]);
    cudaEventElapsedTime(&g->ms[1], g->ev[1], g->ev[3]);
    cudaEventElapsedTime(&g->ms[2], g->ev[3], g->ev[4]);
    cudaEventElapsedTime(&g->ms[3], g->ev[0], g->ev[4]);
    cudaEventElapsedTime(&g->ms[4], g->ev[1], g->ev[2]);
    cudaEventElapsedTime(&g->ms[5], g->ev[5], g->ev[6]);
    float from_beam = 0.f, from_fwd = 0.f;
    cudaEventElapsedTime(&from_beam, g->ev[2], g->ev[3]);
    cudaEventElapsedTime(&from_fwd, g->ev[6], g->ev[3]);
    g->ms[6] = from_beam < from_fwd ? from_beam : from_fwd;
    g->ms[7] = 0.f;
    if (g->stripped) cudaEventElapsedTime(&g->ms[7], g->ev[8], g->ev[0]);
    g->stripped = false;
    return OPENFISH_B200_OK;
}

extern "C" int ofb_stream_wait_decode(void *stream, const openfish_gpubuf_t *gpubuf) {
    GpuBuf *g = priv(gpubuf);
    if (!g->pending) return OPENFISH_B200_OK;  // nothing in flight: nothing to wait for
    CU(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), g->ev[4], 0));
    return OPENFISH_B200_OK;
}

extern "C" int ofb_selfcheck_wait(const openfish_gpubuf_t *gpubuf, unsigned limit_us) {
    GpuBuf *g = priv(gpubuf);
    if (g->pending) return fail(OPENFISH_B200_ERR_ARGUMENT, "a decode is in flight on this gpubuf");
    int dev = -1;
    CU(cudaGetDevice(&dev));
    if (dev != g->device) return fail(OPENFISH_B200_ERR_ARGUMENT, "gpubuf belongs to device %d, current device is %d", g->device, dev);
    CU(of_launch_wait_that_runs_out(g->d_status, (uint64_t)limit_us * 1000ull, g->stream));
    CU(cudaMemcpyAsync(g->h_status, g->d_status, sizeof(int), cudaMemcpyDeviceToHost, g->stream));
    return stream_done_and_status(g);
}

extern "C" int ofb_last_decode_ms(const openfish_gpubuf_t *gpubuf, float ms[8]) {
    const GpuBuf *g = priv(gpubuf);
    for (int i = 0; i < 8; ++i) ms[i] = g->ms[i];
    return OPENFISH_B200_OK;
}

// Device time of this thread's last rotary call: two events per device, made on first use.
namespace {
constexpr int kMaxDevices = 64;
struct RotaryClock {
    cudaEvent_t ev[kMaxDevices][2] = {};
    bool made[kMaxDevices] = {};
    float last_ms = 0.f;
};
thread_local RotaryClock t_rotary;
}  // namespace

extern "C" int ofb_rotary(void *x, const void *sin_t, const void *cos_t, int batch, int seqlen,
                          int nheads, int rotary_half, long long stride_batch,
                          long long stride_seq, long long stride_head) {
    int dev = 0, sms = 0;
    CU(cudaGetDevice(&dev));
    CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const bool timed = dev >= 0 && dev < kMaxDevices;
    if (timed && !t_rotary.made[dev]) {
        CU(cudaEventCreate(&t_rotary.ev[dev][0]));
        CU(cudaEventCreate(&t_rotary.ev[dev][1]));
        t_rotary.made[dev] = true;
    }
    // the reference launches on the legacy default stream and waits for the device
    // (src/nn_cuda.cu:27-39); same stream here, and a wait on that stream only
    if (timed) CU(cudaEventRecord(t_rotary.ev[dev][0], 0));
    CU(of_launch_rotary(x, sin_t, cos_t, batch, seqlen, nheads, rotary_half, stride_batch,
                        stride_seq, stride_head, sms, 0));
    if (timed) CU(cudaEventRecord(t_rotary.ev[dev][1], 0));
    CU(cudaStreamSynchronize(0));
    t_rotary.last_ms = 0.f;
    if (timed) CU(cudaEventElapsedTime(&t_rotary.last_ms, t_rotary.ev[dev][0], t_rotary.ev[dev][1]));
    return OPENFISH_B200_OK;
}

extern "C" float ofb_last_rotary_ms(void) { return t_rotary.last_ms; }

// ---- helpers for a driver program in the style of the reference's (src/decode_cuda.cu:214-240)
extern "C" int ofb_set_device(int device) {
    CU(cudaSetDevice(device));
    return OPENFISH_B200_OK;
}
extern "C" int ofb_device_upload(const void *host, size_t bytes, void **out) {
    void *d = nullptr;
    CU(cudaMalloc(&d, bytes ? bytes : 1));
    cudaError_t e = cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(d);
        return fail(OPENFISH_B200_ERR_CUDA, "host-to-device copy failed: %s", cudaGetErrorString(e));
    }
    *out = d;
    return OPENFISH_B200_OK;
}
extern "C" int ofb_device_free(void *device) {
    CU(cudaFree(device));
    return OPENFISH_B200_OK;
}
extern "C" int ofb_device_download(void *host, const void *device, size_t bytes) {
    CU(cudaMemcpy(host, device, bytes, cudaMemcpyDeviceToHost));
    return OPENFISH_B200_OK;
}

