/* openfish_cli.c -- command-line driver with the calling convention of the reference's test
 * program (src/main.c:200-352):
 *
 *     openfish <scores.blob> <BATCH_SIZE> <STATE_LEN> [--timesteps T] [--dump] [--batches K]
 *                                                      [--device D]
 *
 * Reads a raw score tensor [T][N][C], C = 4 * 4^STATE_LEN, either fp16 (the layout the
 * reference's GPU builds read) or fp32 (its CPU builds; converted to fp16 here, exact for
 * values that came from fp16), decodes it on the GPU and writes moves.blob, sequence.blob and
 * qstring.blob (N*T bytes each) into the current directory.  Which of the two element types
 * the file holds follows from its size.  T defaults to 1666 as in the reference.  --dump also
 * writes the gpubuf tensors (bwd_NTC.blob, post_NTC.blob, qual_data.blob, base_probs.blob,
 * total_probs.blob), which the reference does in its debug builds.  --batches repeats the
 * decode K times, as the reference's benchmark build does, and reports the rate.
 *
 * Uses only the C API of libopenfish.so; needs no CUDA header. */
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "openfish/openfish.h"
#include "openfish/openfish_error.h"
#include "openfish_b200.h"

static void die(const char *what, const char *detail) {
    fprintf(stderr, "openfish: %s%s%s\n", what, detail ? ": " : "", detail ? detail : "");
    exit(EXIT_FAILURE);
}

/* IEEE binary32 -> binary16, round to nearest even, overflow to infinity. */
static uint16_t half_from_float(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t mag = x & 0x7fffffffu;
    if (mag >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (mag > 0x7f800000u ? 0x200u : 0u));
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);       /* rounds to >= 65520 */
    if (mag < 0x33000001u) return (uint16_t)sign;                    /* below half of the smallest subnormal */
    int e = (int)(mag >> 23) - 127;
    uint32_t m = (mag & 0x007fffffu) | 0x00800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }                /* subnormal result */
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x007fffffu; }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;          /* may carry into the exponent: correct */
    return (uint16_t)(sign | (base + q));
}

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static void write_blob(const char *path, const void *data, size_t bytes) {
    FILE *fp = fopen(path, "w");
    if (!fp) die(path, strerror(errno));
    if (fwrite(data, 1, bytes, fp) != bytes) die(path, "short write");
    fclose(fp);
}

int main(int argc, char *argv[]) {
    if (argc < 4) {
        fprintf(stderr, "Usage: %s <scores.blob> <BATCH_SIZE> <STATE_LEN> [--timesteps T] [--dump] [--batches K] [--device D]\n",
                argv[0]);
        fprintf(stderr, "e.g. %s hac_scores_TNC_half.blob 512 4\n", argv[0]);
        return EXIT_FAILURE;
    }
    const char *path = argv[1];
    const long N = strtol(argv[2], NULL, 10), state_len = strtol(argv[3], NULL, 10);
    long T = 1666, batches = 1, device = 0;
    int dump = 0;
    for (int i = 4; i < argc; ++i) {
        if (!strcmp(argv[i], "--dump")) dump = 1;
        else if (!strcmp(argv[i], "--timesteps") && i + 1 < argc) T = strtol(argv[++i], NULL, 10);
        else if (!strcmp(argv[i], "--batches") && i + 1 < argc) batches = strtol(argv[++i], NULL, 10);
        else if (!strcmp(argv[i], "--device") && i + 1 < argc) device = strtol(argv[++i], NULL, 10);
        else die("unknown argument", argv[i]);
    }
    if (N <= 0 || T <= 0 || batches <= 0) die("BATCH_SIZE, T and K must be positive", NULL);
    if (state_len < 3 || state_len > 5) die("STATE_LEN must be 3, 4 or 5", NULL);
    const long C = 4L << (2 * state_len);
    const size_t count = (size_t)T * (size_t)N * (size_t)C;

    FILE *fp = fopen(path, "rb");
    if (!fp) die(path, strerror(errno));
    if (fseek(fp, 0, SEEK_END) != 0) die(path, strerror(errno));
    const long long size = ftell(fp);
    rewind(fp);
    uint16_t *scores = malloc(count * sizeof(uint16_t));
    if (!scores) die("out of memory", NULL);
    if ((unsigned long long)size == count * 2ull) {
        if (fread(scores, 2, count, fp) != count) die("error reading score file", path);
    } else if ((unsigned long long)size == count * 4ull) {
        float *row = malloc((size_t)C * sizeof(float));
        if (!row) die("out of memory", NULL);
        for (size_t r = 0; r < (size_t)T * (size_t)N; ++r) {
            if (fread(row, 4, (size_t)C, fp) != (size_t)C) die("error reading score file", path);
            for (long c = 0; c < C; ++c) scores[r * (size_t)C + (size_t)c] = half_from_float(row[c]);
        }
        free(row);
    } else {
        fprintf(stderr, "openfish: %s holds %lld bytes; T=%ld N=%ld C=%ld needs %zu (fp16) or %zu (fp32)\n", path,
                size, T, N, C, count * 2, count * 4);
        return EXIT_FAILURE;
    }
    fclose(fp);

    set_openfish_log_level(OPENFISH_LOG_DBUG);
    set_device_cuda((int)device);
    void *scores_gpu = upload_scores_to_cuda((int)T, (int)N, (int)C, scores);
    openfish_gpubuf_t *gpubuf = openfish_gpubuf_init((int)T, (int)N, (int)state_len);

    /* per-model quality calibration, as the reference's driver applies it (src/main.c:255-265) */
    openfish_opt_t options = DECODER_INIT;
    if (state_len == 3) { options.q_scale = 0.97f; options.q_shift = -1.8f; }
    else if (state_len == 4) { options.q_scale = 0.95f; options.q_shift = -0.2f; }
    else { options.q_scale = 0.95f; options.q_shift = 0.5f; }

    uint8_t *moves = NULL;
    char *sequence = NULL, *qstring = NULL;
    const double t0 = now_s();
    for (long b = 0; b < batches; ++b) {
        if (b) { free(moves); free(sequence); free(qstring); }
        openfish_decode_gpu((int)T, (int)N, (int)C, scores_gpu, (int)state_len, &options, gpubuf, &moves, &sequence,
                            &qstring);
    }
    const double elapsed = now_s() - t0;
    fprintf(stderr, "[openfish] decode completed in %f secs (%ld batch%s of %ld chunks, %.0f chunks/s)\n", elapsed,
            batches, batches == 1 ? "" : "es", N, (double)batches * (double)N / elapsed);

    const size_t out_bytes = (size_t)N * (size_t)T;
    write_blob("moves.blob", moves, out_bytes);
    write_blob("sequence.blob", sequence, out_bytes);
    write_blob("qstring.blob", qstring, out_bytes);
    free(moves);
    free(sequence);
    free(qstring);
    free(scores);
    if (dump) write_gpubuf_cuda((uint64_t)T, (uint64_t)N, (int)state_len, gpubuf);
    openfish_gpubuf_free(gpubuf);
    free_scores_cuda(scores_gpu);
    return 0;
}
