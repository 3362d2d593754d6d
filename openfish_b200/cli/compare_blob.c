/* compare_blob.c -- element-wise comparison of two raw float32 tensor files, reporting what the
 * reference's helper of the same name reports (test/compare_blob.cpp:49-73): the largest and the
 * mean absolute difference, the number of differing elements and the value range of each file.
 *
 *     compare_blob <tens_0.blob> <tens_1.blob>
 *
 * It is how the reference's scripts compare the tensors a debug build dumps (bwd_NTC.blob,
 * post_NTC.blob, qual_data.blob, total_probs.blob ...; scripts/gpu_quick_run.sh:64-73) with stored
 * ones; `openfish --dump` writes the same files.  The report goes to stderr in the reference's
 * format and, for scripts, to stdout as `max_diff avg_diff tens_len n_diffs`.  Exit status 0
 * when the files could be compared (whatever the differences), 1 otherwise. */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

static float *slurp(const char *path, size_t *n_out) {
    FILE *fp = fopen(path, "rb");
    if (!fp) {
        fprintf(stderr, "compare_blob: cannot open %s\n", path);
        exit(1);
    }
    fseek(fp, 0, SEEK_END);
    const long bytes = ftell(fp);
    rewind(fp);
    const size_t n = (size_t)bytes / sizeof(float);
    float *v = (float *)malloc(n ? n * sizeof(float) : 1);
    if (!v || fread(v, sizeof(float), n, fp) != n) {
        fprintf(stderr, "compare_blob: error reading %s\n", path);
        exit(1);
    }
    fclose(fp);
    *n_out = n;
    return v;
}

int main(int argc, char *argv[]) {
    if (argc != 3) {
        fprintf(stderr, "usage: compare_blob <tens_0.blob> <tens_1.blob>\n");
        return 1;
    }
    fprintf(stderr, "comparing files %s and %s\n", argv[1], argv[2]);
    size_t n0 = 0, n1 = 0;
    float *a = slurp(argv[1], &n0), *b = slurp(argv[2], &n1);
    fprintf(stderr, "tens len: %zu\n", n0);
    if (n0 != n1) {
        fprintf(stderr, "file 0 mismatch len with file 1\n");
        return 1;
    }
    float max_diff = 0.0f, lo0 = FLT_MAX, hi0 = -FLT_MAX, lo1 = FLT_MAX, hi1 = -FLT_MAX;
    double sum_diff = 0.0;
    uint64_t n_diff = 0;
    for (size_t i = 0; i < n0; ++i) {
        if (a[i] > hi0) hi0 = a[i];
        if (a[i] < lo0) lo0 = a[i];
        if (b[i] > hi1) hi1 = b[i];
        if (b[i] < lo1) lo1 = b[i];
        const float d = fabsf(a[i] - b[i]);
        if (d != 0.0f) {
            if (d > max_diff) max_diff = d;
            sum_diff += d;
            ++n_diff;
        }
    }
    const float avg_diff = n0 ? (float)(sum_diff / (double)n0) : 0.0f;
    fprintf(stderr, "tensor max elem diff by %.32f, avg diff: %f, tens_len: %zu, n_diffs: %zu\n", max_diff,
            avg_diff, n0, (size_t)n_diff);
    fprintf(stderr, "min_val_0: %.3f, max_val_0: %.3f, min_val_1: %.3f, max_val_1: %.3f\n", lo0, hi0, lo1, hi1);
    printf("%.9g %.9g %zu %zu\n", max_diff, avg_diff, n0, (size_t)n_diff);
    free(a);
    free(b);
    return 0;
}
