/* A plain C99 host program against the C ABI of libsalt_gpu_b200.so, the way the
 * reference's own host code (src/kernels.c:1414, 1558-1567) calls its GPU backend:
 * no C++, no CUDA headers, no Python.  Reads golden cases from a flat file
 *   int32 n_cases; per case: int32 R, C; uint32 vals[R*C/8]; uint16 scales[R*C/64];
 *   uint16 biases[R*C/64]; float x[C]; float y[R]
 * runs salt_gpu_q4_matvec on each and compares the outputs bit for bit.
 * Exit code 0 = all equal. */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "salt_gpu_b200.h"

static void *read_block(FILE *f, size_t bytes) {
    void *p = malloc(bytes ? bytes : 1);
    if (!p || fread(p, 1, bytes, f) != bytes) {
        fprintf(stderr, "short read\n");
        exit(2);
    }
    return p;
}

int main(int argc, char **argv) {
    if (argc < 2) return 2;
    FILE *f = fopen(argv[1], "rb");
    if (!f) return 2;
    int32_t n_cases = 0;
    if (fread(&n_cases, sizeof n_cases, 1, f) != 1) return 2;
    if (salt_gpu_init() != 0) {
        fprintf(stderr, "salt_gpu_init failed (no sm_100 device)\n");
        return 3;
    }
    int bad = 0;
    for (int i = 0; i < n_cases; i++) {
        int32_t rc[2];
        if (fread(rc, sizeof rc, 1, f) != 1) return 2;
        const size_t R = (size_t)rc[0], C = (size_t)rc[1];
        const size_t groups = (R * C + 63) / 64;
        uint32_t *vals = read_block(f, (R * C + 7) / 8 * 4);
        uint16_t *scales = read_block(f, groups * 2);
        uint16_t *biases = read_block(f, groups * 2);
        float *x = read_block(f, C * 4);
        float *want = read_block(f, R * 4);
        float *y = calloc(R, 4);
        if (salt_gpu_q4_matvec(vals, scales, biases, (int)R, (int)C, x, y) != 0) {
            fprintf(stderr, "case %d: salt_gpu_q4_matvec returned an error\n", i);
            bad++;
        } else if (memcmp(y, want, R * 4) != 0) {
            fprintf(stderr, "case %d (%zux%zu): output differs\n", i, R, C);
            bad++;
        }
        free(vals); free(scales); free(biases); free(x); free(want); free(y);
    }
    fclose(f);
    salt_gpu_free();
    printf("%d cases, %d mismatches\n", (int)n_cases, bad);
    return bad ? 1 : 0;
}
