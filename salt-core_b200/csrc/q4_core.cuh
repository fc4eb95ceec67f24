// Affine-Q4 (group 64, bf16 scale + bias) projection kernels, bit-exact against
// the reference row DAG (reference src/kernels.c:220-250):
//
//   for c ascending:  d = fl(fl(q*s) + b);  p = fl(d * x[c]);
//                     acc[c & 31] = fl(acc[c & 31] + p)
//   L_j = ((((0 + acc[j]) + acc[j+4]) + ...) + acc[j+28]),  j = 0..3
//   y   = fl(fl(L0 + L2) + fl(L1 + L3))
//
// Thread mapping of the tiled kernel: four lanes share a weight row; lane
// quarter t owns accumulators 8t..8t+7, i.e. exactly the eight nibbles of packed
// word 4i+t of every 32-column step i.  Each lane keeps two weight rows
// (gate + up of the same output row, or rows r and r+8) so the activation
// values it loads are used twice, and TT tokens share one dequantisation.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "bitmath.cuh"

namespace sb {

// One grouped projection job.  ntok activation rows share the weights.
struct Q4Job {
    const uint8_t* vals;     // matrix A: packed nibbles, row-major, C/2 bytes per row
    const uint8_t* scales;   // bf16 [R*C/64]
    const uint8_t* biases;   // bf16 [R*C/64] or null (bias 0)
    const uint8_t* vals2;    // matrix B (fused gate/up: A = gate, B = up) or null
    const uint8_t* scales2;
    const uint8_t* biases2;
    const float* x;          // activation rows
    float* y;                // output rows: y[t*y_stride + r]
    const int* x_rows;       // optional row indirection (length ntok); row = x_rows[t] / x_div
    int x_div;
    int R, C, ntok;
    int x_stride, y_stride;
};

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// Scales whose exponent field is this large can overflow q*s; for those the
// literal two-rounding form is used.  Everywhere else q*s is exact in fp32
// (a 4-bit integer times an 8-bit significand), so fma(q, s, b) has the same
// single rounding as fl(fl(q*s) + b).
__device__ __forceinline__ bool scale_needs_literal(uint32_t sbits16) {
    return (sbits16 & 0x7f80u) >= 0x7c00u;
}

// The eight nibbles of one packed word as exact floats 0..15.  Nibble k is
// masked in place and OR-ed with the exponent of 2^(23-4k'), which makes the
// float equal 2^(23-4k') + q; subtracting that power of two is exact.
__device__ __forceinline__ void nibbles_to_float(uint32_t w, float (&q)[8]) {
    uint32_t hi = w >> 16;
    q[0] = __fsub_rn(__uint_as_float((w & 0x0000000fu) | 0x4b000000u), 8388608.0f);
    q[1] = __fsub_rn(__uint_as_float((w & 0x000000f0u) | 0x49000000u), 524288.0f);
    q[2] = __fsub_rn(__uint_as_float((w & 0x00000f00u) | 0x47000000u), 32768.0f);
    q[3] = __fsub_rn(__uint_as_float((w & 0x0000f000u) | 0x45000000u), 2048.0f);
    q[4] = __fsub_rn(__uint_as_float((hi & 0x0000000fu) | 0x4b000000u), 8388608.0f);
    q[5] = __fsub_rn(__uint_as_float((hi & 0x000000f0u) | 0x49000000u), 524288.0f);
    q[6] = __fsub_rn(__uint_as_float((hi & 0x00000f00u) | 0x47000000u), 32768.0f);
    q[7] = __fsub_rn(__uint_as_float((hi & 0x0000f000u) | 0x45000000u), 2048.0f);
}

__device__ __forceinline__ void dequant8(uint32_t w, float s, float b, bool literal, float (&d)[8]) {
    float q[8];
    nibbles_to_float(w, q);
    if (!literal) {
#pragma unroll
        for (int m = 0; m < 8; m++) d[m] = __fmaf_rn(q[m], s, b);
    } else {
#pragma unroll
        for (int m = 0; m < 8; m++) d[m] = __fadd_rn(__fmul_rn(q[m], s), b);
    }
}

// Canonical fold of one row whose 32 accumulators live 8 per lane in four
// adjacent lanes (quarter t = lane & 3).  The result is valid in the lane with
// t == 3.  The chain runs through the quarters in order: quarter t contributes
// acc[8t + j] then acc[8t + 4 + j] to L_j.
__device__ __forceinline__ float fold_row_quarters(const float (&a)[8], int t) {
    float L0 = 0.0f, L1 = 0.0f, L2 = 0.0f, L3 = 0.0f;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        if (s > 0) {
            L0 = __shfl_up_sync(0xffffffffu, L0, 1, 4);
            L1 = __shfl_up_sync(0xffffffffu, L1, 1, 4);
            L2 = __shfl_up_sync(0xffffffffu, L2, 1, 4);
            L3 = __shfl_up_sync(0xffffffffu, L3, 1, 4);
        }
        if (t == s) {
            L0 = __fadd_rn(__fadd_rn(L0, a[0]), a[4]);
            L1 = __fadd_rn(__fadd_rn(L1, a[1]), a[5]);
            L2 = __fadd_rn(__fadd_rn(L2, a[2]), a[6]);
            L3 = __fadd_rn(__fadd_rn(L3, a[3]), a[7]);
        }
    }
    return __fadd_rn(__fadd_rn(L0, L2), __fadd_rn(L1, L3));
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }

// Wait until at most `pending` of this thread's committed groups are still in flight.
__device__ __forceinline__ void cp_async_wait_dyn(int pending) {
    switch (pending) {
        case 0: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;\n" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;\n" ::: "memory"); break;
        case 6: asm volatile("cp.async.wait_group 6;\n" ::: "memory"); break;
        case 7: asm volatile("cp.async.wait_group 7;\n" ::: "memory"); break;
        case 8: asm volatile("cp.async.wait_group 8;\n" ::: "memory"); break;
        case 9: asm volatile("cp.async.wait_group 9;\n" ::: "memory"); break;
        case 10: asm volatile("cp.async.wait_group 10;\n" ::: "memory"); break;
        case 11: asm volatile("cp.async.wait_group 11;\n" ::: "memory"); break;
        case 12: asm volatile("cp.async.wait_group 12;\n" ::: "memory"); break;
        case 13: asm volatile("cp.async.wait_group 13;\n" ::: "memory"); break;
        case 14: asm volatile("cp.async.wait_group 14;\n" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 15;\n" ::: "memory"); break;
    }
}

}  // namespace sb
