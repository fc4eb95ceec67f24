// Affine-Q4 (group 64, bf16 scale + bias) arithmetic shared by the projection kernels, bit-exact
// against the reference row DAG (reference src/kernels.c:220-250):
//
//   for c ascending:  d = fl(fl(q*s) + b);  p = fl(d * x[c]);
//                     acc[c & 31] = fl(acc[c & 31] + p)
//   L_j = ((((0 + acc[j]) + acc[j+4]) + ...) + acc[j+28]),  j = 0..3
//   y   = fl(fl(L0 + L2) + fl(L1 + L3))
//
// Thread mapping: sixteen adjacent lanes share a weight row; lane v = tid & 15 owns the
// accumulators 2v and 2v + 1, i.e. the two nibbles of byte v of every 32-column step (16 packed
// bytes), so "accumulator c mod 32, columns ascending" is a sequential loop per lane and the
// canonical fold is a chain through the sixteen lanes.  Each lane keeps two weight rows (gate +
// up of the same output row, or two rows of one matrix) so the activation values it loads are
// used twice, and TT tokens share one dequantisation.  Dequantisation and the products are
// issued as sm_100 packed pairs (add/mul/fma.rn.f32x2): each half of a pair is an independent
// IEEE round-to-nearest operation.
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

// ---- packed fp32 pairs -------------------------------------------------
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 pack2u(uint32_t lo, uint32_t hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Exponent patterns of 2^23, 2^19, 2^15, 2^11.  They are read from constant
// memory into registers on purpose: with the pattern in a register and the
// nibble mask as the immediate, "(h & mask) | pattern" is ONE three-input
// logic operation; written with two literals the compiler emits two.
__constant__ uint32_t c_nibble_magic[4] = {0x4b000000u, 0x49000000u, 0x47000000u, 0x45000000u};

// -0.0f, kept out of the compiler's sight (see product_then_add).
__constant__ uint32_t c_neg_zero = 0x80000000u;

struct NibbleMagic {
    uint32_t m0, m1, m2, m3;
};
__device__ __forceinline__ NibbleMagic load_nibble_magic() {
    NibbleMagic m;
    m.m0 = c_nibble_magic[0]; m.m1 = c_nibble_magic[1]; m.m2 = c_nibble_magic[2]; m.m3 = c_nibble_magic[3];
    return m;
}

// acc = fl(acc + fl(d * x)) on register pairs.  ptxas contracts a packed multiply followed
// by a packed add (and even a packed fma with a multiplier of 1) into one fused
// multiply-add, which changes the last bit.  The product is therefore formed as
// fma(d, x, -0): adding -0 leaves every product, signed zeros included, unchanged, a fused
// multiply-add cannot be merged into the following add, and the -0 comes from constant
// memory so that the compiler cannot simplify the fma back into a multiply.
__device__ __forceinline__ void product_then_add(f32x2& acc, f32x2 d, f32x2 x, f32x2 negzero) {
    acc = add2(acc, fma2(d, x, negzero));
}

// ---- the tile kernel: 16 lanes per row ----------------------------------------------
// A row's 32 accumulators are spread over sixteen adjacent lanes (lane v = tid & 15 holds
// acc[2v], acc[2v + 1], i.e. one packed byte per 32-column step).  An earlier form with eight
// lanes per row (four accumulators each, half the warps) ran decode at the same speed and
// batches of 64 tokens 1.4x slower.

// One packed byte (two nibbles) as exact floats.
template <bool LIT>
__device__ __forceinline__ f32x2 dequant2(uint32_t b, const NibbleMagic& mg, f32x2 ss, f32x2 bb) {
    const f32x2 neg01 = pack2(-8388608.0f, -524288.0f);
    uint32_t f0, f1;
    asm("lop3.b32 %0, %1, 0x0f, %2, 0xEA;" : "=r"(f0) : "r"(b), "r"(mg.m0));
    asm("lop3.b32 %0, %1, 0xf0, %2, 0xEA;" : "=r"(f1) : "r"(b), "r"(mg.m1));
    const f32x2 q = add2(pack2u(f0, f1), neg01);
    if (LIT) {
        float p0, p1, b0, b1;
        unpack2(mul2(q, ss), p0, p1);
        unpack2(bb, b0, b1);
        return pack2(__fadd_rn(p0, b0), __fadd_rn(p1, b1));
    }
    return fma2(q, ss, bb);
}

template <int TT, bool LIT, int NSTEPS>
__device__ __forceinline__ void tile16_steps(const NibbleMagic& mg, const uint8_t* wA, const uint8_t* wB,
                                             const uint32_t* tA, const uint32_t* tB, const float* const (&xs)[TT],
                                             f32x2 (&accA)[TT], f32x2 (&accB)[TT], f32x2 nz) {
#pragma unroll
    for (int g = 0; g < NSTEPS / 2; g++) {
        const uint32_t wa = tA[g], wb = tB[g];
        const float sa = __uint_as_float(wa & 0xffff0000u), ba = __uint_as_float(wa << 16);
        const float sb_ = __uint_as_float(wb & 0xffff0000u), bb_ = __uint_as_float(wb << 16);
        const f32x2 ssA = pack2(sa, sa), bbA = pack2(ba, ba), ssB = pack2(sb_, sb_), bbB = pack2(bb_, bb_);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int k = 2 * g + half;
            const f32x2 dA = dequant2<LIT>(wA[k * 16], mg, ssA, bbA);
            const f32x2 dB = dequant2<LIT>(wB[k * 16], mg, ssB, bbB);
#pragma unroll
            for (int tt = 0; tt < TT; tt++) {
                const f32x2 xv = *(const f32x2*)(xs[tt] + k * 32);
                product_then_add(accA[tt], dA, xv, nz);
                product_then_add(accB[tt], dB, xv, nz);
            }
        }
    }
}

template <int TT, bool LIT>
__device__ __forceinline__ void tile16_run(const NibbleMagic& mg, int s_begin, int s_end, const uint8_t* wA,
                                           const uint8_t* wB, const uint32_t* tA, const uint32_t* tB,
                                           const float* sX, int x_pitch, f32x2 (&accA)[TT], f32x2 (&accB)[TT],
                                           f32x2 nz) {
    int st = s_begin;
    constexpr int BLK = 8;
    for (; st + BLK <= s_end; st += BLK) {
        const float* xs[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) xs[tt] = sX + tt * x_pitch + st * 32;
        tile16_steps<TT, LIT, BLK>(mg, wA + st * 16, wB + st * 16, tA + (st >> 1), tB + (st >> 1), xs, accA, accB, nz);
    }
    for (; st + 2 <= s_end; st += 2) {
        const float* xs[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) xs[tt] = sX + tt * x_pitch + st * 32;
        tile16_steps<TT, LIT, 2>(mg, wA + st * 16, wB + st * 16, tA + (st >> 1), tB + (st >> 1), xs, accA, accB, nz);
    }
}

// Canonical fold (src/kernels.c:240-250) of a row whose accumulators sit two per lane in
// sixteen adjacent lanes: L_j = sum over a = 0..7 of acc[4a + j], added in that order from
// +0, then y = (L0 + L2) + (L1 + L3).  acc[4a + j] is component j & 1 of lane 2a + (j >> 1).
// mask: the lanes that take part (the whole warp, or the row's own sixteen lanes when the two
// halves of a warp may run different code).
__device__ __forceinline__ float fold_row_hexadecants(f32x2 acc, int v, uint32_t mask = 0xffffffffu) {
    float lo, hi;
    unpack2(acc, lo, hi);
    const int j = v & 3;
    const int base = (threadIdx.x & 31) & ~15;
    float L = 0.0f;
#pragma unroll
    for (int a = 0; a < 8; a++) {
        const int src = base + 2 * a + (j >> 1);
        const float vlo = __shfl_sync(mask, lo, src);
        const float vhi = __shfl_sync(mask, hi, src);
        L = __fadd_rn(L, (j & 1) ? vhi : vlo);
    }
    const float L0 = __shfl_sync(mask, L, base + 0);
    const float L1 = __shfl_sync(mask, L, base + 1);
    const float L2 = __shfl_sync(mask, L, base + 2);
    const float L3 = __shfl_sync(mask, L, base + 3);
    return __fadd_rn(__fadd_rn(L0, L2), __fadd_rn(L1, L3));
}

// The four nibbles of one packed half-word as exact floats 0..15, as two pairs.
// Nibble k is masked in place and OR-ed with the exponent of 2^(23-4k), which
// makes the float equal 2^(23-4k) + q; adding -2^(23-4k) is exact.
__device__ __forceinline__ void nibbles4(uint32_t h, const NibbleMagic& mg, f32x2& q01, f32x2& q23) {
    const f32x2 neg01 = pack2(-8388608.0f, -524288.0f);
    const f32x2 neg23 = pack2(-32768.0f, -2048.0f);
    uint32_t f0, f1, f2, f3;
    asm("lop3.b32 %0, %1, 0x000f, %2, 0xEA;" : "=r"(f0) : "r"(h), "r"(mg.m0));
    asm("lop3.b32 %0, %1, 0x00f0, %2, 0xEA;" : "=r"(f1) : "r"(h), "r"(mg.m1));
    asm("lop3.b32 %0, %1, 0x0f00, %2, 0xEA;" : "=r"(f2) : "r"(h), "r"(mg.m2));
    asm("lop3.b32 %0, %1, 0xf000, %2, 0xEA;" : "=r"(f3) : "r"(h), "r"(mg.m3));
    q01 = add2(pack2u(f0, f1), neg01);
    q23 = add2(pack2u(f2, f3), neg23);
}

// Canonical fold of one row whose 32 accumulators live 4 per lane in eight
// adjacent lanes (octant u = lane & 7; lane holds acc[4u + j], j = 0..3).
// Lane u of the octet gathers acc[4s + (u & 3)] from octant s = 0..7 in order and
// runs the chain L_j = (((0 + acc[j]) + acc[4 + j]) + ...) for j = u & 3 (lanes
// 4..7 repeat lanes 0..3); the four L values are then combined as
// (L0 + L2) + (L1 + L3).  The result is valid in every lane of the octet.
// mask: the lanes that take part (the whole warp, or the row's own eight lanes).
__device__ __forceinline__ float fold_row_octants(const float (&a)[4], int u, uint32_t mask = 0xffffffffu) {
    const int j = u & 3;
    const int base = (threadIdx.x & 31) & ~7;
    float L = 0.0f;
#pragma unroll
    for (int s = 0; s < 8; s++) {
        // every lane offers all four of its accumulators; the reader picks column j of octant s
        const float v0 = __shfl_sync(mask, a[0], base + s);
        const float v1 = __shfl_sync(mask, a[1], base + s);
        const float v2 = __shfl_sync(mask, a[2], base + s);
        const float v3 = __shfl_sync(mask, a[3], base + s);
        const float v = j == 0 ? v0 : (j == 1 ? v1 : (j == 2 ? v2 : v3));
        L = __fadd_rn(L, v);
    }
    const float L0 = __shfl_sync(mask, L, base + 0);
    const float L1 = __shfl_sync(mask, L, base + 1);
    const float L2 = __shfl_sync(mask, L, base + 2);
    const float L3 = __shfl_sync(mask, L, base + 3);
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
