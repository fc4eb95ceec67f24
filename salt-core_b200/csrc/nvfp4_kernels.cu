// NVFP4 (E2M1 codes, one E4M3FN scale per 16 elements, per-tensor fp32 scalars)
// kernels, bit-exact against the reference src/nvfp4.c:
//
//   nvfp4_qdq_kernel     dynamic group-16 activation quantise -> dequantise
//                        (salt_nvfp4_quantize_input_reference, nvfp4.c:82-130)
//   nvfp4_tile_kernel    W4A4 projection on the dequantised activations with the
//                        canonical 32-accumulator order (nvfp4.c:173-192, 157-171)
//   nvfp4_generic_kernel any C that is a multiple of 16
//
// The encoders are arithmetic instead of the reference's nearest-code searches:
// "nearest, ties to the even code" over a monotone code table is round-to-
// nearest-even in that format (checked against the searches in the tests).
#include <algorithm>

#include "internal.h"
#include "pdl.cuh"
#include "q4_core.cuh"

namespace sb {

static __device__ __forceinline__ void flag_status(int* status, int bit) {
    if (status) atomicOr(status, bit);
}

// E4M3FN decode (nvfp4.c:25-39) for the finite codes.
__device__ __forceinline__ float e4m3_decode(uint32_t code) {
    const uint32_t ex = (code >> 3) & 15u, man = code & 7u;
    float v;
    if (ex == 0) v = __fmul_rn((float)man, 0.001953125f);
    else if (ex == 15 && man == 7) v = __int_as_float(0x7fc00000);
    else v = __uint_as_float(((ex + 120u) << 23) | (man << 20));
    return (code & 0x80u) ? -v : v;
}

// E4M3FN encode of a finite value in [0, 448] (nvfp4.c:41-63): nearest code,
// ties to the even code.
__device__ __forceinline__ uint32_t e4m3_encode_pos(float v) {
    if (v < 0.015625f) return (uint32_t)__float2int_rn(__fmul_rn(v, 512.0f));  // subnormal grid 2^-9
    uint32_t b = __float_as_uint(v);
    b = (b + 0x7ffffu + ((b >> 20) & 1u)) >> 20;   // round to 3 mantissa bits, ties to even
    return (((b >> 3) - 120u) << 3) | (b & 7u);
}

// E2M1 encode of a value already clamped to [-6, 6] (nvfp4.c:65-80): magnitudes
// {0, .5, 1, 1.5, 2, 3, 4, 6}; on a tie the even code wins.
__device__ __forceinline__ uint32_t e2m1_encode(float t) {
    const float m = fabsf(t);
    uint32_t c = (m > 0.25f) + (m >= 0.75f) + (m > 1.25f) + (m >= 1.75f) + (m > 2.5f) + (m >= 3.5f) + (m > 5.0f);
    if (__float_as_uint(t) & 0x80000000u) c |= 8u;
    return c;
}

// E2M1 decode (nvfp4.c:19-23): both zero codes give +0.
__device__ __forceinline__ float e2m1_decode(uint32_t code) {
    const uint32_t e = (code >> 1) & 3u, m = code & 1u;
    float v = e == 0 ? (m ? 0.5f : 0.0f) : __uint_as_float(((e + 126u) << 23) | (m << 22));
    if (v == 0.0f) return 0.0f;
    return (code & 8u) ? -v : v;
}

// One thread per block of 16 activations.  ig_rows[row] is the row's input
// global scale.  Non-finite activations set the status word (the reference
// function returns -1).
// src_rows != null: row r of the call reads activation row src_rows[r % src_mod] / src_div (the grouped
// order of a MoE layer: several quantisations of the same token row with different global scales).
// GEGLU: the activations are formed on the fly as gelu_tanh(x[i]) * up[i] (reference gemma4.c:80-83 and the
// product of gemma4_text.c:8927-8930) - the quantiser of a layer's second projection batch needs no GeGLU buffer.
template <bool WANT_DQ, bool GEGLU>
__global__ void __launch_bounds__(512)
nvfp4_qdq_kernel(const float* __restrict__ x, const float* __restrict__ up, int rows, int C,
                 const float* __restrict__ ig_rows, uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                 float* __restrict__ dequant, int* status, const int* __restrict__ src_rows, int src_mod, int src_div) {
    // blocks (x, y): row x, 16-element blocks y * blockDim.x + thread; the row's source and scale are found once
    pdl_wait();                    // scales, row table and activations come from the kernels before this one
    pdl_launch_dependents();
    const int bpr = C >> 4;
    const int row = blockIdx.x;
    const float ig = ig_rows[row];
    if (!(ig > 0.0f)) return;         // a row nobody will read (its expert lives on another rank): its source may be unwritten
    const int in_row = src_rows ? src_rows[row % src_mod] / src_div : row;
    for (int blk = blockIdx.y * blockDim.x + threadIdx.x; blk < bpr; blk += gridDim.y * blockDim.x) {
        const float4* in4 = (const float4*)(x + (size_t)in_row * C + blk * 16);
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 t = in4[i];
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
        if (GEGLU) {
            const float4* up4 = (const float4*)(up + (size_t)in_row * C + blk * 16);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float4 t = up4[i];
                v[4 * i] = __fmul_rn(gelu_tanh_exact(v[4 * i]), t.x);
                v[4 * i + 1] = __fmul_rn(gelu_tanh_exact(v[4 * i + 1]), t.y);
                v[4 * i + 2] = __fmul_rn(gelu_tanh_exact(v[4 * i + 2]), t.z);
                v[4 * i + 3] = __fmul_rn(gelu_tanh_exact(v[4 * i + 3]), t.w);
            }
        }
        float amax = 0.0f;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float m = fabsf(v[i]);
            bad |= !finite_f(m);
            if (m > amax) amax = m;
        }
        if (bad) {
            flag_status(status, SB_ERR_NONFINITE);
            continue;
        }
        float raw = __fmul_rn(ig, __fmul_rn(amax, 0.16666667163372039794921875f));
        if (raw > 448.0f) raw = 448.0f;
        const uint32_t sc = e4m3_encode_pos(raw);
        const float scale = e4m3_decode(sc);
        const float out_scale = scale == 0.0f ? 0.0f : __fdiv_rn(ig, scale);
        const float dq_scale = WANT_DQ ? __fdiv_rn(scale, ig) : 0.0f;
        uint32_t lo = 0, hi = 0;
        float dq[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            float t = __fmul_rn(v[i], out_scale);
            if (t > 6.0f) t = 6.0f;
            if (t < -6.0f) t = -6.0f;
            const uint32_t c = e2m1_encode(t);
            if (WANT_DQ) dq[i] = __fmul_rn(e2m1_decode(c), dq_scale);
            if (i < 8) lo |= c << (4 * i);
            else hi |= c << (4 * (i - 8));
        }
        scales[(size_t)row * bpr + blk] = (uint8_t)sc;
        *(uint2*)(packed + (size_t)row * (C >> 1) + blk * 8) = make_uint2(lo, hi);
        if (WANT_DQ) {
            float4* out4 = (float4*)(dequant + (size_t)row * C + blk * 16);
#pragma unroll
            for (int i = 0; i < 4; i++) out4[i] = make_float4(dq[4 * i], dq[4 * i + 1], dq[4 * i + 2], dq[4 * i + 3]);
        }
    }
}

cudaError_t launch_nvfp4_qdq(const float* x, int rows, int C, const float* ig_rows, uint8_t* packed, uint8_t* scales,
                             float* dequant, int* status, cudaStream_t stream, const int* src_rows, int src_mod,
                             int src_div, const float* geglu_up) {
    if (rows < 1) return cudaSuccess;
    if (src_rows && (src_mod < 1 || src_div < 1 || geglu_up)) return cudaErrorInvalidValue;
    const int bpr = C >> 4;
    const int threads = bpr >= 512 ? 512 : ((bpr + 31) & ~31);
    const dim3 grid((unsigned)rows, (unsigned)std::min(65535, (bpr + threads - 1) / threads));
#define SB_QDQ(DQ, GG) \
    launch_pdl(nvfp4_qdq_kernel<DQ, GG>, grid, dim3(threads), 0, stream, x, geglu_up, rows, C, ig_rows, packed, scales, \
               dequant, status, src_rows, src_mod, src_div)
    if (dequant) return geglu_up ? SB_QDQ(true, true) : SB_QDQ(true, false);
    return geglu_up ? SB_QDQ(false, true) : SB_QDQ(false, false);     // the tensor-core consumer reads codes and scales only
#undef SB_QDQ
}

// Four E2M1 codes of one half-word as floats, by the hardware conversion (two codes -> f16x2, exact: every E2M1
// value is an f16).  It decodes the code 8 as -0 where the reference's table has +0 (src/nvfp4.c:19-23): as a
// WEIGHT that cannot change a result - the product is a zero of either sign, and an accumulator that starts
// at +0 never becomes -0 (x + (-0) = x, +0 + (-0) = +0) - so the dot-product kernels may use it; the
// quantise-dequantise kernel, whose decoded values are output, keeps the table form.
__device__ __forceinline__ void e2m1x4(uint32_t h, f32x2& w01, f32x2& w23) {
    uint32_t p0, p1;
    asm("{ .reg .b8 b0, b1;\n\t"
        "mov.b16 {b0, b1}, %2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1; }\n"
        : "=r"(p0), "=r"(p1)
        : "h"((unsigned short)h));
    float f0, f1, f2, f3;
    asm("{ .reg .b16 l, u;\n\t"
        "mov.b32 {l, u}, %2;\n\t"
        "cvt.f32.f16 %0, l;\n\t"
        "cvt.f32.f16 %1, u; }\n"
        : "=f"(f0), "=f"(f1)
        : "r"(p0));
    asm("{ .reg .b16 l, u;\n\t"
        "mov.b32 {l, u}, %2;\n\t"
        "cvt.f32.f16 %0, l;\n\t"
        "cvt.f32.f16 %1, u; }\n"
        : "=f"(f2), "=f"(f3)
        : "r"(p1));
    w01 = pack2(f0, f1);
    w23 = pack2(f2, f3);
}

// Tile kernel: 16 weight rows per block, eight lanes per row, lane octant u owns accumulators
// 4u..4u+3 (same mapping as the Q4 kernel).  RPL = rows per lane group: 2 (64 threads, lane rows r and r + 8:
// one activation load serves two rows - batches) or 1 (128 threads: twice the warps on the same shared
// memory, which is what a one-token pass, bound by latency, wants).
// Requires C % 256 == 0 and 16-byte aligned operands.
template <int TT, int RPL>
__global__ void __launch_bounds__(128 / RPL)
nvfp4_tile_kernel(const Fp4Job* __restrict__ jobs, int C, const int* __restrict__ live, const int* __restrict__ n_live) {
    constexpr int NTH = 128 / RPL;
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_wait();                    // jobs, live list and activations come from the kernels before this one
    pdl_launch_dependents();
    // with a list of the jobs that have tokens the grid only spans those (a decode step touches 4 of 64 experts)
    if (live != nullptr && (int)blockIdx.y >= *n_live) return;
    const Fp4Job jb = jobs[live != nullptr ? live[blockIdx.y] : blockIdx.y];
    const int r0 = blockIdx.x * 16;
    if (r0 >= jb.R || jb.ntok < 1) return;
    const int tid = threadIdx.x, u = tid & 7, pr = tid >> 3;
    const int nvalid = min(16, jb.R - r0);
    const int row_bytes = C >> 1, w_stride = row_bytes + 16;
    const int sc_row = C >> 4, sc_stride = sc_row + 16;
    const int steps = C >> 5;
    int chunk_steps = 8, nch = (steps + 7) / 8;
    if (nch > 15) {
        chunk_steps = (((steps + 14) / 15) + 1) & ~1;
        nch = (steps + chunk_steps - 1) / chunk_steps;
    }
    uint8_t* sW = smem;                                 // [16][w_stride]
    uint8_t* sS = sW + 16 * w_stride;                   // [16][sc_stride]
    float* sTbl = (float*)(sS + 16 * sc_stride);        // [256] fl(e4m3(code) * wg)
    float* sX = sTbl + 256;                             // [TT][C]

    auto issue_x = [&](int tb) {
        const int ppr = C >> 2;
        for (int p = tid; p < TT * ppr; p += NTH) {
            const int tt = p / ppr, pc = p - tt * ppr;
            const int tok = min(tb + tt, jb.ntok - 1);
            cp_async16(sX + tt * C + pc * 4, jb.x + (size_t)tok * jb.x_stride + pc * 4);
        }
    };
    issue_x(0);
    {
        const int ppr = sc_row >> 4;
        for (int p = tid; p < nvalid * ppr; p += NTH) {
            const int rr = p / ppr, pc = p - rr * ppr;
            cp_async16(sS + rr * sc_stride + pc * 16, jb.scales + (size_t)(r0 + rr) * sc_row + pc * 16);
        }
    }
    for (int ch = 0; ch < nch; ch++) {
        const int s_begin = ch * chunk_steps;
        const int cs = min(chunk_steps, steps - s_begin);
        for (int p = tid; p < 16 * cs; p += NTH) {
            const int rr = p / cs, pc = p - rr * cs;
            const int grow = min(r0 + rr, jb.R - 1);
            cp_async16(sW + rr * w_stride + (s_begin + pc) * 16,
                       jb.codes + (size_t)grow * row_bytes + (s_begin + pc) * 16);
        }
        cp_async_commit();
    }
    for (int c = tid; c < 256; c += NTH) sTbl[c] = __fmul_rn(e4m3_decode((uint32_t)c), jb.wg);

    const uint8_t* wA = sW + pr * w_stride + 2 * u;
    const uint8_t* wB = sW + (RPL == 2 ? pr + 8 : pr) * w_stride + 2 * u;
    const uint8_t* scA = sS + pr * sc_stride + (u >> 2);
    const uint8_t* scB = sS + (RPL == 2 ? pr + 8 : pr) * sc_stride + (u >> 2);
    const float* xs = sX + 4 * u;
    const f32x2 nz = pack2u(c_neg_zero, c_neg_zero);

    for (int tb = 0; tb < jb.ntok; tb += TT) {
        if (tb > 0) {
            __syncthreads();
            issue_x(tb);
            cp_async_commit();
            cp_async_wait_dyn(0);
            __syncthreads();
        }
        // accumulators 4u .. 4u + 3 of each row as two packed pairs (add.rn.f32x2 = two independent roundings)
        f32x2 accA[TT][2], accB[TT][2];
#pragma unroll
        for (int tt = 0; tt < TT; tt++)
#pragma unroll
            for (int j = 0; j < 2; j++) { accA[tt][j] = pack2(0.0f, 0.0f); accB[tt][j] = pack2(0.0f, 0.0f); }
        for (int ch = 0; ch < nch; ch++) {
            if (tb == 0) {
                cp_async_wait_dyn(nch - 1 - ch);
                __syncthreads();
            }
            const int s_begin = ch * chunk_steps;
            const int s_end = min(s_begin + chunk_steps, steps);
#pragma unroll 2
            for (int st = s_begin; st < s_end; st++) {
                const float sa = sTbl[scA[2 * st]];
                const uint32_t hA = *(const uint16_t*)(wA + st * 16);
                f32x2 a01, a23, b01, b23;
                e2m1x4(hA, a01, a23);
                const f32x2 ssa = pack2(sa, sa);
                a01 = mul2(a01, ssa); a23 = mul2(a23, ssa);
                if (RPL == 2) {
                    const float sb_ = sTbl[scB[2 * st]];
                    const uint32_t hB = *(const uint16_t*)(wB + st * 16);
                    e2m1x4(hB, b01, b23);
                    const f32x2 ssb = pack2(sb_, sb_);
                    b01 = mul2(b01, ssb); b23 = mul2(b23, ssb);
                }
#pragma unroll
                for (int tt = 0; tt < TT; tt++) {
                    const ulonglong2 xv = *(const ulonglong2*)(xs + tt * C + st * 32);
                    // the product as fma(w, x, -0): exactly fl(w * x), and an add that the assembler cannot
                    // contract with it into one fused multiply-add (it would with a plain mul.f32x2)
                    accA[tt][0] = add2(accA[tt][0], fma2(a01, xv.x, nz));
                    accA[tt][1] = add2(accA[tt][1], fma2(a23, xv.y, nz));
                    if (RPL == 2) {
                        accB[tt][0] = add2(accB[tt][0], fma2(b01, xv.x, nz));
                        accB[tt][1] = add2(accB[tt][1], fma2(b23, xv.y, nz));
                    }
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            float fa[4], fb[4];
            unpack2(accA[tt][0], fa[0], fa[1]); unpack2(accA[tt][1], fa[2], fa[3]);
            unpack2(accB[tt][0], fb[0], fb[1]); unpack2(accB[tt][1], fb[2], fb[3]);
            const float y0 = fold_row_octants(fa, u);
            const float y1 = RPL == 2 ? fold_row_octants(fb, u) : 0.0f;
            const int tok = tb + tt;
            if (u == 7 && tok < jb.ntok) {
                float* yrow = jb.y + (size_t)tok * jb.y_stride;
                if (pr < nvalid) yrow[r0 + pr] = y0;
                if (RPL == 2 && pr + 8 < nvalid) yrow[r0 + pr + 8] = y1;
            }
        }
    }
}

// Any C (multiple of 16), any alignment: one warp per (row, token), lane l owns
// accumulator l.
__global__ void __launch_bounds__(128)
nvfp4_generic_kernel(const Fp4Job* __restrict__ jobs, const int* __restrict__ live, const int* __restrict__ n_live) {
    if (live != nullptr && (int)blockIdx.z >= *n_live) return;
    const Fp4Job jb = jobs[live != nullptr ? live[blockIdx.z] : blockIdx.z];
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5), tok = blockIdx.y;
    if (r >= jb.R || tok >= jb.ntok) return;
    const int lane = threadIdx.x & 31;
    const float* x = jb.x + (size_t)tok * jb.x_stride;
    float acc = 0.0f;
    for (int c = lane; c < jb.C; c += 32) {
        const size_t k = (size_t)r * jb.C + c;
        const uint8_t byte = jb.codes[k >> 1];
        const uint32_t code = (k & 1) ? (byte >> 4) : (byte & 15u);
        const float sc = __fmul_rn(e4m3_decode(jb.scales[(size_t)r * (jb.C >> 4) + (c >> 4)]), jb.wg);
        const float w = __fmul_rn(e2m1_decode(code), sc);
        acc = __fadd_rn(acc, __fmul_rn(w, x[c]));
    }
    float L = 0.0f;
#pragma unroll
    for (int a = 0; a < 8; a++) L = __fadd_rn(L, __shfl_sync(0xffffffffu, acc, (lane & 3) + 4 * a));
    const float L2 = __shfl_sync(0xffffffffu, L, 2);
    const float L1 = __shfl_sync(0xffffffffu, L, 1);
    const float L3 = __shfl_sync(0xffffffffu, L, 3);
    if (lane == 0) jb.y[(size_t)tok * jb.y_stride + r] = __fadd_rn(__fadd_rn(L, L2), __fadd_rn(L1, L3));
}

// ---- a MoE layer of NVFP4 experts (reference caller: models/gemma4-26b-a4b/src/gemma4_text.c:8912-8945,
// two projection batches with the GeGLU between them) ------------------------------------------------
// One thread per expert: the projection jobs of its token group and the input global scale of every
// grouped row (gate rows [0, J), up rows [J, 2J) of the gathered activations; down rows [0, J)).
static __device__ __forceinline__ void
nvfp4_plan_expert(int e, const int* __restrict__ group_offsets, int E, int expert_begin, int expert_end, int J,
                  const Fp4ExpertDesc* __restrict__ experts, int H, int M, const float* dq_gu, float* gate_out,
                  float* up_out, const float* dq_dn, float* grouped_out, Fp4Job* gu_jobs, Fp4Job* dn_jobs, float* ig_gu,
                  float* ig_dn, Fp4TcJob* tc_gu, Fp4TcJob* tc_dn, int* live, int* n_gu, int* n_dn);

__global__ void __launch_bounds__(128)
nvfp4_moe_plan_kernel(const int* __restrict__ group_offsets, int E, int expert_begin, int expert_end, int J,
                      const Fp4ExpertDesc* __restrict__ experts, int H, int M, const float* dq_gu, float* gate_out,
                      float* up_out, const float* dq_dn, float* grouped_out, Fp4Job* gu_jobs, Fp4Job* dn_jobs,
                      float* ig_gu, float* ig_dn, Fp4TcJob* tc_gu, Fp4TcJob* tc_dn, int* live) {
    // live (optional): [0] / [1] = number of gate|up / down jobs with tokens, then their indices ([2, 2 + 2E)
    // into gu_jobs, [2 + 2E, 2 + 3E) into dn_jobs) so the projection launches span only those
    __shared__ int n_gu, n_dn;
    if (threadIdx.x == 0) n_gu = n_dn = 0;
    pdl_wait();                    // the group offsets come from the plan kernel before this one
    pdl_launch_dependents();
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        nvfp4_plan_expert(e, group_offsets, E, expert_begin, expert_end, J, experts, H, M, dq_gu, gate_out, up_out, dq_dn,
                          grouped_out, gu_jobs, dn_jobs, ig_gu, ig_dn, tc_gu, tc_dn, live, &n_gu, &n_dn);
    __syncthreads();
    if (threadIdx.x == 0 && live != nullptr) {
        live[0] = n_gu;
        live[1] = n_dn;
    }
}

static __device__ __forceinline__ void
nvfp4_plan_expert(int e, const int* __restrict__ group_offsets, int E, int expert_begin, int expert_end, int J,
                  const Fp4ExpertDesc* __restrict__ experts, int H, int M, const float* dq_gu, float* gate_out,
                  float* up_out, const float* dq_dn, float* grouped_out, Fp4Job* gu_jobs, Fp4Job* dn_jobs, float* ig_gu,
                  float* ig_dn, Fp4TcJob* tc_gu, Fp4TcJob* tc_dn, int* live, int* n_gu, int* n_dn) {
    const int g0 = group_offsets[e], cnt = group_offsets[e + 1] - g0;
    const bool local = e >= expert_begin && e < expert_end;
    Fp4ExpertDesc d;
    if (local) d = experts[e - expert_begin];
    Fp4Job j;
    j.R = M; j.C = H; j.ntok = local ? cnt : 0; j.x_stride = H; j.y_stride = M;
    j.codes = local ? d.codes[0] : nullptr; j.scales = local ? d.scales[0] : nullptr; j.wg = local ? d.wg[0] : 0.0f;
    j.x = dq_gu + (size_t)g0 * H; j.y = gate_out + (size_t)g0 * M;
    gu_jobs[e] = j;
    j.codes = local ? d.codes[1] : nullptr; j.scales = local ? d.scales[1] : nullptr; j.wg = local ? d.wg[1] : 0.0f;
    j.x = dq_gu + (size_t)(J + g0) * H; j.y = up_out + (size_t)g0 * M;
    gu_jobs[E + e] = j;
    j.R = H; j.C = M; j.x_stride = M; j.y_stride = H;
    j.codes = local ? d.codes[2] : nullptr; j.scales = local ? d.scales[2] : nullptr; j.wg = local ? d.wg[2] : 0.0f;
    j.x = dq_dn + (size_t)g0 * M; j.y = grouped_out + (size_t)g0 * H;
    dn_jobs[e] = j;
    if (live != nullptr && local && cnt > 0) {
        const int i = atomicAdd(n_gu, 2);
        live[2 + i] = e;
        live[3 + i] = E + e;
        live[2 + 2 * E + atomicAdd(n_dn, 1)] = e;
    }
    if (tc_gu) {
        // the same jobs for the tensor-core kernel: the up matrix follows the gate codes (M rows) and the gate
        // scales (M / 8 rows of H / 2 bytes) in the expert's slot; the quantised activations' block scales
        // use the rows of the packed codes (gate [0, J), up [J, 2J); down [0, J) after the second quantisation);
        // scale rows are C / 16 bytes long: in those units the up scales start 9 M rows (one tensor) after the
        // gate scales
        Fp4TcJob t;
        t.ntok = local ? cnt : 0; t.w_slice = local ? e - expert_begin : 0;
        t.R = M; t.y_stride = M; t.w_row0 = 0; t.ws_row0 = 0; t.x_row0 = g0;
        t.wg = local ? d.wg[0] : 0.0f; t.ig = local ? d.ig[0] : 1.0f; t.y = gate_out + (size_t)g0 * M;
        tc_gu[e] = t;
        t.w_row0 = M + (M >> 3); t.ws_row0 = 9 * M; t.x_row0 = J + g0;
        t.wg = local ? d.wg[1] : 0.0f; t.ig = local ? d.ig[1] : 1.0f; t.y = up_out + (size_t)g0 * M;
        tc_gu[E + e] = t;
        t.R = H; t.y_stride = H; t.w_row0 = 0; t.ws_row0 = 0; t.x_row0 = g0;
        t.wg = local ? d.wg[2] : 0.0f; t.ig = local ? d.ig[2] : 1.0f; t.y = grouped_out + (size_t)g0 * H;
        tc_dn[e] = t;
    }
    for (int t = 0; t < cnt; t++) {                   // rows of remote experts are marked (scale 0) and skipped by the quantiser
        ig_gu[g0 + t] = local ? d.ig[0] : 0.0f;
        ig_gu[J + g0 + t] = local ? d.ig[1] : 0.0f;
        ig_dn[g0 + t] = local ? d.ig[2] : 0.0f;
    }
}

cudaError_t launch_nvfp4_moe_plan(const int* group_offsets, int E, int expert_begin, int expert_end, int J,
                                  const Fp4ExpertDesc* experts, int H, int M, const float* dq_gu, float* gate_out,
                                  float* up_out, const float* dq_dn, float* grouped_out, Fp4Job* gu_jobs, Fp4Job* dn_jobs,
                                  float* ig_gu, float* ig_dn, cudaStream_t stream, Fp4TcJob* tc_gu, Fp4TcJob* tc_dn,
                                  int* live) {
    return launch_pdl(nvfp4_moe_plan_kernel, dim3(1), dim3(128), 0, stream, group_offsets, E, expert_begin, expert_end, J,
                      experts, H, M, dq_gu, gate_out, up_out, dq_dn, grouped_out, gu_jobs, dn_jobs, ig_gu, ig_dn, tc_gu,
                      tc_dn, live);
}

static size_t fp4_smem(int C, int tt) {
    return (size_t)16 * (C / 2 + 16) + (size_t)16 * (C / 16 + 16) + 256 * sizeof(float) + (size_t)tt * C * sizeof(float);
}

template <int TT>
static cudaError_t launch_fp4_tile(const Fp4Job* jobs, int njobs, int max_rows, int C, cudaStream_t stream,
                                   const int* live, const int* n_live) {
    {
        cudaError_t e = ensure_dynamic_smem((const void*)nvfp4_tile_kernel<TT, (TT == 1 ? 1 : 2)>, (size_t)(200 * 1024));
        if (e != cudaSuccess) return e;
    }
    dim3 grid((max_rows + 15) / 16, njobs);
    constexpr int RPL = TT == 1 ? 1 : 2;
    return launch_pdl(nvfp4_tile_kernel<TT, RPL>, grid, dim3(128 / RPL), fp4_smem(C, TT), stream, jobs, C, live, n_live);
}

cudaError_t launch_nvfp4_jobs(const Fp4Job* jobs, int njobs, int max_rows, int max_tok, int C, bool aligned,
                              cudaStream_t stream, const int* live, const int* n_live, int typical_tok) {
    if (njobs < 1 || max_rows < 1 || max_tok < 1) return cudaSuccess;
    if (aligned && (C % 256) == 0) {
        // tokens per pass: sized for the typical group, not the largest possible one - a wider pass stages that
        // many activation rows in shared memory and costs resident blocks when most groups hold one token
        const int tt = typical_tok > 0 ? std::min(typical_tok, max_tok) : max_tok;
        if (tt >= 3 && fp4_smem(C, 4) <= 200 * 1024) return launch_fp4_tile<4>(jobs, njobs, max_rows, C, stream, live, n_live);
        if (tt >= 2 && fp4_smem(C, 2) <= 200 * 1024) return launch_fp4_tile<2>(jobs, njobs, max_rows, C, stream, live, n_live);
        if (fp4_smem(C, 1) <= 200 * 1024) return launch_fp4_tile<1>(jobs, njobs, max_rows, C, stream, live, n_live);
    }
    dim3 grid((max_rows + 3) / 4, max_tok, njobs);
    if (grid.y > 65535 || grid.z > 65535) return cudaErrorInvalidValue;
    nvfp4_generic_kernel<<<grid, 128, 0, stream>>>(jobs, live, n_live);
    return cudaGetLastError();
}

}  // namespace sb
