// Grouped affine-Q4 projections (decode and exact prefill), hand-written for sm_100a.
//
// q4_tile_kernel  -- the hot kernel.  One warp per block of 8 output rows x 2
//   matrices (fused gate/up + GeGLU) or 16 output rows x 1 matrix.  The packed
//   rows are pulled into shared memory with 16-byte cp.async copies, one commit
//   group per 256-column chunk, ALL chunks requested before the first is
//   consumed, so every SM has its whole share of the weight stream in flight
//   from the first cycle and arithmetic starts as soon as chunk 0 lands.
//   Shared rows are padded by 16 bytes so the eight rows a warp reads at the
//   same word index fall in eight different bank groups.
// q4_generic_kernel -- any C, any byte alignment, absolute group indices
//   (rows may straddle quantisation groups); one warp per (row, token).
//
// Both reproduce the reference row DAG (src/kernels.c:220-250) bit for bit.
#include "internal.h"
#include "q4_core.cuh"

namespace sb {

static __device__ __forceinline__ int align16(int v) { return (v + 15) & ~15; }

template <int NMAT, int TT>
__global__ void __launch_bounds__(32)
q4_tile_kernel(const Q4Job* __restrict__ jobs, const int* __restrict__ njobs_dev, int C) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int job_id = blockIdx.y;
    if (njobs_dev != nullptr && job_id >= *njobs_dev) return;
    const Q4Job jb = jobs[job_id];
    constexpr int ROWS_A = (NMAT == 2) ? 8 : 16;
    const int r0 = blockIdx.x * ROWS_A;
    if (r0 >= jb.R || jb.ntok < 1) return;
    const int lane = threadIdx.x, t = lane & 3, rsub = lane >> 2;
    const int nvalid = min(ROWS_A, jb.R - r0);

    const int row_bytes = C >> 1;
    const int w_stride = row_bytes + 16;
    const int sc_row = C >> 5;  // bytes of bf16 scales per row
    const bool sc_padded = (sc_row & 15) == 0;
    const int sc_stride = sc_padded ? sc_row + 16 : sc_row;
    const int sc_block = align16(ROWS_A * sc_stride);  // one matrix' scales
    uint8_t* sW = smem;                                // [16][w_stride]
    uint8_t* sS = sW + 16 * w_stride;                  // [NMAT][sc_block]
    uint8_t* sB = sS + NMAT * sc_block;                // [NMAT][sc_block]

    const int steps = C >> 5;
    int chunk_steps = 8;
    int nch = (steps + chunk_steps - 1) / chunk_steps;
    if (nch > 15) {
        chunk_steps = (steps + 14) / 15;
        nch = (steps + chunk_steps - 1) / chunk_steps;
    }

    // ---- issue every copy of this block, one commit group per K chunk ----
    {
        // scales / biases of the block (group 0)
#pragma unroll
        for (int m = 0; m < NMAT; m++) {
            const uint8_t* gs = (m == 0 ? jb.scales : jb.scales2) + (size_t)r0 * sc_row;
            const uint8_t* gb = (m == 0 ? jb.biases : jb.biases2);
            if (gb) gb += (size_t)r0 * sc_row;
            uint8_t* ds = sS + m * sc_block;
            uint8_t* db = sB + m * sc_block;
            if (sc_padded) {
                const int ppr = sc_row >> 4;  // 16-byte pieces per row
                for (int p = lane; p < nvalid * ppr; p += 32) {
                    int rr = p / ppr, pc = p - rr * ppr;
                    cp_async16(ds + rr * sc_stride + pc * 16, gs + (size_t)rr * sc_row + pc * 16);
                    if (gb) cp_async16(db + rr * sc_stride + pc * 16, gb + (size_t)rr * sc_row + pc * 16);
                }
            } else {
                const int total = nvalid * sc_row;
                const int full = total >> 4;
                for (int p = lane; p < full; p += 32) {
                    cp_async16(ds + p * 16, gs + p * 16);
                    if (gb) cp_async16(db + p * 16, gb + p * 16);
                }
                for (int i = (full << 4) + lane; i < total; i += 32) {
                    ds[i] = gs[i];
                    if (gb) db[i] = gb[i];
                }
            }
            if (!gb) {
                for (int i = lane; i < (sc_block >> 2); i += 32) ((uint32_t*)db)[i] = 0u;
            }
        }
        for (int ch = 0; ch < nch; ch++) {
            const int s_begin = ch * chunk_steps;
            const int cs = min(chunk_steps, steps - s_begin);
            for (int p = lane; p < 16 * cs; p += 32) {
                const int rr = p / cs, pc = p - rr * cs;
                const int m = (NMAT == 2) ? (rr >> 3) : 0;
                int grow = r0 + ((NMAT == 2) ? (rr & 7) : rr);
                grow = min(grow, jb.R - 1);
                const uint8_t* g = (m == 0 ? jb.vals : jb.vals2) + (size_t)grow * row_bytes + (s_begin + pc) * 16;
                cp_async16(sW + rr * w_stride + (s_begin + pc) * 16, g);
            }
            cp_async_commit();
        }
    }

    // thread's two weight rows: shared rows rsub and rsub + 8
    const uint32_t* w0 = (const uint32_t*)(sW + rsub * w_stride) + t;
    const uint32_t* w1 = (const uint32_t*)(sW + (rsub + 8) * w_stride) + t;
    const int sc_m1 = (NMAT == 2) ? sc_block : 0;
    const int sc_r1 = (NMAT == 2) ? rsub : rsub + 8;
    const uint16_t* s0p = (const uint16_t*)(sS + rsub * sc_stride);
    const uint16_t* b0p = (const uint16_t*)(sB + rsub * sc_stride);
    const uint16_t* s1p = (const uint16_t*)(sS + sc_m1 + sc_r1 * sc_stride);
    const uint16_t* b1p = (const uint16_t*)(sB + sc_m1 + sc_r1 * sc_stride);

    for (int tb = 0; tb < jb.ntok; tb += TT) {
        const float* xp[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            int tok = min(tb + tt, jb.ntok - 1);
            int row = jb.x_rows ? (jb.x_rows[tok] / jb.x_div) : tok;
            xp[tt] = jb.x + (size_t)row * jb.x_stride + 8 * t;
        }
        float acc0[TT][8], acc1[TT][8];
#pragma unroll
        for (int tt = 0; tt < TT; tt++)
#pragma unroll
            for (int m = 0; m < 8; m++) { acc0[tt][m] = 0.0f; acc1[tt][m] = 0.0f; }

        for (int ch = 0; ch < nch; ch++) {
            if (tb == 0) {
                cp_async_wait_dyn(nch - 1 - ch);
                __syncwarp();
            }
            const int s_begin = ch * chunk_steps;
            const int s_end = min(s_begin + chunk_steps, steps);
            float sA = 0.0f, bA = 0.0f, sB_ = 0.0f, bB_ = 0.0f;
            bool litA = false, litB = false;
#pragma unroll 2
            for (int st = s_begin; st < s_end; st++) {
                if ((st & 1) == 0 || st == s_begin) {
                    const int g = st >> 1;
                    uint32_t hs0 = s0p[g], hs1 = s1p[g];
                    sA = bf16_bits_to_f32(hs0); bA = bf16_bits_to_f32(b0p[g]);
                    sB_ = bf16_bits_to_f32(hs1); bB_ = bf16_bits_to_f32(b1p[g]);
                    litA = scale_needs_literal(hs0); litB = scale_needs_literal(hs1);
                }
                float d0[8], d1[8];
                dequant8(w0[st * 4], sA, bA, litA, d0);
                dequant8(w1[st * 4], sB_, bB_, litB, d1);
#pragma unroll
                for (int tt = 0; tt < TT; tt++) {
                    const float4 xa = __ldg((const float4*)(xp[tt] + st * 32));
                    const float4 xb = __ldg((const float4*)(xp[tt] + st * 32 + 4));
                    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int m = 0; m < 8; m++) {
                        acc0[tt][m] = __fadd_rn(acc0[tt][m], __fmul_rn(d0[m], xv[m]));
                        acc1[tt][m] = __fadd_rn(acc1[tt][m], __fmul_rn(d1[m], xv[m]));
                    }
                }
            }
        }

#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            const float y0 = fold_row_quarters(acc0[tt], t);
            const float y1 = fold_row_quarters(acc1[tt], t);
            const int tok = tb + tt;
            if (t == 3 && tok < jb.ntok) {
                float* yrow = jb.y + (size_t)tok * jb.y_stride;
                if (NMAT == 2) {
                    // fused GeGLU (reference gemma4.c:80-83 then gate*up)
                    if (rsub < nvalid) yrow[r0 + rsub] = __fmul_rn(gelu_tanh_exact(y0), y1);
                } else {
                    if (rsub < nvalid) yrow[r0 + rsub] = y0;
                    if (rsub + 8 < nvalid) yrow[r0 + rsub + 8] = y1;
                }
            }
        }
    }
}

// Any shape, any alignment.  Lane l owns accumulator l (columns c == l mod 32).
template <int NMAT>
__global__ void __launch_bounds__(128)
q4_generic_kernel(const Q4Job* __restrict__ jobs, const int* __restrict__ njobs_dev) {
    const int job_id = blockIdx.z;
    if (njobs_dev != nullptr && job_id >= *njobs_dev) return;
    const Q4Job jb = jobs[job_id];
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int tok = blockIdx.y;
    if (r >= jb.R || tok >= jb.ntok) return;
    const int lane = threadIdx.x & 31;
    const int xrow = jb.x_rows ? (jb.x_rows[tok] / jb.x_div) : tok;
    const float* x = jb.x + (size_t)xrow * jb.x_stride;
    float yv[NMAT];
#pragma unroll
    for (int m = 0; m < NMAT; m++) {
        const uint8_t* vals = m == 0 ? jb.vals : jb.vals2;
        const uint8_t* scales = m == 0 ? jb.scales : jb.scales2;
        const uint8_t* biases = m == 0 ? jb.biases : jb.biases2;
        float acc = 0.0f;
        for (int c = lane; c < jb.C; c += 32) {
            const size_t k = (size_t)r * (size_t)jb.C + (size_t)c;
            const size_t g = k >> 6;
            const uint8_t byte = vals[k >> 1];
            const uint32_t q = (k & 1) ? (uint32_t)(byte >> 4) : (uint32_t)(byte & 15u);
            const uint32_t hs = (uint32_t)scales[2 * g] | ((uint32_t)scales[2 * g + 1] << 8);
            const uint32_t hb = biases ? ((uint32_t)biases[2 * g] | ((uint32_t)biases[2 * g + 1] << 8)) : 0u;
            float d = __fmul_rn((float)q, bf16_bits_to_f32(hs));
            d = __fadd_rn(d, bf16_bits_to_f32(hb));
            acc = __fadd_rn(acc, __fmul_rn(d, x[c]));
        }
        // L_j for j = lane & 3 is needed in lanes 0..3: gather acc[j + 4a] in order.
        float L = 0.0f;
#pragma unroll
        for (int a = 0; a < 8; a++) L = __fadd_rn(L, __shfl_sync(0xffffffffu, acc, (lane & 3) + 4 * a));
        const float L2 = __shfl_sync(0xffffffffu, L, 2);
        const float L1 = __shfl_sync(0xffffffffu, L, 1);
        const float L3 = __shfl_sync(0xffffffffu, L, 3);
        yv[m] = __fadd_rn(__fadd_rn(L, L2), __fadd_rn(L1, L3));  // meaningful in lane 0
    }
    if (lane == 0) {
        float* yrow = jb.y + (size_t)tok * jb.y_stride;
        yrow[r] = (NMAT == 2) ? __fmul_rn(gelu_tanh_exact(yv[0]), yv[NMAT - 1]) : yv[0];
    }
}

static size_t tile_smem_bytes(int C, int nmat) {
    int row_bytes = C / 2, w_stride = row_bytes + 16;
    int sc_row = C / 32;
    int sc_stride = (sc_row % 16 == 0) ? sc_row + 16 : sc_row;
    int rows_a = nmat == 2 ? 8 : 16;
    int sc_block = (rows_a * sc_stride + 15) & ~15;
    return (size_t)16 * w_stride + (size_t)2 * nmat * sc_block;
}

bool q4_tile_supported(int C) { return C >= 64 && (C % 64) == 0 && tile_smem_bytes(C, 2) <= 200 * 1024; }

template <int NMAT, int TT>
static cudaError_t launch_tile(const Q4Job* jobs, int njobs_max, const int* njobs_dev, int max_rows, int C,
                               cudaStream_t stream) {
    size_t smem = tile_smem_bytes(C, NMAT);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(q4_tile_kernel<NMAT, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)(200 * 1024));
        if (e != cudaSuccess) return e;
        configured = 200 * 1024;
    }
    constexpr int ROWS_A = NMAT == 2 ? 8 : 16;
    dim3 grid((max_rows + ROWS_A - 1) / ROWS_A, njobs_max);
    q4_tile_kernel<NMAT, TT><<<grid, 32, smem, stream>>>(jobs, njobs_dev, C);
    return cudaGetLastError();
}

cudaError_t launch_q4_jobs(const Q4Job* jobs, int njobs_max, const int* njobs_dev, int max_rows, int max_tok, int C,
                           int nmat, bool aligned, cudaStream_t stream) {
    if (njobs_max < 1 || max_rows < 1 || max_tok < 1) return cudaSuccess;
    if (aligned && q4_tile_supported(C)) {
        const int tt = max_tok >= 3 ? 4 : (max_tok == 2 ? 2 : 1);
        if (nmat == 2) {
            if (tt == 1) return launch_tile<2, 1>(jobs, njobs_max, njobs_dev, max_rows, C, stream);
            if (tt == 2) return launch_tile<2, 2>(jobs, njobs_max, njobs_dev, max_rows, C, stream);
            return launch_tile<2, 4>(jobs, njobs_max, njobs_dev, max_rows, C, stream);
        }
        if (tt == 1) return launch_tile<1, 1>(jobs, njobs_max, njobs_dev, max_rows, C, stream);
        if (tt == 2) return launch_tile<1, 2>(jobs, njobs_max, njobs_dev, max_rows, C, stream);
        return launch_tile<1, 4>(jobs, njobs_max, njobs_dev, max_rows, C, stream);
    }
    dim3 grid((max_rows + 3) / 4, max_tok, njobs_max);
    if (grid.y > 65535 || grid.z > 65535) return cudaErrorInvalidValue;
    if (nmat == 2) q4_generic_kernel<2><<<grid, 128, 0, stream>>>(jobs, njobs_dev);
    else q4_generic_kernel<1><<<grid, 128, 0, stream>>>(jobs, njobs_dev);
    return cudaGetLastError();
}

}  // namespace sb
