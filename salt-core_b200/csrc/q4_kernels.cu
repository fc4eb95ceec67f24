// Grouped affine-Q4 projections (decode and exact prefill), hand-written for sm_100a.
//
// q4_tile16_kernel -- the hot kernel.  A block holds 8 or 16 row slots of 16 lanes each: 8 or
//   16 output row pairs x 2 matrices (fused gate/up + GeGLU), or twice as many rows x 1 matrix.
//   The packed rows are pulled into shared memory with 16-byte cp.async copies, one commit
//   group per 256-column chunk, ALL chunks requested before the first is consumed, so every
//   SM has its whole share of the weight stream in flight from the first cycle and arithmetic
//   starts as soon as chunk 0 lands.  Shared rows are padded by 16 bytes so the rows a warp
//   reads at the same byte index fall in different bank groups.  Launched as a programmatic
//   dependent launch where the caller asks for it (pdl.cuh).
// q4_generic_kernel -- any C, any byte alignment, absolute group indices
//   (rows may straddle quantisation groups); one warp per (row, token).
//
// Both reproduce the reference row DAG (src/kernels.c:220-250) bit for bit.
#include "internal.h"
#include "pdl.cuh"
#include "q4_core.cuh"

namespace sb {

// Shared-memory geometry of one block (rows_a = rows of the first matrix held by a block).
struct TileGeom {
    int row_bytes, w_stride, sc_row, sc_stride, sc_block, steps, chunk_steps, nch, tpitch;
    bool sc_padded;
};

static __host__ __device__ __forceinline__ TileGeom tile_geom(int C, int rows_a) {
    TileGeom g;
    g.row_bytes = C >> 1;
    g.w_stride = g.row_bytes + 16;   // +16 B: rows r and r+1 start 4 banks apart
    g.sc_row = C >> 5;               // bytes of bf16 scales per row
    g.sc_padded = (g.sc_row & 15) == 0;
    g.sc_stride = g.sc_padded ? g.sc_row + 16 : g.sc_row;
    g.sc_block = (rows_a * g.sc_stride + 15) & ~15;
    // words per row of the interleaved scale|bias table: the smallest pitch >= C/64 that is
    // 8 mod 16, so the four rows a warp reads together start in four different banks
    g.tpitch = (C >> 6) + ((8 - ((C >> 6) & 15)) & 15);
    g.steps = C >> 5;                // 32-column steps (16 packed bytes per row)
    g.chunk_steps = 8;
    g.nch = (g.steps + 7) / 8;
    if (g.nch > 15) {
        g.chunk_steps = (((g.steps + 14) / 15) + 1) & ~1;
        g.nch = (g.steps + g.chunk_steps - 1) / g.chunk_steps;
    }
    return g;
}

// The work of one block once its job is known: TT tokens of the group per pass.
// HALF = row slots of a block (8 or 16): 16 * HALF threads, 2 * HALF weight rows in shared
// memory (NMAT == 2: HALF gate rows then HALF up rows; NMAT == 1: slot pr owns rows pr and
// pr + HALF).  Larger blocks halve the activation copies per weight byte, which matters once a
// group has several tokens.
template <int NMAT, int TT, int HALF>
__device__ void tile16_block(const Q4Job& jb, int C, int jobs_early) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int NT = 16 * HALF;
    constexpr int RT = 2 * HALF;                 // weight rows held in shared memory
    constexpr int ROWS_A = (NMAT == 2) ? HALF : RT;
    const int r0 = blockIdx.x * ROWS_A;
    if (r0 >= jb.R || jb.ntok < 1) return;
    const int tid = threadIdx.x;
    const int v = tid & 15;                      // accumulators 2v, 2v + 1
    const int pr = tid >> 4;                     // row slot 0..HALF-1
    const int nvalid = min(ROWS_A, jb.R - r0);
    const TileGeom G = tile_geom(C, ROWS_A);
    uint8_t* sW = smem;                                   // [RT][w_stride]
    uint8_t* sS = sW + RT * G.w_stride;                   // [NMAT][sc_block]
    uint8_t* sBi = sS + NMAT * G.sc_block;                // [NMAT][sc_block]
    uint32_t* sT = (uint32_t*)(sBi + NMAT * G.sc_block);  // [RT][tpitch] (scale bf16 << 16) | bias bf16
    const int tpitch = G.tpitch;
    float* sX = (float*)(sT + RT * tpitch);               // [TT][C]

    // ---- group 0: K chunk 0, scales, biases, activations of the first token block (the weight
    // copies go first: they need nothing but the job, while the activation rows may sit behind
    // one more dependent load of the row table) ----
    const bool fast_chunks = G.chunk_steps == 8;
    // 8-step chunks: a chunk is RT rows x 8 pieces of 16 bytes = one copy per thread, and the
    // thread's (row, piece) pair is the same in every chunk
    const int f_pc = tid & 7, f_rr = tid >> 3;
    const int f_m = (NMAT == 2) ? (f_rr / HALF) : 0;
    const int f_grow = min(r0 + ((NMAT == 2) ? (f_rr & (HALF - 1)) : f_rr), jb.R - 1);
    const uint8_t* f_src = (f_m == 0 ? jb.vals : jb.vals2) + (size_t)f_grow * G.row_bytes + f_pc * 16;
    uint8_t* f_dst = sW + f_rr * G.w_stride + f_pc * 16;
    if (fast_chunks && f_pc < G.steps) {
        cp_async16(f_dst, f_src);
    }
    auto issue_x = [&](int tb) {
        const int ppr = C >> 2;                  // 16-byte pieces per activation row
#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            const int tok = min(tb + tt, jb.ntok - 1);
            const int row = jb.x_rows ? (jb.x_rows[tok] / jb.x_div) : tok;
            const float* src = jb.x + (size_t)row * jb.x_stride;
            for (int pc = tid; pc < ppr; pc += NT) cp_async16(sX + tt * C + pc * 4, src + pc * 4);
        }
    };
#pragma unroll
    for (int m = 0; m < NMAT; m++) {
        const uint8_t* gs = (m == 0 ? jb.scales : jb.scales2) + (size_t)r0 * G.sc_row;
        const uint8_t* gb = (m == 0 ? jb.biases : jb.biases2);
        if (gb) gb += (size_t)r0 * G.sc_row;
        uint8_t* ds = sS + m * G.sc_block;
        uint8_t* db = sBi + m * G.sc_block;
        if (G.sc_padded) {
            const int ppr = G.sc_row >> 4;
            for (int p = tid; p < nvalid * ppr; p += NT) {
                const int rr = p / ppr, pc = p - rr * ppr;
                cp_async16(ds + rr * G.sc_stride + pc * 16, gs + (size_t)rr * G.sc_row + pc * 16);
                if (gb) cp_async16(db + rr * G.sc_stride + pc * 16, gb + (size_t)rr * G.sc_row + pc * 16);
            }
        } else {
            const int total = nvalid * G.sc_row;
            const int full = total >> 4;
            for (int p = tid; p < full; p += NT) {
                cp_async16(ds + p * 16, gs + p * 16);
                if (gb) cp_async16(db + p * 16, gb + p * 16);
            }
            for (int i = (full << 4) + tid; i < total; i += NT) {
                ds[i] = gs[i];
                if (gb) db[i] = gb[i];
            }
        }
        if (!gb)
            for (int i = tid; i < (G.sc_block >> 2); i += NT) ((uint32_t*)db)[i] = 0u;
    }
    if (jobs_early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    issue_x(0);
    if (fast_chunks) {
        cp_async_commit();
        for (int ch = 1; ch < G.nch; ch++) {
            if (ch * 8 + f_pc < G.steps) cp_async16(f_dst + ch * 128, f_src + ch * 128);
            cp_async_commit();
        }
    } else {
        for (int ch = 0; ch < G.nch; ch++) {
            const int s_begin = ch * G.chunk_steps;
            const int cs = min(G.chunk_steps, G.steps - s_begin);
            for (int p = tid; p < RT * cs; p += NT) {
                const int rr = p / cs;
                const int pc = p - rr * cs;
                const int m = (NMAT == 2) ? (rr / HALF) : 0;
                const int grow = min(r0 + ((NMAT == 2) ? (rr & (HALF - 1)) : rr), jb.R - 1);
                const uint8_t* g = (m == 0 ? jb.vals : jb.vals2) + (size_t)grow * G.row_bytes + (s_begin + pc) * 16;
                cp_async16(sW + rr * G.w_stride + (s_begin + pc) * 16, g);
            }
            cp_async_commit();
        }
    }

    // ---- this thread's operands ----
    const uint8_t* wA = sW + pr * G.w_stride + v;
    const uint8_t* wB = sW + (pr + HALF) * G.w_stride + v;
    const int gpr = C >> 6;                      // quantisation groups per row
    const uint32_t* tA = sT + pr * tpitch;
    const uint32_t* tB = sT + (pr + HALF) * tpitch;
    const NibbleMagic mg = load_nibble_magic();
    const f32x2 nz = pack2u(c_neg_zero, c_neg_zero);
    const float* xs = sX + 2 * v;

    // wait for group 0, interleave the bf16 scales/biases of the 16 rows into one word per
    // group, and note whether any scale needs the literal (two-rounding) dequantisation
    cp_async_wait_dyn(G.nch - 1);
    __syncthreads();
    int lit = 0;
    for (int gg = tid & 7; gg < gpr; gg += 8) {
        const int rr = tid >> 3;                 // NT threads = RT rows x 8 column phases
        const int m = (NMAT == 2) ? (rr / HALF) : 0;
        const int lr = (NMAT == 2) ? (rr & (HALF - 1)) : rr;
        const uint32_t hs = ((const uint16_t*)(sS + m * G.sc_block + lr * G.sc_stride))[gg];
        const uint32_t hb = ((const uint16_t*)(sBi + m * G.sc_block + lr * G.sc_stride))[gg];
        sT[rr * tpitch + gg] = (hs << 16) | hb;
        if (lr < nvalid) lit |= scale_needs_literal(hs) ? 1 : 0;
    }
    lit = __syncthreads_or(lit);

    for (int tb = 0; tb < jb.ntok; tb += TT) {
        if (tb > 0) {
            __syncthreads();                     // everyone is done with the previous activations
            issue_x(tb);
            cp_async_commit();
            cp_async_wait_dyn(0);
            __syncthreads();
        }
        f32x2 accA[TT], accB[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) { accA[tt] = pack2(0.0f, 0.0f); accB[tt] = pack2(0.0f, 0.0f); }
        for (int ch = 0; ch < G.nch; ch++) {
            if (tb == 0 && ch > 0) {
                cp_async_wait_dyn(G.nch - 1 - ch);
                __syncthreads();
            }
            const int s_begin = ch * G.chunk_steps;
            const int s_end = min(s_begin + G.chunk_steps, G.steps);
            if (lit) tile16_run<TT, true>(mg, s_begin, s_end, wA, wB, tA, tB, xs, C, accA, accB, nz);
            else tile16_run<TT, false>(mg, s_begin, s_end, wA, wB, tA, tB, xs, C, accA, accB, nz);
        }
#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            const float y0 = fold_row_hexadecants(accA[tt], v);
            const float y1 = fold_row_hexadecants(accB[tt], v);
            const int tok = tb + tt;
            if (v == 0 && tok < jb.ntok) {
                float* yrow = jb.y + (size_t)tok * jb.y_stride;
                if (NMAT == 2) {
                    // fused GeGLU (reference gemma4.c:80-83 then gate*up)
                    if (pr < nvalid) yrow[r0 + pr] = __fmul_rn(gelu_tanh_exact(y0), y1);
                } else {
                    if (pr < nvalid) yrow[r0 + pr] = y0;
                    if (pr + HALF < nvalid) yrow[r0 + pr + HALF] = y1;
                }
            }
        }
    }
}

// One block = 128 threads = 8 row pairs (NMAT == 2: gate row r and up row r, fused GeGLU
// epilogue) or 16 rows (NMAT == 1: rows r and r + 8 per lane group).  TTMAX = most tokens of a
// group handled per pass (and what the shared activation area is sized for); a block whose
// group is smaller runs the code specialised for 1 or 2 tokens, so decode batches whose
// expert groups hold one or two tokens do not pay for four.
template <int NMAT, int TTMAX, int HALF>
__global__ void __launch_bounds__(16 * HALF)
q4_tile16_kernel(const Q4Job* __restrict__ jobs, const int* __restrict__ njobs_dev, int C, int jobs_early) {
    // jobs_early: the job table was written at least two launches back, so everything except the
    // activation rows (the previous kernel's output) may be fetched before the dependency wait
    if (!jobs_early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const int job_id = blockIdx.y;
    // both loads are issued before the count is tested (blockIdx.y always indexes inside the job array)
    // (read through L2: with jobs_early these loads run before the dependency wait, when this
    // SM's L1 may still hold the table of an earlier pass)
    const int njobs_live = njobs_dev != nullptr ? __ldcg(njobs_dev) : 0x7fffffff;
    Q4Job jb;
    {
        static_assert(sizeof(Q4Job) % 16 == 0, "job descriptors are copied in 16-byte pieces");
        const uint4* src = (const uint4*)(jobs + job_id);
        uint4* dst = (uint4*)&jb;
#pragma unroll
        for (int q = 0; q < (int)(sizeof(Q4Job) / 16); q++) dst[q] = __ldcg(src + q);
    }
    if (job_id >= njobs_live) return;
    if (TTMAX >= 4 && jb.ntok >= 3) tile16_block<NMAT, (TTMAX >= 4 ? 4 : TTMAX), HALF>(jb, C, jobs_early);
    else if (TTMAX >= 2 && jb.ntok == 2) tile16_block<NMAT, (TTMAX >= 2 ? 2 : TTMAX), HALF>(jb, C, jobs_early);
    else tile16_block<NMAT, 1, HALF>(jb, C, jobs_early);
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

static size_t tile_smem_bytes(int C, int nmat, int tt, int half) {
    const TileGeom g = tile_geom(C, nmat == 2 ? half : 2 * half);
    return (size_t)(2 * half) * g.w_stride + (size_t)2 * nmat * g.sc_block + (size_t)(2 * half) * g.tpitch * 4 +
           (size_t)tt * C * sizeof(float);
}

bool q4_tile_supported(int C) { return C >= 64 && (C % 64) == 0 && tile_smem_bytes(C, 2, 4, 16) <= 200 * 1024; }

template <int NMAT, int TT>
static cudaError_t launch_tile(const Q4Job* jobs, int njobs_max, const int* njobs_dev, int max_rows, int C,
                               cudaStream_t stream, int pdl) {
    // single-token groups: 8 row slots per block (more, smaller blocks: lowest latency);
    // several tokens per group: 16 row slots (half the activation copies per weight byte)
    constexpr int HALF = TT == 1 ? 8 : 16;
    size_t smem = tile_smem_bytes(C, NMAT, TT, HALF);
    if (smem > 48 * 1024) {
        cudaError_t e = ensure_dynamic_smem((const void*)q4_tile16_kernel<NMAT, TT, HALF>, (size_t)(200 * 1024));
        if (e != cudaSuccess) return e;
    }
    constexpr int ROWS_A = NMAT == 2 ? HALF : 2 * HALF;
    dim3 grid((max_rows + ROWS_A - 1) / ROWS_A, njobs_max);
    if (pdl >= 0)
        return launch_pdl(q4_tile16_kernel<NMAT, TT, HALF>, grid, dim3(16 * HALF), smem, stream, jobs, njobs_dev, C, pdl);
    q4_tile16_kernel<NMAT, TT, HALF><<<grid, 16 * HALF, smem, stream>>>(jobs, njobs_dev, C, 0);
    return cudaGetLastError();
}

cudaError_t launch_q4_jobs(const Q4Job* jobs, int njobs_max, const int* njobs_dev, int max_rows, int max_tok, int C,
                           int nmat, bool aligned, cudaStream_t stream, int pdl) {
    if (njobs_max < 1 || max_rows < 1 || max_tok < 1) return cudaSuccess;
    if (aligned && q4_tile_supported(C)) {
        const int tt = max_tok >= 3 ? 4 : (max_tok == 2 ? 2 : 1);
        if (nmat == 2) {
            if (tt == 1) return launch_tile<2, 1>(jobs, njobs_max, njobs_dev, max_rows, C, stream, pdl);
            if (tt == 2) return launch_tile<2, 2>(jobs, njobs_max, njobs_dev, max_rows, C, stream, pdl);
            return launch_tile<2, 4>(jobs, njobs_max, njobs_dev, max_rows, C, stream, pdl);
        }
        if (tt == 1) return launch_tile<1, 1>(jobs, njobs_max, njobs_dev, max_rows, C, stream, pdl);
        if (tt == 2) return launch_tile<1, 2>(jobs, njobs_max, njobs_dev, max_rows, C, stream, pdl);
        return launch_tile<1, 4>(jobs, njobs_max, njobs_dev, max_rows, C, stream, pdl);
    }
    dim3 grid((max_rows + 3) / 4, max_tok, njobs_max);
    if (grid.y > 65535 || grid.z > 65535) return cudaErrorInvalidValue;
    if (nmat == 2) q4_generic_kernel<2><<<grid, 128, 0, stream>>>(jobs, njobs_dev);
    else q4_generic_kernel<1><<<grid, 128, 0, stream>>>(jobs, njobs_dev);
    return cudaGetLastError();
}

}  // namespace sb
