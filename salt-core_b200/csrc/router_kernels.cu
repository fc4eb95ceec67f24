// Router, grouping and reduction kernels of the MoE feed-forward path.
//
// Everything here is bit-exact against the reference CPU functions; the reference arithmetic
// contains several chains that are serial by definition (sums of squares, router logits,
// softmax denominators).  Signed chains (logits, denominators) are kept serial per row / expert,
// with the independent products formed ahead by other lanes and many chains running side by
// side; the sums of squares are reproduced by a predict-and-verify scheme (block_sum_nonneg)
// that does most of the additions as order-free integer increments.
#include "internal.h"
#include "pdl.cuh"
#include "q4_core.cuh"
#include "router_core.cuh"

namespace sb {

// mode 0: RMSNorm  y = (x*inv) [* weight]             (gemma4.c:85-101)
// mode 1: router input  y = ((x*inv)*scale)*root      (gemma4.c:103-130)
template <int MODE>
__global__ void __launch_bounds__(256)
norm_rows_kernel(const float* __restrict__ x, const float* __restrict__ weight, float* __restrict__ y, int n,
                 float eps, int with_scale, float root_in, int* status) {
    extern __shared__ __align__(16) float srow[];   // [n] row, then [n (padded to 4)] squares
    float* ssq = srow + ((n + 3) & ~3);
    __shared__ float s_inv, s_root;
    __shared__ __align__(8) uint32_t s_scan[POSSUM_SCRATCH];
    const float* xr = x + (size_t)blockIdx.x * n;
    float* yr = y + (size_t)blockIdx.x * n;
    bool bad = false;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i];
        srow[i] = v;
        ssq[i] = __fmul_rn(v, v);
        bad |= !finite_f(v);
        if (MODE == 1 || with_scale) bad |= !finite_f(weight[i]);
    }
    const float ss = ordered_sum_of_squares(ssq, n, bad, s_scan);
    if (threadIdx.x == 0) {
        {
            const float mean = __fadd_rn(__fdiv_rn(ss, (float)n), eps);
            const float inv = pow_neg_half(mean);
            float root = 1.0f;
            if (MODE == 1) root = root_in > 0.0f ? root_in : __fdiv_rn(1.0f, sqrtf_exact((float)n));
            s_inv = inv;
            s_root = root;
            if (!finite_f(inv) || !finite_f(root)) flag(status, SB_ERR_NONFINITE);
        }
    }
    __syncthreads();
    const float inv = s_inv, root = s_root;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = __fmul_rn(srow[i], inv);
        if (MODE == 1) {
            v = __fmul_rn(v, weight[i]);
            v = __fmul_rn(v, root);
        } else if (with_scale) {
            v = __fmul_rn(v, weight[i]);
        }
        bad |= !finite_f(v);
        yr[i] = v;
    }
    if (bad) flag(status, SB_ERR_NONFINITE);
}

// Token-wise glue between the expert phase of one layer and the router of the
// next, in one launch per row:
//   [reduce]  v = ordered weighted sum of the row's grouped expert outputs
//             (src/tensorops.c:291-325), else v = x_in
//   [norm]    v = RMSNorm(v) * norm_w                      (gemma4.c:85-101)
//             y_out = v  (written whenever reduce or norm ran)
//   [router]  rin = ((v * inv) * scale) * (1/sqrt(n))      (gemma4.c:103-130)
// The two sums of squares are formed in element order by block_sum_nonneg over
// squares computed in parallel.
// ---- affine 8-bit matvec (router projections of packages that quantise the router) -----------
// src/kernels.c:343-369: one byte per element, bf16 scale / bias per 64 consecutive elements of
// the flattened matrix (rows may straddle groups), ONE serial chain per row:
// acc = fl(acc + fl(d * x[c])), d = fl(fl(q*s) + b).  One block per (row, token, job): the
// products are formed in parallel, one thread runs the chain.
__global__ void __launch_bounds__(128) q8_rows_kernel(const Q4Job* __restrict__ jobs) {
    extern __shared__ __align__(16) float q8_sm[];
    const Q4Job jb = jobs[blockIdx.z];
    const int r = blockIdx.x, tok = blockIdx.y;
    if (r >= jb.R || tok >= jb.ntok) return;
    const float* x = jb.x + (size_t)tok * jb.x_stride;
    const size_t k0 = (size_t)r * (size_t)jb.C;
    for (int c = threadIdx.x; c < jb.C; c += blockDim.x) {
        const size_t k = k0 + (size_t)c, g = k >> 6;
        const float s = bf16_bits_to_f32(((const uint16_t*)jb.scales)[g]);
        const float b = jb.biases ? bf16_bits_to_f32(((const uint16_t*)jb.biases)[g]) : 0.0f;
        const float d = __fadd_rn(__fmul_rn((float)jb.vals[k], s), b);
        q8_sm[c] = __fmul_rn(d, x[c]);
    }
    __syncthreads();
    if (threadIdx.x == 0) jb.y[(size_t)tok * jb.y_stride + r] = serial_sum(q8_sm, jb.C);
}

cudaError_t launch_q8_jobs(const Q4Job* jobs, int njobs, int max_rows, int max_tok, int C, cudaStream_t stream) {
    if (njobs < 1 || max_rows < 1 || max_tok < 1) return cudaSuccess;
    const size_t smem = (size_t)((C + 3) & ~3) * sizeof(float);
    if (smem > 200 * 1024 || max_tok > 65535 || njobs > 65535) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = ensure_dynamic_smem((const void*)q8_rows_kernel, (size_t)(200 * 1024));
        if (e != cudaSuccess) return e;
    }
    q8_rows_kernel<<<dim3(max_rows, max_tok, njobs), 128, smem, stream>>>(jobs);
    return cudaGetLastError();
}

// ---- consumers of the routed-expert output (exact cells) -------------------------------------
// y = (x * inv) * w with inv = (mean(x^2) + eps)^-1/2, one row per block; sq = n floats of shared
// memory.  Returns with y complete and visible to the whole block.
static __device__ void norm_row_block(const float* x, const float* w, float* y, int n, float eps, float* sq,
                                      uint32_t* scan, float* s_inv, bool& bad, int* status) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        sq[i] = __fmul_rn(v, v);
        bad |= !finite_f(v) || !finite_f(w[i]);
    }
    const float ss = ordered_sum_of_squares(sq, n, bad, scan);
    if (threadIdx.x == 0) {
        *s_inv = pow_neg_half(__fadd_rn(__fdiv_rn(ss, (float)n), eps));
        if (!finite_f(*s_inv)) flag(status, SB_ERR_NONFINITE);
    }
    __syncthreads();
    const float inv = *s_inv;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float t = __fmul_rn(__fmul_rn(x[i], inv), w[i]);
        bad |= !finite_f(t);
        y[i] = t;
    }
    __syncthreads();
}

// out = residual + RMSNorm(branch) * weight   (models/gemma4-26b-a4b/src/gemma4.c:188-213)
__global__ void __launch_bounds__(1024)
residual_postnorm_rows_kernel(const float* __restrict__ residual, const float* __restrict__ branch,
                              const float* __restrict__ weight, float* __restrict__ out, int n, float eps,
                              int* status) {
    extern __shared__ __align__(16) float cell_sm[];     // [n] squares, [n] normalised branch
    __shared__ float s_inv;
    __shared__ __align__(8) uint32_t s_scan[POSSUM_SCRATCH];
    const size_t row = blockIdx.x;
    float* normed = cell_sm + ((n + 3) & ~3);
    bool bad = false;
    norm_row_block(branch + row * n, weight, normed, n, eps, cell_sm, s_scan, &s_inv, bad, status);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float r = residual[row * n + i];
        const float y = __fadd_rn(r, normed[i]);
        bad |= !finite_f(r) || !finite_f(y);
        out[row * n + i] = y;
    }
    if (bad) flag(status, SB_ERR_NONFINITE);
}

// sum = RMSNorm(dense)*wd + RMSNorm(routed)*wr; fin = RMSNorm(sum)*wf; out = (residual + fin) * scalar
// (gemma4.c:215-276).  scratch_a / scratch_b receive sum / fin as the reference leaves them.
__global__ void __launch_bounds__(1024)
parallel_combine_rows_kernel(const float* __restrict__ residual, const float* __restrict__ dense,
                             const float* __restrict__ routed, const float* __restrict__ wd,
                             const float* __restrict__ wr, const float* __restrict__ wf, float* scratch_a,
                             float* scratch_b, float* __restrict__ out, int n, float eps, float scalar, int* status) {
    extern __shared__ __align__(16) float cell_sm[];     // [n] squares
    __shared__ float s_inv;
    __shared__ __align__(8) uint32_t s_scan[POSSUM_SCRATCH];
    const size_t row = blockIdx.x;
    float* sum = scratch_a + row * n;
    float* fin = scratch_b + row * n;
    bool bad = !finite_f(scalar);
    norm_row_block(dense + row * n, wd, sum, n, eps, cell_sm, s_scan, &s_inv, bad, status);
    norm_row_block(routed + row * n, wr, fin, n, eps, cell_sm, s_scan, &s_inv, bad, status);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float c = __fadd_rn(sum[i], fin[i]);
        bad |= !finite_f(c);
        sum[i] = c;
    }
    __syncthreads();
    norm_row_block(sum, wf, fin, n, eps, cell_sm, s_scan, &s_inv, bad, status);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float r = residual[row * n + i];
        const float y = __fmul_rn(__fadd_rn(r, fin[i]), scalar);
        bad |= !finite_f(r) || !finite_f(y);
        out[row * n + i] = y;
    }
    if (bad) flag(status, SB_ERR_NONFINITE);
}

// logits = cap * tanh(logits / cap), in place   (gemma4.c:278-286)
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ logits, int n, float cap, int* status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = logits[i];
    if (!finite_f(v)) {
        flag(status, SB_ERR_NONFINITE);
        return;
    }
    logits[i] = __fmul_rn(cap, tanhf_exact(__fdiv_rn(v, cap)));
}

cudaError_t launch_residual_postnorm(const float* residual, const float* branch, const float* weight, float* out,
                                     int rows, int n, float eps, int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    const size_t smem = (size_t)(2 * ((n + 3) & ~3) + 8) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = ensure_dynamic_smem((const void*)residual_postnorm_rows_kernel, (size_t)(200 * 1024));
        if (e != cudaSuccess) return e;
    }
    residual_postnorm_rows_kernel<<<rows, 1024, smem, stream>>>(residual, branch, weight, out, n, eps, status);
    return cudaGetLastError();
}

cudaError_t launch_parallel_combine(const float* residual, const float* dense, const float* routed, const float* wd,
                                    const float* wr, const float* wf, float* scratch_a, float* scratch_b, float* out,
                                    int rows, int n, float eps, float scalar, int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    const size_t smem = (size_t)(n + 8) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = ensure_dynamic_smem((const void*)parallel_combine_rows_kernel, (size_t)(200 * 1024));
        if (e != cudaSuccess) return e;
    }
    parallel_combine_rows_kernel<<<rows, 1024, smem, stream>>>(residual, dense, routed, wd, wr, wf, scratch_a, scratch_b,
                                                               out, n, eps, scalar, status);
    return cudaGetLastError();
}

cudaError_t launch_softcap(float* logits, int n, float cap, int* status, cudaStream_t stream) {
    if (n < 1) return cudaSuccess;
    softcap_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, n, cap, status);
    return cudaGetLastError();
}

// Each thread owns the columns d = threadIdx.x + j * blockDim.x (j < GLUE_NV, compile
// time) so that every global load of a phase is issued before the first use: the norm
// weights and router scales right at the start, the rows of the expert outputs as soon as
// the rank table is known.
// <4, 8> with 1024 threads serves rows up to 4096 columns; <16, 2> with 512 threads up to 8192.
template <int GLUE_NV, int GLUE_RB>
__global__ void __launch_bounds__(GLUE_NV == 4 ? 1024 : 512) glue_rows_kernel(GlueArgs a) {
    extern __shared__ __align__(16) float gsm[];
    const int n = a.n;
    float* sq = gsm;                       // [n] squares for the ordered sums
    __shared__ float s_inv, s_root;
    __shared__ __align__(8) uint32_t s_scan[POSSUM_SCRATCH];
    __shared__ int s_g[64];
    __shared__ float s_w[64];
    const int row = blockIdx.x, T = blockDim.x, tid = threadIdx.x;
    bool bad = false;
    float v[GLUE_NV], nw[GLUE_NV], rs[GLUE_NV];
#pragma unroll
    for (int j = 0; j < GLUE_NV; j++) {
        const int d = tid + j * T;
        nw[j] = (a.norm_w != nullptr && d < n) ? __ldg(a.norm_w + d) : 1.0f;
        rs[j] = (a.router_scale != nullptr && d < n) ? __ldg(a.router_scale + d) : 1.0f;
        v[j] = 0.0f;
    }
    // the rank table was written by the plan kernel, at least two launches back (unless tables_late)
    int early_g = -1;
    float early_w = 0.0f;
    if (a.grouped != nullptr && tid < a.topk && !a.tables_late) {
        early_g = __ldcg(a.c2g + row * a.topk + tid);      // through L2: this SM's L1 may hold an earlier pass
        early_w = __ldcg(a.weights + row * a.topk + tid);
    }
    pdl_wait();                    // the expert outputs (or x_in) come from the previous kernel
    pdl_launch_dependents();
    if (a.grouped != nullptr && tid < a.topk && a.tables_late) {
        early_g = __ldcg(a.c2g + row * a.topk + tid);
        early_w = __ldcg(a.weights + row * a.topk + tid);
    }
    if (a.grouped != nullptr) {
        // rank -> (grouped row, weight) once per block; invalid ranks are dropped and flagged
        if (tid < a.topk) {
            int g = early_g;
            const float w = early_w;
            if (g < 0 || g >= a.jobs || !finite_f(w)) {
                flag(a.status, g < 0 || g >= a.jobs ? SB_ERR_INDEX : SB_ERR_NONFINITE);
                g = -1;
            }
            s_g[tid] = g;
            s_w[tid] = w;
        }
        __syncthreads();
        for (int r0 = 0; r0 < a.topk; r0 += GLUE_RB) {
            float o[GLUE_NV][GLUE_RB];
#pragma unroll
            for (int i = 0; i < GLUE_RB; i++) {
                const int g = r0 + i < a.topk ? s_g[r0 + i] : -1;
#pragma unroll
                for (int j = 0; j < GLUE_NV; j++) {
                    const int d = tid + j * T;
                    o[j][i] = (g >= 0 && d < n) ? __ldg(a.grouped + (size_t)g * n + d) : 0.0f;
                }
            }
#pragma unroll
            for (int i = 0; i < GLUE_RB; i++)
                if (r0 + i < a.topk && s_g[r0 + i] >= 0) {
                    const float w = s_w[r0 + i];
#pragma unroll
                    for (int j = 0; j < GLUE_NV; j++) v[j] = __fadd_rn(v[j], __fmul_rn(w, o[j][i]));
                }
        }
    } else {
#pragma unroll
        for (int j = 0; j < GLUE_NV; j++) {
            const int d = tid + j * T;
            if (d < n) v[j] = a.x_in[(size_t)row * n + d];
        }
    }
    if (a.norm_w != nullptr) {
#pragma unroll
        for (int j = 0; j < GLUE_NV; j++) {
            const int d = tid + j * T;
            if (d < n) {
                sq[d] = __fmul_rn(v[j], v[j]);
                bad |= !finite_f(v[j]) || !finite_f(nw[j]);
            }
        }
        const float ss = ordered_sum_of_squares<GLUE_NV>(sq, n, bad, s_scan);
        if (tid == 0) {
            s_inv = pow_neg_half(__fadd_rn(__fdiv_rn(ss, (float)n), a.eps_norm));
            if (!finite_f(s_inv)) flag(a.status, SB_ERR_NONFINITE);
        }
        __syncthreads();
        const float inv = s_inv;
#pragma unroll
        for (int j = 0; j < GLUE_NV; j++) {
            v[j] = __fmul_rn(__fmul_rn(v[j], inv), nw[j]);
            if (tid + j * T < n) bad |= !finite_f(v[j]);
        }
    }
    if (a.y_out != nullptr) {
#pragma unroll
        for (int j = 0; j < GLUE_NV; j++) {
            const int d = tid + j * T;
            if (d < n) a.y_out[(size_t)row * n + d] = v[j];
        }
    }
    if (a.router_scale != nullptr) {
        __syncthreads();   // the previous ordered sum has been read by everyone before sq is rewritten
#pragma unroll
        for (int j = 0; j < GLUE_NV; j++) {
            const int d = tid + j * T;
            if (d < n) {
                sq[d] = __fmul_rn(v[j], v[j]);
                bad |= !finite_f(v[j]) || !finite_f(rs[j]);
            }
        }
        const float ss = ordered_sum_of_squares<GLUE_NV>(sq, n, bad, s_scan);
        if (tid == 0) {
            s_inv = pow_neg_half(__fadd_rn(__fdiv_rn(ss, (float)n), a.eps_router));
            s_root = __fdiv_rn(1.0f, sqrtf_exact((float)n));
            if (!finite_f(s_inv) || !finite_f(s_root)) flag(a.status, SB_ERR_NONFINITE);
        }
        __syncthreads();
        const float inv = s_inv, root = s_root;
#pragma unroll
        for (int j = 0; j < GLUE_NV; j++) {
            const int d = tid + j * T;
            if (d < n) {
                const float t = __fmul_rn(__fmul_rn(__fmul_rn(v[j], inv), rs[j]), root);
                bad |= !finite_f(t);
                a.rin[(size_t)row * n + d] = t;
            }
        }
    }
    if (bad) flag(a.status, SB_ERR_NONFINITE);
}

// The same glue for batches of several hundred rows: one WARP per row, lane l holds the CH
// consecutive columns [l*CH, (l+1)*CH) in registers, and each in-order sum is the plain
// dependent-add chain handed from lane to lane (the reference's order: columns ascending from
// +0).  A chain costs about 6.5 us, but thousands of rows run side by side (16 warps per SM),
// where the block-per-row form above keeps a whole SM busy for 13 us per pair of rows.
template <int CH>
static __device__ __forceinline__ float warp_chain_sum_of_squares(const float (&v)[CH], int lane) {
    float acc = 0.0f;
#pragma unroll 1
    for (int l = 0; l < 32; l++) {
        float a = __shfl_sync(0xffffffffu, acc, (l + 31) & 31);
        if (l == 0) a = 0.0f;
        if (lane == l) {
#pragma unroll
            for (int i = 0; i < CH; i++) a = __fadd_rn(a, __fmul_rn(v[i], v[i]));
            acc = a;
        }
    }
    return __shfl_sync(0xffffffffu, acc, 31);
}

template <int CH>
__global__ void __launch_bounds__(128, CH > 96 ? 2 : 4) glue_rows_warp_kernel(GlueArgs a, int rows) {
    static_assert(CH % 4 == 0, "rows are moved in 16-byte pieces");
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int n = a.n;                         // == 32 * CH
    const int c0 = lane * CH;
    bool bad = false;
    float v[CH];
#pragma unroll
    for (int i = 0; i < CH; i++) v[i] = 0.0f;
    if (a.grouped != nullptr) {
        for (int r = 0; r < a.topk; r++) {
            const int g = a.c2g[row * a.topk + r];
            const float w = a.weights[row * a.topk + r];
            if (g < 0 || g >= a.jobs || !finite_f(w)) {
                if (lane == 0) flag(a.status, g < 0 || g >= a.jobs ? SB_ERR_INDEX : SB_ERR_NONFINITE);
                continue;
            }
            const float4* src = (const float4*)(a.grouped + (size_t)g * n + c0);
#pragma unroll
            for (int i = 0; i < CH / 4; i++) {
                const float4 o = __ldg(src + i);
                v[4 * i + 0] = __fadd_rn(v[4 * i + 0], __fmul_rn(w, o.x));
                v[4 * i + 1] = __fadd_rn(v[4 * i + 1], __fmul_rn(w, o.y));
                v[4 * i + 2] = __fadd_rn(v[4 * i + 2], __fmul_rn(w, o.z));
                v[4 * i + 3] = __fadd_rn(v[4 * i + 3], __fmul_rn(w, o.w));
            }
        }
    } else {
        const float4* src = (const float4*)(a.x_in + (size_t)row * n + c0);
#pragma unroll
        for (int i = 0; i < CH / 4; i++) {
            const float4 o = src[i];
            v[4 * i + 0] = o.x; v[4 * i + 1] = o.y; v[4 * i + 2] = o.z; v[4 * i + 3] = o.w;
        }
    }
    if (a.norm_w != nullptr) {
        const float ss = warp_chain_sum_of_squares<CH>(v, lane);
        const float inv = pow_neg_half(__fadd_rn(__fdiv_rn(ss, (float)n), a.eps_norm));
        if (!finite_f(inv) && lane == 0) flag(a.status, SB_ERR_NONFINITE);
        const float4* nw4 = (const float4*)(a.norm_w + c0);
#pragma unroll
        for (int i = 0; i < CH / 4; i++) {
            const float4 w = __ldg(nw4 + i);
            bad |= !finite_f(v[4 * i]) || !finite_f(v[4 * i + 1]) || !finite_f(v[4 * i + 2]) || !finite_f(v[4 * i + 3]);
            bad |= !finite_f(w.x) || !finite_f(w.y) || !finite_f(w.z) || !finite_f(w.w);
            v[4 * i + 0] = __fmul_rn(__fmul_rn(v[4 * i + 0], inv), w.x);
            v[4 * i + 1] = __fmul_rn(__fmul_rn(v[4 * i + 1], inv), w.y);
            v[4 * i + 2] = __fmul_rn(__fmul_rn(v[4 * i + 2], inv), w.z);
            v[4 * i + 3] = __fmul_rn(__fmul_rn(v[4 * i + 3], inv), w.w);
        }
    }
    if (a.y_out != nullptr) {
        float4* dst = (float4*)(a.y_out + (size_t)row * n + c0);
#pragma unroll
        for (int i = 0; i < CH / 4; i++) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
    if (a.router_scale != nullptr) {
        const float ss = warp_chain_sum_of_squares<CH>(v, lane);
        const float inv = pow_neg_half(__fadd_rn(__fdiv_rn(ss, (float)n), a.eps_router));
        const float root = __fdiv_rn(1.0f, sqrtf_exact((float)n));
        if ((!finite_f(inv) || !finite_f(root)) && lane == 0) flag(a.status, SB_ERR_NONFINITE);
        const float4* rs4 = (const float4*)(a.router_scale + c0);
        float4* dst = (float4*)(a.rin + (size_t)row * n + c0);
#pragma unroll
        for (int i = 0; i < CH / 4; i++) {
            const float4 w = __ldg(rs4 + i);
            float4 t;
            t.x = __fmul_rn(__fmul_rn(__fmul_rn(v[4 * i + 0], inv), w.x), root);
            t.y = __fmul_rn(__fmul_rn(__fmul_rn(v[4 * i + 1], inv), w.y), root);
            t.z = __fmul_rn(__fmul_rn(__fmul_rn(v[4 * i + 2], inv), w.z), root);
            t.w = __fmul_rn(__fmul_rn(__fmul_rn(v[4 * i + 3], inv), w.w), root);
            bad |= !finite_f(v[4 * i]) || !finite_f(v[4 * i + 1]) || !finite_f(v[4 * i + 2]) || !finite_f(v[4 * i + 3]);
            bad |= !finite_f(w.x) || !finite_f(w.y) || !finite_f(w.z) || !finite_f(w.w);
            bad |= !finite_f(t.x) || !finite_f(t.y) || !finite_f(t.z) || !finite_f(t.w);
            dst[i] = t;
        }
    }
    if (bad) flag(a.status, SB_ERR_NONFINITE);
}

cudaError_t launch_glue(const GlueArgs& a, int rows, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    if (a.topk > 64) return cudaErrorInvalidValue;
    const size_t smem = (size_t)(a.n + 8) * sizeof(float);
    const auto al16 = [](const void* p) { return (((uintptr_t)p) & 15) == 0; };
    if (rows >= 256 && (a.n == 32 * 88 || a.n == 32 * 160) && al16(a.grouped) && al16(a.x_in) && al16(a.y_out) &&
        al16(a.norm_w) && al16(a.router_scale) && al16(a.rin)) {
        if (a.n == 32 * 88) glue_rows_warp_kernel<88><<<(rows + 3) / 4, 128, 0, stream>>>(a, rows);
        else glue_rows_warp_kernel<160><<<(rows + 3) / 4, 128, 0, stream>>>(a, rows);
        return cudaGetLastError();
    }
    if (a.n <= 4096) {
        // every thread owns 4 columns: wide rows and small batches get the largest block
        const int threads = (rows <= 16 || a.n > 1024) ? 1024 : 256;
        return launch_pdl(glue_rows_kernel<4, 8>, dim3(rows), dim3(threads), smem, stream, a);
    } else if (a.n <= 8192) {
        return launch_pdl(glue_rows_kernel<16, 2>, dim3(rows), dim3(512), smem, stream, a);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm(const float* x, const float* weight, float* y, int rows, int n, float eps, int with_scale,
                           int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    norm_rows_kernel<0><<<rows, 256, (size_t)(2 * n + 8) * sizeof(float), stream>>>(x, weight, y, n, eps, with_scale, 0.0f,
                                                                           status);
    return cudaGetLastError();
}

cudaError_t launch_router_input(const float* x, const float* scale, float* out, int rows, int n, float eps,
                                float root, int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    norm_rows_kernel<1><<<rows, 256, (size_t)(2 * n + 8) * sizeof(float), stream>>>(x, scale, out, n, eps, 1, root, status);
    return cudaGetLastError();
}

// Small batches: one block per (expert, block of up to LOGIT_TB rows).  All
// threads form the products fl(W[e][c]*x[r][c]) (coalesced loads) into shared
// memory; then one thread per row runs the reference chain
// acc = fl(acc + p[c]) over them (src/kernels.c:98-106).
constexpr int LOGIT_TB = 8;

__global__ void __launch_bounds__(256)
router_logits_block_kernel(const float* __restrict__ W, const float* __restrict__ bias,
                           const float* __restrict__ x, float* __restrict__ logits, int rows, int E, int H) {
    extern __shared__ __align__(16) float sprod[];       // [nr][pitch]
    const int e = blockIdx.x;
    const int r0 = blockIdx.y * LOGIT_TB;
    const int nr = min(LOGIT_TB, rows - r0);
    const int pitch = ((H + 3) & ~3) + 4;                // +4 floats: rows start in different banks
    const float* w = W + (size_t)e * H;
    if ((H & 3) == 0) {
        // 16-byte loads; the (up to 4) W quads of a thread are all in flight before the first product
        const int nq = H >> 2;
        float4 wq[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int q = threadIdx.x + i * 256;
            wq[i] = q < nq ? __ldg((const float4*)w + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int q0 = 0; q0 < nq; q0 += 1024) {
            if (q0 > 0) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int q = q0 + threadIdx.x + i * 256;
                    wq[i] = q < nq ? __ldg((const float4*)w + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            for (int r = 0; r < nr; r++) {
                const float4* xr = (const float4*)(x + (size_t)(r0 + r) * H);
                float4 xq[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int q = q0 + threadIdx.x + i * 256;
                    xq[i] = q < nq ? __ldg(xr + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int q = q0 + threadIdx.x + i * 256;
                    if (q < nq)
                        *(float4*)(sprod + r * pitch + 4 * q) =
                            make_float4(__fmul_rn(wq[i].x, xq[i].x), __fmul_rn(wq[i].y, xq[i].y),
                                        __fmul_rn(wq[i].z, xq[i].z), __fmul_rn(wq[i].w, xq[i].w));
                }
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float wv = __ldg(w + c);
            for (int r = 0; r < nr; r++) sprod[r * pitch + c] = __fmul_rn(wv, __ldg(x + (size_t)(r0 + r) * H + c));
        }
    }
    __syncthreads();
    if (threadIdx.x < nr) {
        const float acc = serial_sum(sprod + threadIdx.x * pitch, H);
        logits[(size_t)(r0 + threadIdx.x) * E + e] = __fadd_rn(acc, bias ? bias[e] : 0.0f);
    }
}

// Decode batches of a few rows: one WARP per (expert, row).  Lane l forms the products of
// columns [l*CH, (l+1)*CH) in registers (H == 32*CH), then the reference chain
// acc = fl(acc + p[c]), c ascending (src/kernels.c:98-106), runs lane after lane: lane l
// takes the running value from lane l-1 and adds its CH products from registers, so each
// step costs one dependent-add latency and nothing else.
template <int CH>
__global__ void __launch_bounds__(32)
router_logits_warp_kernel(const float* __restrict__ W, const float* __restrict__ bias, const float* __restrict__ x,
                          float* __restrict__ logits, int E, int H) {
    const int e = blockIdx.x, r = blockIdx.y, lane = threadIdx.x;
    const float4* w4 = (const float4*)(W + (size_t)e * H + lane * CH);
    const float4* x4 = (const float4*)(x + (size_t)r * H + lane * CH);
    float p[CH];
#pragma unroll
    for (int i = 0; i < CH / 4; i++) {       // the router weights do not depend on the previous kernel
        const float4 wv = __ldg(w4 + i);
        p[4 * i + 0] = wv.x; p[4 * i + 1] = wv.y; p[4 * i + 2] = wv.z; p[4 * i + 3] = wv.w;
    }
    pdl_wait();
    pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < CH / 4; i++) {
        const float4 xv = x4[i];
        p[4 * i + 0] = __fmul_rn(p[4 * i + 0], xv.x);
        p[4 * i + 1] = __fmul_rn(p[4 * i + 1], xv.y);
        p[4 * i + 2] = __fmul_rn(p[4 * i + 2], xv.z);
        p[4 * i + 3] = __fmul_rn(p[4 * i + 3], xv.w);
    }
    float acc = 0.0f;
#pragma unroll 1
    for (int l = 0; l < 32; l++) {
        float a = __shfl_sync(0xffffffffu, acc, (l + 31) & 31);
        if (l == 0) a = 0.0f;
        if (lane == l) {
#pragma unroll
            for (int i = 0; i < CH; i++) a = __fadd_rn(a, p[i]);
            acc = a;
        }
    }
    if (lane == 31) logits[(size_t)r * E + e] = __fadd_rn(acc, bias ? bias[e] : 0.0f);
}

// Thread per (row, expert) for large batches: 8 experts x 8 rows per block of 64 threads
// (many small blocks: 64 rows x 128 experts already fill the GPU).  W and x stream through
// shared memory in 256-column slabs, four slabs deep with 16-byte cp.async copies, so the
// only thing a thread ever waits for is its own dependent-add chain.
constexpr int LT_SLAB = 256, LT_PITCH = LT_SLAB + 4, LT_STAGES = 4;

__global__ void __launch_bounds__(64)
router_logits_tile_kernel(const float* __restrict__ W, const float* __restrict__ bias, const float* __restrict__ x,
                          float* __restrict__ logits, int rows, int E, int H) {
    extern __shared__ __align__(16) float lt_sm[];      // [LT_STAGES][16][LT_PITCH]: 8 W rows, then 8 x rows
    const int tid = threadIdx.x;
    const int el = tid & 7, rl = tid >> 3;
    const int e0 = blockIdx.x * 8, row0 = blockIdx.y * 8;
    const int nslab = (H + LT_SLAB - 1) / LT_SLAB;
    auto issue = [&](int sl) {
        float* st = lt_sm + (size_t)(sl % LT_STAGES) * 16 * LT_PITCH;
        const int c0 = sl * LT_SLAB;
        const int pieces = (min(LT_SLAB, H - c0) + 3) >> 2;          // 16-byte pieces per row (H % 4 == 0)
        for (int p = tid; p < 16 * pieces; p += 64) {
            const int r = p / pieces, pc = p - r * pieces;
            const float* src;
            if (r < 8) src = W + (size_t)min(e0 + r, E - 1) * H + c0 + pc * 4;
            else src = x + (size_t)min(row0 + r - 8, rows - 1) * H + c0 + pc * 4;
            cp_async16(st + r * LT_PITCH + pc * 4, src);
        }
    };
    for (int sl = 0; sl < LT_STAGES - 1; sl++) {
        if (sl < nslab) issue(sl);
        cp_async_commit();
    }
    float acc = 0.0f;
    for (int sl = 0; sl < nslab; sl++) {
        cp_async_wait_dyn(LT_STAGES - 2);      // slab sl has landed (one group per slab, empty ones included)
        __syncthreads();                       // ... for every thread, and slab sl - 1 is no longer read
        if (sl + LT_STAGES - 1 < nslab) issue(sl + LT_STAGES - 1);
        cp_async_commit();
        const float* st = lt_sm + (size_t)(sl % LT_STAGES) * 16 * LT_PITCH;
        const float4* w4 = (const float4*)(st + el * LT_PITCH);
        const float4* x4 = (const float4*)(st + (8 + rl) * LT_PITCH);
        const int kc = min(LT_SLAB, H - sl * LT_SLAB);
        int c = 0;
#pragma unroll 4
        for (; c + 4 <= kc; c += 4) {
            const float4 wv = w4[c >> 2], xv = x4[c >> 2];
            acc = __fadd_rn(acc, __fmul_rn(wv.x, xv.x));
            acc = __fadd_rn(acc, __fmul_rn(wv.y, xv.y));
            acc = __fadd_rn(acc, __fmul_rn(wv.z, xv.z));
            acc = __fadd_rn(acc, __fmul_rn(wv.w, xv.w));
        }
    }
    const int e = e0 + el, row = row0 + rl;
    if (e < E && row < rows) logits[(size_t)row * E + e] = __fadd_rn(acc, bias ? bias[e] : 0.0f);
}

// Prefill-sized batches: 16 * RL threads as 16 experts x RL rows, each thread EPT x RPT outputs
// (independent dependent-add chains, so a warp always has an add to issue), tiles of
// 16*EPT experts x RL*RPT rows.  The 8 x 8 tiles above re-read W and x from L2 sixteen times
// more often per output than a 32 x 32 tile; past a few hundred rows that traffic, not the
// chains, set their time.
template <int EPT, int RPT, int RL>
struct LogitsBig {
    static constexpr int THREADS = 16 * RL;                  // 16 expert lanes x RL row lanes
    static constexpr int TE = 16 * EPT, TR = RL * RPT, ROWS = TE + TR;
    // the smallest tiles (one chain per lane, chosen when the grid would not fill the SMs otherwise) run one block
    // per SM: their copy ring is deep enough to cover the L2 latency of a slab that takes a third of a
    // microsecond to consume; the larger tiles keep three stages so that several blocks share an SM
    static constexpr int SLAB = 128, PITCH = SLAB + 4, STAGES = (RL == 8 && EPT == 1) ? 6 : 3;
    static constexpr size_t SMEM = (size_t)STAGES * ROWS * PITCH * sizeof(float);
};

// RL = 16 (256 threads, two blocks per SM) for a thousand rows and more; RL = 8 (128 threads: one warp per
// scheduler, so a warp's dependent-add chains never wait for an issue slot) for a few hundred rows, where
// the number of chains - rows x experts - is what limits the machine and the work should reach many SMs.
template <int EPT, int RPT, int RL>
__global__ void __launch_bounds__(16 * RL, RL == 16 ? 2 : 1)
router_logits_big_kernel(const float* __restrict__ W, const float* __restrict__ bias, const float* __restrict__ x,
                         float* __restrict__ logits, int rows, int E, int H) {
    using G = LogitsBig<EPT, RPT, RL>;
    extern __shared__ __align__(16) float lt_sm[];      // [STAGES][TE W rows, then TR x rows][PITCH]
    const int tid = threadIdx.x;
    const int el = tid & 15, rl = tid >> 4;
    const int e0 = blockIdx.x * G::TE, row0 = blockIdx.y * G::TR;
    const int nslab = (H + G::SLAB - 1) / G::SLAB;
    // a slab row is 32 pieces of 16 bytes: thread tid copies piece tid & 31 of rows tid >> 5, + THREADS / 32, ...
    const int pc = tid & 31;
    auto issue = [&](int sl) {
        float* st = lt_sm + (size_t)(sl % G::STAGES) * G::ROWS * G::PITCH;
        const int c = sl * G::SLAB + pc * 4;
        if (c >= H) return;
#pragma unroll
        for (int r = tid >> 5; r < G::ROWS; r += G::THREADS / 32) {
            const float* src = r < G::TE ? W + (size_t)min(e0 + r, E - 1) * H + c
                                         : x + (size_t)min(row0 + r - G::TE, rows - 1) * H + c;
            cp_async16(st + r * G::PITCH + pc * 4, src);
        }
    };
    for (int sl = 0; sl < G::STAGES - 1; sl++) {
        if (sl < nslab) issue(sl);
        cp_async_commit();
    }
    float acc[EPT][RPT];
#pragma unroll
    for (int i = 0; i < EPT; i++)
#pragma unroll
        for (int j = 0; j < RPT; j++) acc[i][j] = 0.0f;
    for (int sl = 0; sl < nslab; sl++) {
        cp_async_wait_dyn(G::STAGES - 2);
        __syncthreads();
        if (sl + G::STAGES - 1 < nslab) issue(sl + G::STAGES - 1);
        cp_async_commit();
        const float* st = lt_sm + (size_t)(sl % G::STAGES) * G::ROWS * G::PITCH;
        const int kc = min(G::SLAB, H - sl * G::SLAB);
#pragma unroll 2
        for (int c = 0; c + 4 <= kc; c += 4) {
            float4 wv[EPT], xv[RPT];
#pragma unroll
            for (int i = 0; i < EPT; i++) wv[i] = *(const float4*)(st + (el + 16 * i) * G::PITCH + c);
#pragma unroll
            for (int j = 0; j < RPT; j++) xv[j] = *(const float4*)(st + (G::TE + rl + RL * j) * G::PITCH + c);
#pragma unroll
            for (int i = 0; i < EPT; i++)
#pragma unroll
                for (int j = 0; j < RPT; j++) {
                    float a = acc[i][j];
                    a = __fadd_rn(a, __fmul_rn(wv[i].x, xv[j].x));
                    a = __fadd_rn(a, __fmul_rn(wv[i].y, xv[j].y));
                    a = __fadd_rn(a, __fmul_rn(wv[i].z, xv[j].z));
                    a = __fadd_rn(a, __fmul_rn(wv[i].w, xv[j].w));
                    acc[i][j] = a;
                }
        }
    }
#pragma unroll
    for (int i = 0; i < EPT; i++)
#pragma unroll
        for (int j = 0; j < RPT; j++) {
            const int e = e0 + el + 16 * i, row = row0 + rl + RL * j;
            if (e < E && row < rows) logits[(size_t)row * E + e] = __fadd_rn(acc[i][j], bias ? bias[e] : 0.0f);
        }
}

template <int EPT, int RPT, int RL>
static cudaError_t launch_logits_big(const float* W, const float* bias, const float* x, float* logits, int rows, int E,
                                     int H, cudaStream_t stream) {
    using G = LogitsBig<EPT, RPT, RL>;
    cudaError_t e = ensure_dynamic_smem((const void*)router_logits_big_kernel<EPT, RPT, RL>, G::SMEM);
    if (e != cudaSuccess) return e;
    dim3 grid((E + G::TE - 1) / G::TE, (rows + G::TR - 1) / G::TR);
    router_logits_big_kernel<EPT, RPT, RL><<<grid, G::THREADS, G::SMEM, stream>>>(W, bias, x, logits, rows, E, H);
    return cudaGetLastError();
}

// The same without alignment requirements (H not a multiple of 4, or unaligned operands):
// plain loads, 32 experts x 8 rows per block, 64-column slabs.
__global__ void __launch_bounds__(256)
router_logits_tile_plain_kernel(const float* __restrict__ W, const float* __restrict__ bias,
                                const float* __restrict__ x, float* __restrict__ logits, int rows, int E, int H) {
    __shared__ float sW[32][65];
    __shared__ float sX[8][64];
    const int el = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int e = blockIdx.x * 32 + el, row = blockIdx.y * 8 + rl;
    float acc = 0.0f;
    for (int c0 = 0; c0 < H; c0 += 64) {
        const int kc = min(64, H - c0);
        for (int i = threadIdx.x; i < 32 * 64; i += 256) {
            const int ee = i >> 6, cc = i & 63;
            const int ge = blockIdx.x * 32 + ee;
            sW[ee][cc] = (ge < E && cc < kc) ? W[(size_t)ge * H + c0 + cc] : 0.0f;
        }
        for (int i = threadIdx.x; i < 8 * 64; i += 256) {
            const int rr = i >> 6, cc = i & 63;
            const int gr = blockIdx.y * 8 + rr;
            sX[rr][cc] = (gr < rows && cc < kc) ? x[(size_t)gr * H + c0 + cc] : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int c = 0; c < kc; c++) acc = __fadd_rn(acc, __fmul_rn(sW[el][c], sX[rl][c]));
        __syncthreads();
    }
    if (e < E && row < rows) logits[(size_t)row * E + e] = __fadd_rn(acc, bias ? bias[e] : 0.0f);
}

cudaError_t launch_router_logits(const float* W, const float* bias, const float* x, float* logits, int rows, int E,
                                 int H, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    const bool aligned16 = ((((uintptr_t)W) | ((uintptr_t)x)) & 15) == 0;
    if (rows <= 4 && aligned16 && (H == 32 * 88 || H == 32 * 160)) {
        dim3 grid(E, rows);
        if (H == 32 * 88) return launch_pdl(router_logits_warp_kernel<88>, grid, dim3(32), 0, stream, W, bias, x, logits, E, H);
        return launch_pdl(router_logits_warp_kernel<160>, grid, dim3(32), 0, stream, W, bias, x, logits, E, H);
    }
    if (rows <= 32) {
        const int nr = rows < LOGIT_TB ? rows : LOGIT_TB;
        const size_t smem = (size_t)nr * (((H + 3) & ~3) + 4) * sizeof(float);
        if (smem > 48 * 1024) {
            cudaError_t e = ensure_dynamic_smem((const void*)router_logits_block_kernel, (size_t)(200 * 1024));
            if (e != cudaSuccess) return e;
        }
        if (smem > 200 * 1024) return cudaErrorInvalidValue;
        dim3 grid(E, (rows + LOGIT_TB - 1) / LOGIT_TB);
        router_logits_block_kernel<<<grid, 256, smem, stream>>>(W, bias, x, logits, rows, E, H);
    } else if (aligned16 && (H & 3) == 0 && rows >= 1024) {
        return launch_logits_big<2, 2, 16>(W, bias, x, logits, rows, E, H, stream);
    } else if (aligned16 && (H & 3) == 0 && rows >= 256) {
        // two chains per lane while that still gives every SM a block, else one chain per lane and twice the blocks
        if (((E + 31) / 32) * ((rows + 7) / 8) >= 148) return launch_logits_big<2, 1, 8>(W, bias, x, logits, rows, E, H, stream);
        return launch_logits_big<1, 1, 8>(W, bias, x, logits, rows, E, H, stream);
    } else if (aligned16 && (H & 3) == 0) {
        const size_t smem = (size_t)LT_STAGES * 16 * LT_PITCH * sizeof(float);
        {
            cudaError_t e = ensure_dynamic_smem((const void*)router_logits_tile_kernel, (size_t)((int)smem));
            if (e != cudaSuccess) return e;
        }
        dim3 grid((E + 7) / 8, (rows + 7) / 8);
        router_logits_tile_kernel<<<grid, 64, smem, stream>>>(W, bias, x, logits, rows, E, H);
    } else {
        dim3 grid((E + 31) / 32, (rows + 7) / 8);
        router_logits_tile_plain_kernel<<<grid, 256, 0, stream>>>(W, bias, x, logits, rows, E, H);
    }
    return cudaGetLastError();
}

__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ per_expert_scale,
                   int32_t* __restrict__ selected, float* __restrict__ weights, int E, int topk, int sort_by_expert,
                   int* status) {
    extern __shared__ __align__(16) float tk_sm[];
    float* sc = tk_sm + topk_scratch_floats(E, topk) - 4;
    topk_group(true, logits + (size_t)blockIdx.x * E, per_expert_scale, selected + (size_t)blockIdx.x * topk,
               weights + (size_t)blockIdx.x * topk, E, topk, sort_by_expert, status, tk_sm, sc, threadIdx.x,
               blockDim.x);
}

cudaError_t launch_router_topk(const float* logits, const float* per_expert_scale, int32_t* selected, float* weights,
                               int rows, int E, int topk, int sort_by_expert, int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    size_t smem = (size_t)topk_scratch_floats(E, topk) * sizeof(float);
    router_topk_kernel<<<rows, 128, smem, stream>>>(logits, per_expert_scale, selected, weights, E, topk,
                                                    sort_by_expert, status);
    return cudaGetLastError();
}

// ---- grouping ---------------------------------------------------------------
// Stable counting sort of the selections by expert (src/tensorops.c:239-289,
// src/moe_group.c:83-161): grouped order = expert ascending, then canonical
// index ascending.  One block; the canonical range is cut into 32 contiguous
// segments (one per warp), each warp histograms its segment, a scan over
// (expert, segment) gives every warp its starting slot per expert, and each
// warp then walks its segment in order, ranking equal experts inside a 32-wide
// step with match_any.  Experts outside [expert_begin, expert_end) keep their
// slots in the global order but get no job descriptor.
__global__ void __launch_bounds__(1024) moe_plan_kernel(MoePlanArgs a) {
    extern __shared__ __align__(16) int sp[];
    const int E = a.n_experts;
    if (a.logits != nullptr) {
        // fused router top-k for small batches: 128 threads per row, up to 8 rows
        float* tk = (float*)(sp + (34 * E + 4));
        const int grp = threadIdx.x >> 7, ltid = threadIdx.x & 127;
        const int per = topk_scratch_floats(E, a.topk);
        float* mine = tk + grp * per;
        const bool active = grp < a.rows;
        const int row = active ? grp : 0;
        topk_group(active, a.logits + (size_t)row * E, a.per_expert_scale, a.selected_out + (size_t)row * a.topk,
                   a.weights_out + (size_t)row * a.topk, E, a.topk, 1, a.status, mine, mine + per - 4, ltid, 128);
        __syncthreads();   // selections written by this block are read back below
    }
    int* hist = sp;               // [32][E]
    int* offs = sp + 32 * E;      // [E+1]
    int* act = offs + (E + 1);    // [E] active prefix
    const int jobs = a.rows * a.topk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = (jobs + 31) / 32;
    const int s0 = min(jobs, warp * seg), s1 = min(jobs, s0 + seg);
    for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = s0 + lane; i < s1; i += 32) {
        const int e = a.selected[i];
        if (e < 0 || e >= E) flag(a.status, SB_ERR_INDEX);
        else atomicAdd(&hist[warp * E + e], 1);
    }
    __syncthreads();
    // per expert: exclusive scan over segments, total count left in offs[e]
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int run = 0;
        for (int w = 0; w < 32; w++) {
            const int c = hist[w * E + e];
            hist[w * E + e] = run;
            run += c;
        }
        offs[e] = run;
    }
    __syncthreads();
    // exclusive scans over experts (E <= 1024 = one expert per thread): group
    // starts, and the compacted index of each local non-empty expert
    {
        __shared__ int warp_cnt[32], warp_act[32], s_max[32];
        const int e = threadIdx.x;
        const int c = e < E ? offs[e] : 0;
        const int local = (e < E && e >= a.expert_begin && e < a.expert_end && c > 0) ? 1 : 0;
        int pc = c, pa = local, mx = local ? c : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int tc = __shfl_up_sync(0xffffffffu, pc, o);
            const int ta = __shfl_up_sync(0xffffffffu, pa, o);
            if (lane >= o) { pc += tc; pa += ta; }
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (lane == 31) { warp_cnt[warp] = pc; warp_act[warp] = pa; }
        if (lane == 0) s_max[warp] = mx;
        __syncthreads();
        if (warp == 0) {
            int wc = warp_cnt[lane], wa = warp_act[lane], wm = s_max[lane];
            const int tot_c = wc, tot_a = wa;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int tc = __shfl_up_sync(0xffffffffu, wc, o);
                const int ta = __shfl_up_sync(0xffffffffu, wa, o);
                if (lane >= o) { wc += tc; wa += ta; }
                wm = max(wm, __shfl_xor_sync(0xffffffffu, wm, o));
            }
            warp_cnt[lane] = wc - tot_c;     // exclusive prefix of the warp totals
            warp_act[lane] = wa - tot_a;
            if (lane == 31) { offs[E] = wc; *a.n_active = wa; }
            if (lane == 0) *a.max_group = wm;
        }
        __syncthreads();
        if (e < E) {
            offs[e] = warp_cnt[warp] + pc - c;
            act[e] = local ? warp_act[warp] + pa - 1 : -1;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) a.group_offsets[e] = offs[e];
    // ordered placement
    for (int i0 = s0; i0 < s1; i0 += 32) {
        const int i = i0 + lane;
        const bool live = i < s1;
        int e = live ? a.selected[i] : -1;
        if (e < 0 || e >= E) e = -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
            const int before = __popc(peers & ((1u << lane) - 1u));
            const int slot = offs[e] + hist[warp * E + e] + before;
            a.grouped_to_canonical[slot] = i;
            a.canonical_to_grouped[i] = slot;
        }
        __syncwarp();
        if (e >= 0 && (peers >> lane) == 1u)  // highest lane of each peer set bumps the running base
            hist[warp * E + e] += __popc(peers);
        __syncwarp();
    }
    if (a.fused_done != nullptr && threadIdx.x < FUSED_MAX_JOBS) a.fused_done[threadIdx.x] = 0;
    __syncthreads();               // the placement is complete: the descriptors below read it back
    // job descriptors for the local, non-empty experts (ascending expert order)
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int slot = act[e];
        if (slot < 0) continue;
        const int g0 = offs[e], cnt = offs[e + 1] - offs[e];
        const uint8_t* base = a.pool + (size_t)e * a.expert_stride;
        Q4Job gu;
        gu.vals = base; gu.scales = base + a.value_bytes; gu.biases = base + a.value_bytes + a.group_bytes;
        gu.vals2 = base + a.tensor_bytes; gu.scales2 = gu.vals2 + a.value_bytes;
        gu.biases2 = gu.scales2 + a.group_bytes;
        gu.x = a.x; gu.y = a.chain + (size_t)g0 * a.inter;
        gu.x_rows = a.grouped_to_canonical + g0; gu.x_div = a.topk;
        gu.R = a.inter; gu.C = a.hidden; gu.ntok = cnt; gu.x_stride = a.hidden; gu.y_stride = a.inter;
        a.gateup_jobs[slot] = gu;
        Q4Job dn;
        dn.vals = base + 2 * a.tensor_bytes; dn.scales = dn.vals + a.value_bytes;
        dn.biases = dn.scales + a.group_bytes;
        dn.vals2 = nullptr; dn.scales2 = nullptr; dn.biases2 = nullptr;
        dn.x = a.chain + (size_t)g0 * a.inter; dn.y = a.grouped_out + (size_t)g0 * a.hidden;
        dn.x_rows = nullptr; dn.x_div = 1;
        dn.R = a.hidden; dn.C = a.inter; dn.ntok = cnt; dn.x_stride = a.inter; dn.y_stride = a.hidden;
        a.down_jobs[slot] = dn;
        if (a.fused_jobs != nullptr && slot < FUSED_MAX_JOBS) {
            FusedJob fj;
            fj.v[0] = gu.vals; fj.v[1] = gu.vals2; fj.v[2] = dn.vals;
            for (int k = 0; k < 3; k++)
                fj.t[k] = (const uint32_t*)(a.fused_tables + ((size_t)e * 6 + 2 * k) * a.group_bytes);
            for (int t = 0; t < FUSED_MAX_TOKENS; t++)
                fj.x_row[t] = a.grouped_to_canonical[g0 + min(t, cnt - 1)] / a.topk;
            fj.g0 = g0; fj.ntok = cnt; fj.lit = a.fused_lit[e]; fj.pad = 0;
            a.fused_jobs[slot] = fj;
        }
    }
}

// The same plan for at most 32 selections (decode batches of a few tokens), with the
// router top-k always fused: 128 threads per row run the top-k, then ONE warp places the
// selections (slot = selections with a smaller expert + earlier selections of the same
// expert, which is the stable counting sort) and every thread derives its experts' group
// starts and descriptors by counting over the <= 32 selections.  No histogram, no block
// scans: a handful of barriers instead of a dozen.
__global__ void __launch_bounds__(512) moe_plan_small_kernel(MoePlanArgs a) {
    extern __shared__ __align__(16) int sp[];
    const int E = a.n_experts;
    pdl_wait();                    // the logits come from the previous kernel
    pdl_launch_dependents();
    __shared__ int s_sel[32], s_first[32], s_g2c[32];
    if (a.fused_done != nullptr && threadIdx.x < FUSED_MAX_JOBS) a.fused_done[threadIdx.x] = 0;
    {
        float* tk = (float*)sp;
        const int grp = threadIdx.x >> 7, ltid = threadIdx.x & 127;
        const int per = topk_scratch_floats(E, a.topk);
        float* mine = tk + grp * per;
        const bool active = grp < a.rows;
        const int row = active ? grp : 0;
        topk_group(active, a.logits + (size_t)row * E, a.per_expert_scale, a.selected_out + (size_t)row * a.topk,
                   a.weights_out + (size_t)row * a.topk, E, a.topk, 1, a.status, mine, mine + per - 4, ltid, 128);
        __syncthreads();   // selections written by this block are read back below
    }
    const int jobs = a.rows * a.topk;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x < 32) {
        int e = lane < jobs ? a.selected[lane] : -1;
        if (lane < jobs && (e < 0 || e >= E)) { flag(a.status, SB_ERR_INDEX); e = -1; }
        int before = 0;
        bool first = true;
        for (int j = 0; j < jobs; j++) {
            const int ej = __shfl_sync(0xffffffffu, e, j);
            if (ej >= 0 && (ej < e || (ej == e && j < lane))) before++;
            if (ej == e && j < lane) first = false;
        }
        if (e >= 0) {
            a.grouped_to_canonical[before] = lane;
            a.canonical_to_grouped[lane] = before;
            s_g2c[before] = lane;
        }
        s_sel[lane] = e;
        s_first[lane] = (e >= 0 && first) ? 1 : 0;
    }
    __syncthreads();
    int valid = 0;
    for (int j = 0; j < jobs; j++) valid += s_sel[j] >= 0 ? 1 : 0;
    for (int e = threadIdx.x; e <= E; e += blockDim.x) {
        int lt = 0, eq = 0, slot = 0;
        for (int j = 0; j < jobs; j++) {
            const int ej = s_sel[j];
            if (ej < 0) continue;
            lt += ej < e ? 1 : 0;
            eq += ej == e ? 1 : 0;
            slot += (s_first[j] && ej < e && ej >= a.expert_begin && ej < a.expert_end) ? 1 : 0;
        }
        a.group_offsets[e] = e < E ? lt : valid;
        if (e == E || eq == 0 || e < a.expert_begin || e >= a.expert_end) continue;
        const int g0 = lt, cnt = eq;
        const uint8_t* base = a.pool + (size_t)e * a.expert_stride;
        Q4Job gu;
        gu.vals = base; gu.scales = base + a.value_bytes; gu.biases = base + a.value_bytes + a.group_bytes;
        gu.vals2 = base + a.tensor_bytes; gu.scales2 = gu.vals2 + a.value_bytes;
        gu.biases2 = gu.scales2 + a.group_bytes;
        gu.x = a.x; gu.y = a.chain + (size_t)g0 * a.inter;
        gu.x_rows = a.grouped_to_canonical + g0; gu.x_div = a.topk;
        gu.R = a.inter; gu.C = a.hidden; gu.ntok = cnt; gu.x_stride = a.hidden; gu.y_stride = a.inter;
        a.gateup_jobs[slot] = gu;
        Q4Job dn;
        dn.vals = base + 2 * a.tensor_bytes; dn.scales = dn.vals + a.value_bytes;
        dn.biases = dn.scales + a.group_bytes;
        dn.vals2 = nullptr; dn.scales2 = nullptr; dn.biases2 = nullptr;
        dn.x = a.chain + (size_t)g0 * a.inter; dn.y = a.grouped_out + (size_t)g0 * a.hidden;
        dn.x_rows = nullptr; dn.x_div = 1;
        dn.R = a.hidden; dn.C = a.inter; dn.ntok = cnt; dn.x_stride = a.inter; dn.y_stride = a.hidden;
        a.down_jobs[slot] = dn;
        if (a.fused_jobs != nullptr && slot < FUSED_MAX_JOBS) {
            FusedJob fj;
            fj.v[0] = gu.vals; fj.v[1] = gu.vals2; fj.v[2] = dn.vals;
            for (int k = 0; k < 3; k++)
                fj.t[k] = (const uint32_t*)(a.fused_tables + ((size_t)e * 6 + 2 * k) * a.group_bytes);
            for (int t = 0; t < FUSED_MAX_TOKENS; t++)
                fj.x_row[t] = s_g2c[g0 + min(t, cnt - 1)] / a.topk;
            fj.g0 = g0; fj.ntok = cnt; fj.lit = a.fused_lit[e]; fj.pad = 0;
            a.fused_jobs[slot] = fj;
        }
    }
    if (threadIdx.x == 0) {
        int n_active = 0, max_group = 0;
        for (int j = 0; j < jobs; j++) {
            const int ej = s_sel[j];
            if (!s_first[j] || ej < a.expert_begin || ej >= a.expert_end) continue;
            n_active++;
            int cnt = 0;
            for (int k = 0; k < jobs; k++) cnt += s_sel[k] == ej ? 1 : 0;
            max_group = max(max_group, cnt);
        }
        *a.n_active = n_active;
        *a.max_group = max_group;
    }
}

cudaError_t launch_moe_plan(const MoePlanArgs& a, cudaStream_t stream) {
    if (a.logits != nullptr && a.rows >= 1 && a.rows <= 4 && a.rows * a.topk <= 32) {
        const size_t small = (size_t)a.rows * topk_scratch_floats(a.n_experts, a.topk) * sizeof(float);
        if (small <= 40 * 1024) {
            return launch_pdl(moe_plan_small_kernel, dim3(1), dim3(128 * a.rows), small, stream, a);
        }
    }
    size_t smem = (size_t)(34 * a.n_experts + 4) * sizeof(int);
    if (a.logits != nullptr) {
        if (a.rows > 8) return cudaErrorInvalidValue;
        smem += (size_t)8 * topk_scratch_floats(a.n_experts, a.topk) * sizeof(float);
    }
    if (smem > 48 * 1024) {
        cudaError_t e = ensure_dynamic_smem((const void*)moe_plan_kernel, (size_t)(160 * 1024));
        if (e != cudaSuccess) return e;
    }
    if (smem > 160 * 1024) return cudaErrorInvalidValue;
    moe_plan_kernel<<<1, 1024, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace sb
