// Router, grouping and reduction kernels of the MoE feed-forward path.
//
// Everything here is bit-exact against the reference CPU functions; the
// reference arithmetic contains several chains that are serial by definition
// (sum of squares, router logits, softmax denominators).  Those chains are kept
// serial per row/expert and parallelism comes from running many of them side
// by side, with the independent products computed ahead by other lanes.
#include "internal.h"
#include "q4_core.cuh"

namespace sb {

static __device__ __forceinline__ void flag(int* status, int bit) {
    if (status) atomicOr(status, bit);
}

// Serial sum of squares of one row, in element order, as the reference does
// (gemma4.c:46-62, src/text_verify_cpu.c:642-655).  Lanes compute the squares
// of 32 consecutive elements in parallel; every lane then replays the same
// 32-step add chain on shuffled values, so only the adds are serial.
static __device__ __forceinline__ float serial_sum_squares_warp(const float* row_smem, int n, int lane) {
    float ss = 0.0f;
    int base = 0;
    for (; base + 32 <= n; base += 32) {
        const float v = row_smem[base + lane];
        const float sq = __fmul_rn(v, v);
#pragma unroll
        for (int j = 0; j < 32; j++) ss = __fadd_rn(ss, __shfl_sync(0xffffffffu, sq, j));
    }
    if (base < n) {
        const float v = (base + lane < n) ? row_smem[base + lane] : 0.0f;
        const float sq = __fmul_rn(v, v);
        for (int j = 0; j < n - base; j++) ss = __fadd_rn(ss, __shfl_sync(0xffffffffu, sq, j));
    }
    return ss;
}

// mode 0: RMSNorm  y = (x*inv) [* weight]             (gemma4.c:85-101)
// mode 1: router input  y = ((x*inv)*scale)*root      (gemma4.c:103-130)
template <int MODE>
__global__ void __launch_bounds__(256)
norm_rows_kernel(const float* __restrict__ x, const float* __restrict__ weight, float* __restrict__ y, int n,
                 float eps, int with_scale, float root_in, int* status) {
    extern __shared__ float srow[];
    __shared__ float s_inv, s_root;
    const float* xr = x + (size_t)blockIdx.x * n;
    float* yr = y + (size_t)blockIdx.x * n;
    bool bad = false;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i];
        srow[i] = v;
        bad |= !finite_f(v);
        if (MODE == 1 || with_scale) bad |= !finite_f(weight[i]);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const float ss = serial_sum_squares_warp(srow, n, threadIdx.x);
        if (threadIdx.x == 0) {
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

cudaError_t launch_rmsnorm(const float* x, const float* weight, float* y, int rows, int n, float eps, int with_scale,
                           int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    norm_rows_kernel<0><<<rows, 256, (size_t)n * sizeof(float), stream>>>(x, weight, y, n, eps, with_scale, 0.0f,
                                                                           status);
    return cudaGetLastError();
}

cudaError_t launch_router_input(const float* x, const float* scale, float* out, int rows, int n, float eps,
                                float root, int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    norm_rows_kernel<1><<<rows, 256, (size_t)n * sizeof(float), stream>>>(x, scale, out, n, eps, 1, root, status);
    return cudaGetLastError();
}

// One warp per (row, expert): the reference chain acc = fl(acc + fl(W[e][c]*x[c]))
// (src/kernels.c:98-106).  Lanes load W and x coalesced and form the products;
// the add chain is replayed by all lanes on shuffled products.
__global__ void __launch_bounds__(128)
router_logits_warp_kernel(const float* __restrict__ W, const float* __restrict__ bias, const float* __restrict__ x,
                          float* __restrict__ logits, int E, int H) {
    const int e = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int row = blockIdx.y;
    if (e >= E) return;
    const int lane = threadIdx.x & 31;
    const float* w = W + (size_t)e * H;
    const float* xr = x + (size_t)row * H;
    float acc = 0.0f;
    constexpr int G = 8;  // 32-column blocks fetched ahead: covers L2/HBM latency behind the add chain
    float pn[G];
#pragma unroll
    for (int b = 0; b < G; b++) {
        const int c = b * 32 + lane;
        pn[b] = (c < H) ? __fmul_rn(__ldg(w + c), __ldg(xr + c)) : 0.0f;
    }
    for (int g0 = 0; g0 < H; g0 += 32 * G) {
        float p[G];
#pragma unroll
        for (int b = 0; b < G; b++) p[b] = pn[b];
#pragma unroll
        for (int b = 0; b < G; b++) {
            const int c = g0 + 32 * G + b * 32 + lane;
            pn[b] = (c < H) ? __fmul_rn(__ldg(w + c), __ldg(xr + c)) : 0.0f;
        }
#pragma unroll
        for (int b = 0; b < G; b++) {
            const int left = H - (g0 + 32 * b);
            if (left >= 32) {
#pragma unroll
                for (int j = 0; j < 32; j++) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, p[b], j));
            } else {
                for (int j = 0; j < left; j++) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, p[b], j));
            }
        }
    }
    if (lane == 0) logits[(size_t)row * E + e] = __fadd_rn(acc, bias ? bias[e] : 0.0f);
}

// Thread per (row, expert) for large batches: 32 experts x 8 rows per block,
// W and x staged through shared memory in 64-column slabs.
__global__ void __launch_bounds__(256)
router_logits_tile_kernel(const float* __restrict__ W, const float* __restrict__ bias, const float* __restrict__ x,
                          float* __restrict__ logits, int rows, int E, int H) {
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
    if (rows <= 16) {
        dim3 grid((E + 3) / 4, rows);
        router_logits_warp_kernel<<<grid, 128, 0, stream>>>(W, bias, x, logits, E, H);
    } else {
        dim3 grid((E + 31) / 32, (rows + 7) / 8);
        router_logits_tile_kernel<<<grid, 256, 0, stream>>>(W, bias, x, logits, rows, E, H);
    }
    return cudaGetLastError();
}

// Softmax top-k (gemma4.c:132-186) + ascending-expert ordering of the selected
// pairs (gemma4_text.c:8541-8550).  The insertion top-k with strict '>' equals
// ranking by (logit descending, expert ascending); the softmax denominator and
// the renormalisation sum are serial chains in expert / rank order.
__global__ void __launch_bounds__(256)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ per_expert_scale,
                   int32_t* __restrict__ selected, float* __restrict__ weights, int E, int topk, int sort_by_expert,
                   int* status) {
    extern __shared__ float sm[];
    float* sl = sm;                  // [E] logits
    float* se = sm + E;              // [E] exp(l - max)
    int* ssel = (int*)(sm + 2 * E);  // [topk]
    float* sw = sm + 2 * E + topk;   // [topk]
    __shared__ float s_max, s_all, s_selsum;
    __shared__ int s_bad;
    const float* lr = logits + (size_t)blockIdx.x * E;
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const float v = lr[e];
        sl[e] = v;
        if (!finite_f(v) || (per_expert_scale && !finite_f(per_expert_scale[e]))) s_bad = 1;
    }
    __syncthreads();
    if (s_bad) {  // the reference rejects non-finite logits before ranking (gemma4.c:149-152)
        if (threadIdx.x == 0) flag(status, SB_ERR_NONFINITE);
        return;
    }
    if (threadIdx.x < 32) {
        float m = __int_as_float(0xff800000);
        for (int e = threadIdx.x; e < E; e += 32) m = fmaxf(m, sl[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) s_max = m;
    }
    __syncthreads();
    const float mx = s_max;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const float v = sl[e];
        se[e] = expf_exact(__fsub_rn(v, mx));
        int rank = 0;
        for (int o = 0; o < E; o++) {
            const float u = sl[o];
            rank += (u > v || (u == v && o < e)) ? 1 : 0;
        }
        if (rank < topk) ssel[rank] = e;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float all = 0.0f;
        for (int e = 0; e < E; e++) all = __fadd_rn(all, se[e]);
        s_all = all;
        if (!(all > 0.0f) || !finite_f(all)) s_bad = 1;
        float selsum = 0.0f;
        for (int j = 0; j < topk; j++) {
            const float w = __fdiv_rn(se[ssel[j]], all);
            sw[j] = w;
            selsum = __fadd_rn(selsum, w);
        }
        s_selsum = selsum;
        if (!(selsum > 0.0f) || !finite_f(selsum)) s_bad = 1;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < topk; j += blockDim.x) {
        const int e = ssel[j];
        const float nrm = __fdiv_rn(sw[j], s_selsum);
        const float w = __fmul_rn(nrm, per_expert_scale ? per_expert_scale[e] : 1.0f);
        int pos = j;
        if (sort_by_expert) {
            pos = 0;
            for (int i = 0; i < topk; i++) pos += (ssel[i] < e) ? 1 : 0;
        }
        selected[(size_t)blockIdx.x * topk + pos] = e;
        weights[(size_t)blockIdx.x * topk + pos] = w;
    }
    if (threadIdx.x == 0 && s_bad) flag(status, SB_ERR_NONFINITE);
}

cudaError_t launch_router_topk(const float* logits, const float* per_expert_scale, int32_t* selected, float* weights,
                               int rows, int E, int topk, int sort_by_expert, int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    size_t smem = (size_t)(2 * E + 2 * topk) * sizeof(float);
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
    extern __shared__ int sp[];
    const int E = a.n_experts;
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
    if (threadIdx.x == 0) {
        int run = 0, nact = 0, mg = 0;
        for (int e = 0; e < E; e++) {
            const int c = offs[e];
            offs[e] = run;
            run += c;
            const bool local = e >= a.expert_begin && e < a.expert_end && c > 0;
            act[e] = local ? nact : -1;
            if (local) { nact++; mg = max(mg, c); }
        }
        offs[E] = run;
        *a.n_active = nact;
        *a.max_group = mg;
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
    }
}

cudaError_t launch_moe_plan(const MoePlanArgs& a, cudaStream_t stream) {
    size_t smem = (size_t)(32 * a.n_experts + 2 * a.n_experts + 1) * sizeof(int);
    static bool configured = false;
    if (smem > 48 * 1024 && !configured) {
        cudaError_t e = cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    if (smem > 160 * 1024) return cudaErrorInvalidValue;
    moe_plan_kernel<<<1, 1024, smem, stream>>>(a);
    return cudaGetLastError();
}

// src/tensorops.c:291-325 / src/moe_group.c:211-224: per output element a
// serial chain over the ranks, starting from +0.
__global__ void __launch_bounds__(256)
weighted_reduce_kernel(const float* __restrict__ weights, const int32_t* __restrict__ c2g,
                       const float* __restrict__ grouped, float* __restrict__ out, int topk, int width, int jobs,
                       int* status) {
    const int row = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= width) return;
    float acc = 0.0f;
    for (int rank = 0; rank < topk; rank++) {
        const int canonical = row * topk + rank;
        const int g = c2g[canonical];
        const float w = weights[canonical];
        if (g < 0 || g >= jobs || !finite_f(w)) {
            if (d == 0) flag(status, g < 0 || g >= jobs ? SB_ERR_INDEX : SB_ERR_NONFINITE);
            continue;
        }
        acc = __fadd_rn(acc, __fmul_rn(w, grouped[(size_t)g * width + d]));
    }
    out[(size_t)row * width + d] = acc;
}

cudaError_t launch_weighted_reduce(const float* weights, const int32_t* canonical_to_grouped, const float* grouped,
                                   float* out, int rows, int topk, int width, int* status, cudaStream_t stream) {
    if (rows < 1) return cudaSuccess;
    dim3 grid((width + 255) / 256, rows);
    weighted_reduce_kernel<<<grid, 256, 0, stream>>>(weights, canonical_to_grouped, grouped, out, topk, width,
                                                     rows * topk, status);
    return cudaGetLastError();
}

__global__ void __launch_bounds__(256)
routed_gather_kernel(const float* __restrict__ x, const int32_t* __restrict__ g2c, float* __restrict__ routed,
                     int topk, int hidden) {
    const int g = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d < hidden) routed[(size_t)g * hidden + d] = x[(size_t)(g2c[g] / topk) * hidden + d];
}

cudaError_t launch_routed_gather(const float* x, const int32_t* grouped_to_canonical, float* routed, int jobs,
                                 int topk, int hidden, cudaStream_t stream) {
    if (jobs < 1) return cudaSuccess;
    dim3 grid((hidden + 255) / 256, jobs);
    routed_gather_kernel<<<grid, 256, 0, stream>>>(x, grouped_to_canonical, routed, topk, hidden);
    return cudaGetLastError();
}

}  // namespace sb
