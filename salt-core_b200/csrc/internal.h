// Declarations shared by the translation units of libsalt_gpu_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sb {

struct Q4Job;

// ---- q4_kernels.cu -------------------------------------------------------
bool q4_tile_supported(int C);
// Runs every job (all share C and nmat).  njobs_dev (device int, may be null)
// bounds the live jobs when the count is only known on the device; blocks past
// it exit at once.  `aligned` promises 16-byte aligned tensors and x rows.
cudaError_t launch_q4_jobs(const Q4Job* jobs, int njobs_max, const int* njobs_dev, int max_rows, int max_tok, int C,
                           int nmat, bool aligned, cudaStream_t stream);

// ---- router_kernels.cu ---------------------------------------------------
// Device-side error word: 0 = ok; set (never cleared) by kernels that meet a
// non-finite value or an invalid index, as the reference's CPU functions
// return -1 for them.
enum : int { SB_ERR_NONFINITE = 1, SB_ERR_INDEX = 2, SB_ERR_CAPACITY = 4 };

// y = (x * rsqrt(mean(x^2) + eps)) [* weight]        (rows independent)
cudaError_t launch_rmsnorm(const float* x, const float* weight, float* y, int rows, int n, float eps, int with_scale,
                           int* status, cudaStream_t stream);
// out = ((x * inv) * scale) * root; root <= 0 selects 1/sqrt(n)
cudaError_t launch_router_input(const float* x, const float* scale, float* out, int rows, int n, float eps,
                                float root, int* status, cudaStream_t stream);
// logits[t][e] = serial dot of W[e][:] with x[t][:]  (+ bias[e])
cudaError_t launch_router_logits(const float* W, const float* bias, const float* x, float* logits, int rows, int E,
                                 int H, cudaStream_t stream);
// softmax top-k with renormalised weights, selections sorted by expert id
cudaError_t launch_router_topk(const float* logits, const float* per_expert_scale, int32_t* selected, float* weights,
                               int rows, int E, int topk, int sort_by_expert, int* status, cudaStream_t stream);

// Grouping of rows*topk selections by expert (stable counting sort) plus the
// job descriptors the expert kernels consume.
struct MoePlanArgs {
    const int32_t* selected;     // [rows*topk]
    int rows, topk, n_experts;
    int expert_begin, expert_end;  // experts owned by this device (others are skipped)
    int32_t* group_offsets;      // [E+1] start of each expert's group in grouped order
    int32_t* grouped_to_canonical;  // [jobs]
    int32_t* canonical_to_grouped;  // [jobs]
    int32_t* n_active;           // [1] number of non-empty local expert groups
    int32_t* max_group;          // [1] largest group
    // descriptor generation
    const uint8_t* pool;
    size_t expert_stride;
    size_t tensor_bytes;         // bytes of one Q4 tensor (values + scales + biases)
    size_t value_bytes, group_bytes;
    int hidden, inter;
    const float* x;              // [rows][hidden] layer input
    float* chain;                // [jobs][inter] grouped GeGLU output
    float* grouped_out;          // [jobs][hidden] grouped down output
    Q4Job* gateup_jobs;          // [E]
    Q4Job* down_jobs;            // [E]
    int* status;
};
cudaError_t launch_moe_plan(const MoePlanArgs& a, cudaStream_t stream);

// out[row] = sum over rank of fl(w * grouped[c2g[row*topk+rank]]) in rank order from 0
cudaError_t launch_weighted_reduce(const float* weights, const int32_t* canonical_to_grouped, const float* grouped,
                                   float* out, int rows, int topk, int width, int* status, cudaStream_t stream);
// routed[g] = x[grouped_to_canonical[g] / topk]
cudaError_t launch_routed_gather(const float* x, const int32_t* grouped_to_canonical, float* routed, int jobs,
                                 int topk, int hidden, cudaStream_t stream);

}  // namespace sb
