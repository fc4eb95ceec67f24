// Declarations shared by the translation units of libsalt_gpu_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sb {

struct Q4Job;

// ---- backend.cu ------------------------------------------------------------
// Raises a kernel's dynamic shared memory limit to at least `bytes` on the CURRENT device (the limit
// is a per-device attribute of the function; remembered per device and kernel, safe from any thread).
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes);

// ---- q4_kernels.cu -------------------------------------------------------
bool q4_tile_supported(int C);
// Runs every job (all share C and nmat).  njobs_dev (device int, may be null)
// bounds the live jobs when the count is only known on the device; blocks past
// it exit at once.  `aligned` promises 16-byte aligned tensors and x rows.
// pdl: -1 ordinary launch; 0 programmatic dependent launch, the jobs come from the previous
// kernel; 1 the same but the jobs (and njobs_dev) were written at least two launches back, so
// the weights are prefetched while the previous kernel is still running.
cudaError_t launch_q4_jobs(const Q4Job* jobs, int njobs_max, const int* njobs_dev, int max_rows, int max_tok, int C,
                           int nmat, bool aligned, cudaStream_t stream, int pdl = -1);

// ---- q4_fused_decode.cu ------------------------------------------------------
// Decode-sized expert execution in one launch (gate | up -> GeGLU -> down).
constexpr int FUSED_MAX_JOBS = 32;       // expert groups per launch
constexpr int FUSED_MAX_TOKENS = 4;      // activation rows per launch (and tokens per group)
struct FusedJob {
    const uint8_t* v[3];                       // packed values of gate, up, down (16-byte aligned)
    const uint32_t* t[3];                      // their derived tables: (scale bf16 << 16) | bias bf16 per group, [rows][C / 64]
    int32_t x_row[FUSED_MAX_TOKENS];           // activation row of each token of the group
    int32_t g0;                                // first grouped row (GeGLU rows and output rows g0, g0 + 1, ...)
    int32_t ntok;
    int32_t lit, pad;                          // lit bit k: tensor k has a scale that needs the two-rounding dequantisation
};
// Builds the derived tables of n_experts expert slots (gate | up | down, each values | scales | biases).
// words: [n_experts][3][groups] (groups = R * C / 64 of one tensor); flags: [n_experts].
cudaError_t launch_q4_interleave_tables(const uint8_t* pool, size_t expert_stride, size_t tensor_bytes, size_t value_bytes,
                                        size_t groups, int n_experts, uint32_t* words, int* flags, cudaStream_t stream);
struct FusedArgs {
    const FusedJob* jobs;        // [n_jobs_max]
    const int* n_jobs_dev;       // live jobs (device)
    int n_jobs_max;
    int* done;                   // [n_jobs_max] arrival counters, zero at launch
    const float* x;              // [n_x][x_stride] activation rows
    int x_stride, n_x;
    float* chain;                // [grouped rows][M]
    float* out;                  // [grouped rows][H]
    int H, M;
    int jobs_per_round;          // filled in by the launcher
    int* status;
};
struct FusedLaunch { int grid, jobs_per_round, tt; size_t smem; };
// Whether the fused kernel serves this geometry on the current device (and how it would be launched).
bool q4_fused_plan(int H, int M, int n_x, int n_jobs_max, FusedLaunch* out);
// Launched as a programmatic dependent launch; jobs, counters and x come from the previous kernel.
cudaError_t launch_q4_fused(const FusedArgs& args, cudaStream_t stream);

// One decode layer (one token) in one launch: [reduce + RMSNorm of the previous layer] -> router
// input -> logits -> top-k -> experts.
struct alignas(16) LayerDecodeArgs {
    FusedArgs f;                   // H, M, chain, out (this layer's grouped rows), done (this layer's counters), status
    const float* x_in;             // [H] the stack input, used when prev_grouped is null
    const float* prev_grouped;     // [topk][H] grouped outputs of the previous layer (rank order) or null
    const float* prev_weights;     // [topk]
    const float* norm_w;           // [H] RMSNorm weight applied to the reduced row, or null
    float eps_norm;
    float* y_out;                  // optional [H]: the layer's input row (block 0 writes it)
    const float* router_scale;     // [H]
    float eps_router;
    const float* router_w;         // [E][H]
    const float* per_expert_scale; // [E]
    float* logits;                 // [E]
    int* logits_count;             // arrival counter of this layer, zero at launch
    int E, topk, expert_begin, expert_end;
    int32_t* selected;             // [topk] outputs of block 0 ...
    float* weights_out;            // [topk] (a different buffer than prev_weights)
    int32_t *c2g, *g2c, *group_offsets;
    const uint8_t* pool;           // slot of expert e at pool + (e - expert_begin) * expert_stride
    const uint8_t* tables;         // derived scale | bias tables of the local experts
    const int* lit_flags;          // [local experts]
    size_t expert_stride, tensor_bytes, value_bytes, group_bytes;
};
bool q4_layer_decode_plan(int H, int M, int E, int topk, int n_jobs_max, FusedLaunch* out);
cudaError_t launch_q4_layer_decode(const LayerDecodeArgs& args, int n_jobs_max, cudaStream_t stream);
// All layers in one launch: d_layers [n_layers] arguments in device memory (f.jobs_per_round = the value of
// q4_layer_decode_jobs_per_round, f.n_x = 1), d_done [n_layers] arrival counters, zero at launch.
cudaError_t launch_q4_stack_decode(const LayerDecodeArgs* d_layers, int n_layers, int* d_done, int H, int M, int E, int topk,
                                   int n_jobs_max, cudaStream_t stream);
int q4_layer_decode_jobs_per_round(int H, int M, int E, int topk, int n_jobs_max);

// Affine 8-bit jobs (same descriptor; vals = one byte per element): one block per (row, token, job).
cudaError_t launch_q8_jobs(const Q4Job* jobs, int njobs, int max_rows, int max_tok, int C, cudaStream_t stream);

// ---- q4_gemm_tc.cu (tcgen05 / TMEM, tolerance path) --------------------------
cudaError_t launch_gather_convert(const float* x, const int32_t* g2c, void* xh, void* xl, int jobs, int topk,
                                  int hidden, cudaStream_t stream);
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
cudaError_t tensor_map_encoder(TensorMapEncodeFn* out);
// TMA descriptors of a [rows][cols] fp16 activation buffer and of its residual buffer:
// boxes of 64 columns x (16 << i) rows.
struct TcMaps {
    CUtensorMap hi[4];
    CUtensorMap lo[4];
};
cudaError_t make_tc_maps(TcMaps* out, const void* hi, const void* lo, int rows, int cols);
// fused: gate/up + GeGLU -> out_h (+ out_l) [grouped rows][R] fp16; plain: -> out_f [grouped rows][R] fp32.
// split: operands carried as hi + lo fp16 halves.  bmaps describes the activations (grouped order).
// Tiled maps over a layer's expert pool (packed nibbles) and its (scale << 16) | bias tables, one per tensor
// of an expert slot (gate, up, down); tab_tma[k]: tensor k's table rows are a multiple of 16 bytes and come
// by tiled copies (otherwise a row tile's table is copied whole).
struct TcWeightMaps {
    CUtensorMap w[3];
    CUtensorMap t[3];
    CUtensorMap w256[3];      // the same with boxes of 256 rows (wide single-precision kernel)
    CUtensorMap t256[3];
    const uint8_t* pool;
    size_t expert_stride;
    const uint32_t* tables;
    int tab_tma[3];
};
cudaError_t make_q4_tc_weight_maps(TcWeightMaps* out, const uint8_t* pool, size_t expert_stride, const uint32_t* tables,
                                   int hidden, int inter, int experts);
// Can the tensor-core kernels take this geometry?  Sizes must be multiples of 64; a size that is no multiple of
// 256 keeps a tile's scale table in shared memory and must not exceed 3520 (single) / 960 (hi + lo halves).
bool q4_tc_supported(int hidden, int inter, bool split);
// Work lists of a layer's two tensor-core launches (written on the device from the grouped jobs): items_* hold
// q4_tc_work_items_max() entries of 16 bytes each, work eight ints: {items, next, largest pass, -} of the fused
// launch, then of the plain one.
size_t q4_tc_work_items_max(int n_experts, int rows_total, int hidden, int inter);
cudaError_t launch_q4_tc_work_list(const Q4Job* gateup_jobs, const int* njobs_dev, int njobs_max, const float* y_base,
                                   int y_cols, const TcWeightMaps& wm, int hidden, int inter, void* items_fused,
                                   void* items_plain, int* work, cudaStream_t stream);
// items / work: this launch's list and its {items, next, largest pass} triple.  R, C: rows and columns of the weight matrices.
cudaError_t launch_q4_gemm_tc(bool fused, bool split, const void* items, int* work, const TcMaps& bmaps,
                              const TcWeightMaps& wm, void* out_h, void* out_l, float* out_f, int R, int C, int* status,
                              cudaStream_t stream);

// ---- bf16_kernels.cu ---------------------------------------------------------
// y[r] = W[r][:] . x in the reference's eight-accumulator order; ys[t][r] in the serial column order
cudaError_t launch_bf16_matvec(const uint16_t* W, const float* x, float* y, int R, int C, cudaStream_t stream);
cudaError_t launch_bf16_batch(const uint16_t* W, const float* xs, float* ys, int R, int C, int B, cudaStream_t stream);

// ---- nvfp4_kernels.cu ------------------------------------------------------
// One NVFP4 projection job: ntok rows of already dequantised activations.
struct Fp4Job {
    const uint8_t* codes;    // [R][C/2] E2M1, low nibble = even column
    const uint8_t* scales;   // [R][C/16] E4M3FN
    float wg;                // 1 / stored weight divisor
    const float* x;          // [ntok][x_stride] dequantised activations
    float* y;                // y[t*y_stride + r]
    int R, C, ntok, x_stride, y_stride;
};
// ig_rows[row] = input global scale of the row's tensor; src_rows (optional): row r reads activation row
// src_rows[r % src_mod] / src_div
// geglu_up (optional, without src_rows): quantise gelu_tanh(x[i]) * geglu_up[i] instead of x[i]
cudaError_t launch_nvfp4_qdq(const float* x, int rows, int C, const float* ig_rows, uint8_t* packed, uint8_t* scales,
                             float* dequant, int* status, cudaStream_t stream, const int* src_rows = nullptr,
                             int src_mod = 1, int src_div = 1, const float* geglu_up = nullptr);
// An NVFP4 expert: gate, up, down codes / block scales, 1 / weight divisor and input global scale of each.
struct Fp4ExpertDesc {
    const uint8_t* codes[3];
    const uint8_t* scales[3];
    float wg[3], ig[3];
};
// Jobs of a grouped NVFP4 MoE layer (gu_jobs: [2E] gate then up; dn_jobs: [E]; groups of remote experts get
// ntok = 0) and the per-row input global scales (ig_gu: [2J], ig_dn: [J]).
cudaError_t launch_nvfp4_moe_plan(const int* group_offsets, int E, int expert_begin, int expert_end, int J,
                                  const Fp4ExpertDesc* experts, int H, int M, const float* dq_gu, float* gate_out,
                                  float* up_out, const float* dq_dn, float* grouped_out, Fp4Job* gu_jobs, Fp4Job* dn_jobs,
                                  float* ig_gu, float* ig_dn, cudaStream_t stream, struct Fp4TcJob* tc_gu = nullptr,
                                  struct Fp4TcJob* tc_dn = nullptr, int* live = nullptr);
// ---- nvfp4_gemm_tc.cu: block-scaled tensor-core form of a grouped NVFP4 projection (tolerance path) ----
struct Fp4TcJob {
    float* y;                  // y[n * y_stride + m]
    float wg, ig;              // 1 / weight divisor, input global scale: y = acc * wg / ig
    int w_row0, ws_row0;       // the matrix' first row in the layer's code map and in its scale map
    int w_slice;               // the expert's slice in both
    int x_row0;                // the job's first row in the packed-activation map and in its scale map
    int ntok, R, y_stride;
};
struct Fp4TcMaps {
    CUtensorMap w, ws;         // weight codes and their block scales: bytes x rows x experts
    CUtensorMap x[3], xs[3];   // packed activations and their block scales: boxes of 16 / 32 / 64 rows
};
cudaError_t make_fp4_weight_scale_map(CUtensorMap* out, const void* base, int C, int rows, int slices, size_t slice_stride);
cudaError_t make_fp4_act_scale_maps(CUtensorMap* out3, const void* base, int C, int rows);
cudaError_t make_fp4_weight_map(CUtensorMap* out, const void* base, int C, int rows, int slices, size_t slice_stride);
cudaError_t make_fp4_act_maps(CUtensorMap* out3, const void* base, int C, int rows);
cudaError_t launch_nvfp4_gemm_tc(const Fp4TcJob* jobs, int njobs, int R, int C, const Fp4TcMaps& maps, int* status,
                                 cudaStream_t stream);
// live / n_live (optional, device): indices of the jobs that have tokens and their number; njobs is then the
// largest number of such jobs the call can have, and the grid spans only that many
cudaError_t launch_nvfp4_jobs(const Fp4Job* jobs, int njobs, int max_rows, int max_tok, int C, bool aligned,
                              cudaStream_t stream, const int* live = nullptr, const int* n_live = nullptr,
                              int typical_tok = 0);

// ---- router_kernels.cu ---------------------------------------------------
// Device-side error word: 0 = ok; set (never cleared) by kernels that meet a
// non-finite value or an invalid index, as the reference's CPU functions
// return -1 for them.
enum : int { SB_ERR_NONFINITE = 1, SB_ERR_INDEX = 2, SB_ERR_CAPACITY = 4, SB_ERR_TIMEOUT = 8 };

// y = (x * rsqrt(mean(x^2) + eps)) [* weight]        (rows independent)
cudaError_t launch_rmsnorm(const float* x, const float* weight, float* y, int rows, int n, float eps, int with_scale,
                           int* status, cudaStream_t stream);
// out = ((x * inv) * scale) * root; root <= 0 selects 1/sqrt(n)
cudaError_t launch_router_input(const float* x, const float* scale, float* out, int rows, int n, float eps,
                                float root, int* status, cudaStream_t stream);
// Consumers of the routed-expert output (reference gemma4.c:188-286), rows independent:
// out = residual + RMSNorm(branch)*weight
cudaError_t launch_residual_postnorm(const float* residual, const float* branch, const float* weight, float* out,
                                     int rows, int n, float eps, int* status, cudaStream_t stream);
// out = (residual + RMSNorm(RMSNorm(dense)*wd + RMSNorm(routed)*wr)*wf) * scalar; scratch_a/b = [rows][n] each
cudaError_t launch_parallel_combine(const float* residual, const float* dense, const float* routed, const float* wd,
                                    const float* wr, const float* wf, float* scratch_a, float* scratch_b, float* out,
                                    int rows, int n, float eps, float scalar, int* status, cudaStream_t stream);
// logits = cap * tanh(logits / cap), in place
cudaError_t launch_softcap(float* logits, int n, float cap, int* status, cudaStream_t stream);
// Fused per-row glue: [ordered weighted reduce] -> [RMSNorm] -> [router input].
struct GlueArgs {
    const float* weights;        // reduce: [rows*topk]; grouped == null skips the reduce
    const int32_t* c2g;
    const float* grouped;        // [jobs][n]
    int topk, jobs;
    const float* x_in;           // [rows][n], used when there is no reduce
    float* y_out;                // [rows][n] row after reduce/norm, or null
    const float* norm_w;         // [n] or null
    float eps_norm;
    const float* router_scale;   // [n] or null
    float eps_router;
    float* rin;                  // [rows][n]
    int n;
    int tables_late;             // weights / c2g are written by the kernel launched just before this one
    int* status;
};
cudaError_t launch_glue(const GlueArgs& a, int rows, cudaStream_t stream);
// logits[t][e] = serial dot of W[e][:] with x[t][:]  (+ bias[e])
cudaError_t launch_router_logits(const float* W, const float* bias, const float* x, float* logits, int rows, int E,
                                 int H, cudaStream_t stream);
// softmax top-k with renormalised weights, selections sorted by expert id
cudaError_t launch_router_topk(const float* logits, const float* per_expert_scale, int32_t* selected, float* weights,
                               int rows, int E, int topk, int sort_by_expert, int* status, cudaStream_t stream);

// Grouping of rows*topk selections by expert (stable counting sort) plus the
// job descriptors the expert kernels consume.
struct MoePlanArgs {
    // optional fused router top-k (rows <= 8): when logits != null the kernel first
    // computes selected_out / weights_out from the logits, and `selected` must alias selected_out
    const float* logits;
    const float* per_expert_scale;
    int32_t* selected_out;
    float* weights_out;
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
    // optional: descriptors and zeroed arrival counters of the fused decode kernel
    // (the first FUSED_MAX_JOBS local groups; the caller only uses them when there can be no more)
    FusedJob* fused_jobs;        // [FUSED_MAX_JOBS] or null
    int* fused_done;             // [FUSED_MAX_JOBS] or null
    const uint8_t* fused_tables; // derived scale | bias tables, expert e at fused_tables + e * 6 * group_bytes
    const int* fused_lit;        // [experts] indexed like the pool (globally; local slot 0 = expert_begin)
    int* status;
};
cudaError_t launch_moe_plan(const MoePlanArgs& a, cudaStream_t stream);

// ---- ep_exchange.cu ---------------------------------------------------------
// Exchange of grouped expert outputs between expert-parallel ranks over peer memory.
// A region = header (epoch) + two landing buffers of [rows_cap][width / 2] 16-byte slots.
enum : int { EP_MAX_WORLD = 8, EP_THREADS = 256, EP_HEADER_BYTES = 4096 };
enum : int { EP_PHASE_PUSH = 1, EP_PHASE_PULL = 2 };
enum : int { EP_DEFAULT_SPIN_LIMIT = 1 << 23 };
struct EpExchangeArgs {
    uint8_t* region[EP_MAX_WORLD];   // region[rank] is this device's own, the others are peer mappings
    int rank, world;
    const int32_t* group_offsets;    // [n_experts + 1], identical on every rank
    int expert_begin, expert_end, n_experts;
    float* grouped;                  // [rows][width]: own rows are read, the others written
    int width, rows_cap;
    int spin_limit;                  // polls of a slot before the wait gives up (EP_DEFAULT_SPIN_LIMIT: a few seconds)
    int phase;                       // EP_PHASE_PUSH | EP_PHASE_PULL; one at a time only when all
                                     // ranks share a device and their launches are serialised
    int* status;
};
size_t ep_region_bytes(int rows_cap, int width);
// rows = grouped rows of this call (all ranks'), sizes the grid
cudaError_t launch_ep_exchange(const EpExchangeArgs& a, int rows, cudaStream_t stream);

}  // namespace sb
