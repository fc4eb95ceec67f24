/* salt_gpu_b200.h -- C ABI of libsalt_gpu_b200.so, a B200 (sm_100a) physical
 * backend for the quantized MoE feed-forward path of SALT-core.
 *
 * Part 1 declares the operator surface the reference engine links a GPU
 * backend through: every symbol the reference's stub backend defines
 * (reference src/gpu_stub.c:9-431), with the signatures of reference
 * include/salt/gpu.h.  A reference build links this library in place of its
 * own src/gpu_cuda.o; each declaration cites the reference line it replaces.
 * Operations outside the MoE-FFN path are present and fail closed (-1), exactly
 * like the stub.
 *
 * Part 2 is additive: device-resident entry points (salt_b200_*) so that
 * activations need not cross PCIe between layers.  They have no counterpart
 * in the reference.
 *
 * Conventions (reference include/salt/gpu.h:22-25): 0 = success, -1 =
 * unavailable or failed, never a partial result.  Pointers in Part 1 are
 * caller-owned HOST memory unless stated otherwise.  One calling thread at a
 * time.  There is no CPU fallback inside this library: if no CUDA device is
 * usable, salt_gpu_init() returns -1 and every operation fails.
 *
 * Deviation from the reference CUDA backend, by design: weights are COPIED into
 * HBM when a resource is activated (the reference reads host memory zero-copy,
 * which suits a unified-memory part and would be PCIe-bound here).  The copied
 * bytes are reported in SaltGpuWeightResourceUsage.device_copied_weight_bytes.
 */
#ifndef SALT_GPU_B200_H
#define SALT_GPU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ====================================================================== */
/* Part 1: the reference operator surface                                  */
/* ====================================================================== */

struct SaltTextGpuProgramOps;      /* reference include/salt/text_verify.h:746 */

/* Device-local residency (reference include/salt/gpu_residency.h:13, 26-36, 63-89).  The reference's state
 * machine (src/gpu_residency.c) owns seats, tickets, generations and leases; the backend supplies the
 * physical half: one HBM arena, pinned staging buffers, asynchronous staging->seat copies. */
#define SALT_GPU_RESIDENCY_ABI_VERSION 1u
typedef struct SaltGpuResidencyPlan {
    uint64_t device_budget_bytes; /* whole arena */
    uint64_t permanent_bytes;     /* leading part that is never evicted */
    uint64_t slot_base_offset;    /* first seat, a multiple of device_alignment */
    uint64_t slot_bytes;          /* seat stride */
    uint64_t staging_bytes;       /* one pinned staging buffer, >= the largest payload */
    uint32_t slot_count, staging_count;
    uint32_t device_alignment, flags;
} SaltGpuResidencyPlan;
struct SaltGpuResidencyPermanentLayout; /* gpu_residency.h:51 (permanent population: not provided) */
struct SaltGpuResidencyPermanentSpan;   /* gpu_residency.h:58 */
typedef struct SaltGpuResidencyBackendOps {
    uint32_t abi_version;
    size_t ops_size;
    int (*create)(void *context, const SaltGpuResidencyPlan *plan);
    int (*staging)(void *context, uint32_t staging_slot, void **address, size_t *capacity);
    int (*populate)(void *context, uint32_t physical_slot, uint64_t device_offset, uint32_t staging_slot,
                    size_t nbytes, uint64_t ticket);
    int (*poll)(void *context, uint32_t physical_slot, uint64_t ticket, int *complete);
    int (*resolve)(void *context, uint64_t device_offset, size_t nbytes, uintptr_t *address);
    int (*retire)(void *context, uint32_t physical_slot, uint64_t generation);
    int (*destroy)(void *context);
    int (*permanent_layout)(void *context, struct SaltGpuResidencyPermanentLayout *layout, size_t layout_size);
    int (*permanent_span)(void *context, uint32_t span_index, struct SaltGpuResidencyPermanentSpan *span,
                          size_t span_size);
    int (*permanent_copy)(void *context, uint32_t span_index, uint64_t device_offset, uint32_t staging_slot,
                          size_t nbytes, uint64_t ticket);
    int (*permanent_publish)(void *context);
} SaltGpuResidencyBackendOps;

/* gpu.h:102-109 */
typedef struct SaltGpuBatchStats {
    uint64_t arena_batches, trunk_batches, expert_layer_batches;
    uint64_t mapped_only_misses, direct_output_batches, direct_output_jobs;
} SaltGpuBatchStats;

/* gpu.h:111-132 */
typedef struct SaltGpuBatchStatsV2 {
    uint64_t arena_batches, trunk_batches, expert_layer_batches;
    uint64_t mapped_only_misses, direct_output_batches, direct_output_jobs;
    uint64_t nvfp4_logical_packed_weight_bytes, nvfp4_logical_weight_scale_bytes;
    uint64_t nvfp4_activation_input_bytes, nvfp4_activation_qdq_bytes;
    uint64_t nvfp4_projection_output_bytes, nvfp4_kernel_launches;
    uint64_t nvfp4_completion_fences;
    uint64_t nvfp4_h2d_ns, nvfp4_qdq_ns, nvfp4_projection_ns, nvfp4_d2h_ns;
    uint64_t q4_weight_stationary_batches;
} SaltGpuBatchStatsV2;

/* gpu.h:140-157 */
typedef struct SaltGpuBatchDesc {
    const uint32_t *const *vals;
    const uint16_t *const *scales;
    const uint16_t *const *biases;
    const float *const *xs;
    float *const *ys;
    const void *const *ids;
    const int *Rj;
    int C, njobs;
} SaltGpuBatchDesc;

typedef struct SaltGpuDispatch {
    const char *name;
    int (*init)(void **state);
    int (*replay)(void *state, const SaltGpuBatchDesc *d);
    void (*destroy)(void *state);
} SaltGpuDispatch;

/* gpu.h:198-202: host-visible storage that is also a device buffer.
 * contents = pinned host pointer, backend = its device alias. */
typedef struct SaltGpuSharedBuffer {
    void *contents;
    size_t nbytes;
    void *backend;
} SaltGpuSharedBuffer;

/* gpu.h:211-234 */
typedef enum SaltGpuExactCellKind {
    SALT_GPU_EXACT_RMSNORM = 1,
    SALT_GPU_EXACT_TOPK = 2,
    SALT_GPU_EXACT_RESIDUAL_POSTNORM = 3,
    SALT_GPU_EXACT_PARALLEL_COMBINE = 4,
    SALT_GPU_EXACT_SOFTCAP = 5,
    SALT_GPU_EXACT_ROUTER_INPUT = 6
} SaltGpuExactCellKind;

typedef struct SaltGpuExactCell {
    SaltGpuExactCellKind kind;
    SaltGpuSharedBuffer *views[8];
    size_t offsets[8];
    uint32_t n;
    uint32_t aux;
    float eps;
    float scalar;
} SaltGpuExactCell;

/* gpu.h:276-295 */
typedef struct SaltGpuMoeExpert {
    const uint32_t *gate_vals;
    const uint16_t *gate_scales;
    const uint16_t *gate_biases;
    const void *gate_id;
    const uint32_t *up_vals;
    const uint16_t *up_scales;
    const uint16_t *up_biases;
    const void *up_id;
    const uint32_t *down_vals;
    const uint16_t *down_scales;
    const uint16_t *down_biases;
    const void *down_id;
    int group;
    int resource_slot;
    uint64_t logical_resource_id;
} SaltGpuMoeExpert;

/* gpu.h:297-309 */
typedef struct SaltGpuSelectedProjectionJob {
    const uint32_t *vals;
    const uint16_t *scales;
    const uint16_t *biases;
    const void *id;
    const float *inputs;
    float *outputs;
    int rows;
    int cols;
    int batch;
    int resource_slot;
    uint64_t logical_resource_id;
} SaltGpuSelectedProjectionJob;

/* gpu.h:411-416 */
typedef enum SaltGpuWeightAddressability {
    SALT_GPU_WEIGHT_ADDRESS_AUTO = 0,
    SALT_GPU_WEIGHT_ADDRESS_BOUNDED_WINDOW = 1,
    SALT_GPU_WEIGHT_ADDRESS_REGISTERED_PERSISTENT = 2,
    SALT_GPU_WEIGHT_ADDRESS_PAGEABLE = 3
} SaltGpuWeightAddressability;

/* gpu.h:418-429 */
typedef struct SaltGpuWeightResourceUsage {
    uint64_t described_bytes, registered_bytes, pageable_bytes;
    uint64_t active_window_bytes, peak_window_bytes, device_copied_weight_bytes;
    uint32_t described_resources, active_resources, active_windows, reserved;
} SaltGpuWeightResourceUsage;

/* gpu.h:431-440 */
typedef struct SaltGpuStartupRequirements {
    uint64_t fixed_device_bytes, fixed_pinned_host_bytes, descriptor_bytes;
    uint64_t device_copied_weight_bytes;
    uint32_t max_output_floats, max_batch_jobs, shared_buffer_slots, reserved;
} SaltGpuStartupRequirements;

/* resource kinds, reference include/salt/gpu_resource.h:10-14 */
enum { SALT_GPU_RESOURCE_ARENA = 0, SALT_GPU_RESOURCE_TRUNK = 1, SALT_GPU_RESOURCE_EXPERT_LAYER = 2 };

/* ---- lifecycle ------------------------------------------------------- */
int salt_gpu_init(void);                                                    /* gpu.h:26 */
int salt_gpu_free(void);                                                    /* gpu.h:27 */
int salt_gpu_startup_requirements(SaltGpuStartupRequirements *r, size_t n); /* gpu.h:443 */
int salt_gpu_set_defer(int on);                                             /* gpu.h:190 */
int salt_gpu_defer(void);                                                   /* gpu.h:191 */
int salt_gpu_sync(void);                                                    /* gpu.h:192 */
void salt_gpu_set_mapped_only(int on);                                      /* gpu.h:99 */
int salt_gpu_mapped_only(void);                                             /* gpu.h:100 */
void salt_gpu_batch_stats_get(SaltGpuBatchStats *stats);                    /* gpu.h:134 */
int salt_gpu_batch_stats_get_v2(SaltGpuBatchStatsV2 *stats, size_t n);      /* gpu.h:135 */
const SaltGpuDispatch *salt_dispatch_get(void);                             /* gpu.h:163, NULL */
int salt_gpu_cuda_present(void);                                            /* gpu.h:168, 1 */
int salt_gpu_rocm_present(void);                                            /* gpu.h:170, 0 */
int salt_gpu_pageable_mmap_active(void);                                    /* gpu.h:173, 0 */
const struct SaltTextGpuProgramOps *salt_gpu_tensor_program_ops(void);      /* gpu.h:209, NULL */
const struct SaltGpuResidencyBackendOps *salt_gpu_residency_backend_ops(void); /* gpu_residency.h:147 */

/* ---- weight resources (gpu.h:443-487, 380-409) ------------------------ */
int salt_gpu_weight_resource_describe(uint32_t kind, uint32_t id, const void *base, size_t nbytes);
int salt_gpu_weight_resource_activate(uint32_t kind, uint32_t id, SaltGpuWeightAddressability policy);
int salt_gpu_weight_resource_pool_bind(uint32_t kind, uint32_t id);
int salt_gpu_weight_resource_deactivate(uint32_t kind, uint32_t id);
int salt_gpu_weight_resource_usage(SaltGpuWeightResourceUsage *usage, size_t n);
int salt_gpu_weight_resource_bind(uint32_t kind, uint32_t id, const void *base, size_t nbytes);
int salt_gpu_weight_window_bind(uint32_t kind, uint32_t id, uint64_t offset, size_t nbytes);
int salt_gpu_weight_window_unbind(uint32_t kind, uint32_t id);
int salt_gpu_weight_resource_slot(uint32_t kind, uint32_t id, const void *key, const uint32_t *vals,
                                  const uint16_t *scales, const uint16_t *biases, int bits, int R, int C);
int salt_gpu_nvfp4_resource_slot(uint32_t kind, uint32_t id, const void *key, const uint8_t *weight_packed,
                                 const uint8_t *weight_scales, const float *weight_global_scale,
                                 const float *input_global_scale, int R, int C);
int salt_gpu_bf16_resource_slot(uint32_t kind, uint32_t id, const void *key, const uint16_t *weights, int R,
                                int C);                                      /* gpu.h:60, -1 */
int salt_gpu_weight_resource_unbind(uint32_t kind, uint32_t id);
int salt_gpu_resident_trunk_map(const void *base, size_t nbytes);           /* gpu.h:180 */
int salt_gpu_resident_trunk_unmap(void);                                    /* gpu.h:183 */
int salt_gpu_resident_pool_map(const void *base, size_t nbytes);            /* gpu.h:484 */
int salt_gpu_resident_slot(const void *key, const uint32_t *vals, const uint16_t *scales,
                           const uint16_t *biases, int R, int C);           /* gpu.h:392 */
int salt_gpu_expert_resource_bind(uint32_t id, const void *base, size_t nbytes);   /* gpu.h:403 */
int salt_gpu_expert_resource_slot(uint32_t id, const void *key, const uint32_t *vals, const uint16_t *scales,
                                  const uint16_t *biases, int R, int C);    /* gpu.h:405 */
int salt_gpu_expert_resource_unbind(uint32_t id);                           /* gpu.h:409 */

/* ---- selected-expert table (gpu.h:335-347) ---------------------------- */
int salt_gpu_selected_resources_prepare(int capacity, int logical_capacity);
int salt_gpu_selected_resource_bind(int slot, uint64_t logical_id, const void *base, size_t nbytes,
                                    const void *payload);
int salt_gpu_selected_resource_bind_resident(int slot, uint64_t logical_id, const void *payload, size_t nbytes,
                                             uintptr_t device_address, uint64_t generation);
int salt_gpu_selected_resources_fence(void);
int salt_gpu_selected_resource_unbind(int slot, uint64_t logical_id);

/* ---- affine-Q4 compute ------------------------------------------------ */
int salt_gpu_q4_matvec(const uint32_t *vals, const uint16_t *scales, const uint16_t *biases, int R, int C,
                       const float *x, float *y);                           /* gpu.h:34 */
int salt_gpu_q4_batch(const uint32_t *const *vals, const uint16_t *const *scales, const uint16_t *const *biases,
                      const float *const *xs, float *const *ys, const void *const *ids, const int *Rj, int C,
                      int njobs);                                            /* gpu.h:83 */
int salt_gpu_proj_batch(const uint32_t *vals, const uint16_t *scales, const uint16_t *biases, int R, int C, int B,
                        const float *const *xs, float *const *ys, const void *id);   /* gpu.h:388 */
int salt_gpu_proj_batch_indexed(const uint32_t *vals, const uint16_t *scales, const uint16_t *biases, int R,
                                int C, int B, int first_job, int job_count, const float *xs,
                                SaltGpuSharedBuffer *output, size_t y_float_offset, const void *id); /* gpu.h:354 */
int salt_gpu_proj_batch_indexed_exact_views(const uint32_t *vals, const uint16_t *scales, const uint16_t *biases,
                                            int R, int C, int B, int first_job, int job_count, const float *xs,
                                            SaltGpuSharedBuffer *output, size_t y_float_offset,
                                            const void *id);                /* gpu.h:363 */
int salt_gpu_q4_selected_shared(const SaltGpuSelectedProjectionJob *jobs, int job_count,
                                SaltGpuSharedBuffer *arena);                /* gpu.h:314 */
int salt_gpu_q4_moe_chain(const SaltGpuMoeExpert *experts, int count, int hidden, int routed, const float *inputs,
                          float *outputs, float *gate_scratch, float *up_scratch,
                          size_t scratch_float_capacity);                   /* gpu.h:320 */
int salt_gpu_q4_moe_chain_selected(const SaltGpuMoeExpert *experts, int count, int hidden, int routed,
                                   const float *inputs, float *outputs, float *gate_scratch, float *up_scratch,
                                   size_t scratch_float_capacity);          /* gpu.h:325 */

/* ---- NVFP4 compute (gpu.h:41-59) --------------------------------------- */
int salt_gpu_nvfp4_qdq(const float *input, int C, float input_global_scale, uint8_t *packed, uint8_t *scales,
                       float *dequant);
int salt_gpu_nvfp4_matvec(const void *key, int R, int C, const float *input, float *output);
int salt_gpu_nvfp4_matvec_batch(const void *key, int R, int C, int B, const float *inputs, float *outputs);
int salt_gpu_nvfp4_batch(const void *const *keys, const float *const *inputs, float *const *outputs,
                         const int *batches, int R, int C, int njobs);
int salt_gpu_nvfp4_mixed_batch(const void *const *keys, const float *const *inputs, float *const *outputs,
                               const int *batches, const int *rows, int C, int njobs);

/* ---- exact cells and shared buffers (gpu.h:198-234) -------------------- */
int salt_gpu_shared_buffer_alloc(SaltGpuSharedBuffer *buffer, size_t nbytes);
int salt_gpu_shared_buffer_free(SaltGpuSharedBuffer *buffer);
int salt_gpu_exact_cells(const SaltGpuExactCell *cells, int count);

/* ---- present, fail closed: outside the MoE-FFN path -------------------- */
int salt_gpu_q8_matvec(const uint32_t *vals, const uint16_t *scales, const uint16_t *biases, int R, int C,
                       const float *x, float *y);                           /* gpu.h:37 */
int salt_gpu_q8_batch(const uint32_t *const *vals, const uint16_t *const *scales, const uint16_t *const *biases,
                      const float *const *xs, float *const *ys, const void *const *ids, const int *Rj, int C,
                      int njobs);                                            /* gpu.h:89 */
int salt_gpu_bf16_matvec(const void *key, int R, int C, const float *input, float *output);        /* gpu.h:63 */
int salt_gpu_bf16_matvec_batch(const void *key, int R, int C, int B, const float *inputs, float *outputs);
int salt_gpu_attention_batch(int full_attention, int n_heads, int n_kv_heads, int head_dim, int window,
                             const SaltGpuSharedBuffer *queries, size_t query_float_offset,
                             const SaltGpuSharedBuffer *kv, size_t key_float_offset, size_t value_float_offset,
                             int start_position, int batch, int query_stride, int kv_stride,
                             SaltGpuSharedBuffer *outputs, size_t output_float_offset,
                             SaltGpuSharedBuffer *score_workspace, size_t score_float_offset,
                             size_t score_stride, int score_task_capacity);  /* gpu.h:239 */
int salt_gpu_attention_prepare(const SaltGpuSharedBuffer *kv);
int salt_gpu_attention_bind_kv(size_t key_float_offset, size_t value_float_offset, int kv_stride);
int salt_gpu_attention_materialize(SaltGpuSharedBuffer *kv, int position, uint64_t *copied_bytes);
int salt_gpu_attention_import(SaltGpuSharedBuffer *kv, int position, uint64_t *copied_bytes);
int salt_gpu_attention_rewind(int position);
int salt_gpu_attention_transform(int n_heads, int n_kv_heads, int head_dim, int rope_dim, int start_position,
                                 int batch, int query_stride, int kv_stride, float eps,
                                 SaltGpuSharedBuffer *queries, size_t query_float_offset,
                                 SaltGpuSharedBuffer *keys, size_t key_float_offset, SaltGpuSharedBuffer *values,
                                 size_t value_float_offset, const float *q_weight, const float *k_weight,
                                 const float *cosines, const float *sines, int rope_pairs,
                                 SaltGpuSharedBuffer *kv, size_t key_cache_float_offset,
                                 size_t value_cache_float_offset);           /* gpu.h:262 */

/* ====================================================================== */
/* Part 2: device-resident MoE stack (no counterpart in the reference)     */
/* ====================================================================== */

/* One MoE feed-forward layer with affine-Q4 experts.  All pointers are HOST
 * memory; salt_b200_stack_add_q4_layer copies them into HBM.  The pool holds
 * n_experts slots of expert_stride bytes, each gate | up | down, each tensor
 * values | scales | biases (the slot order of the reference's expert pool,
 * tools/gemma4-mlx4-source.py:180-199).  norm_weight, when not NULL, is the
 * RMSNorm weight applied to this layer's output before the next layer. */
typedef struct SaltB200Q4LayerSpec {
    int hidden, inter, n_experts, topk;
    float eps;
    const float *router_w;          /* [n_experts][hidden] fp32 */
    const float *router_scale;      /* [hidden] */
    const float *per_expert_scale;  /* [n_experts] */
    const void *pool;
    size_t expert_stride;
    const float *norm_weight;       /* [hidden] or NULL */
} SaltB200Q4LayerSpec;

/* Device pointers of the per-call workspace, for callers that run their own
 * exchange step between the expert phase and the combine phase. */
typedef struct SaltB200Workspace {
    float *grouped_out;             /* [max_tokens*topk][hidden], grouped order */
    int32_t *group_offsets;         /* [n_experts+1] */
    int32_t *selected;              /* [max_tokens*topk] sorted by expert within a token */
    float *weights;                 /* [max_tokens*topk] */
    int32_t *canonical_to_grouped;  /* [max_tokens*topk] */
    int32_t *grouped_to_canonical;  /* [max_tokens*topk] */
    float *logits;                  /* [max_tokens][n_experts] */
    int32_t *status;                /* device error word */
    size_t grouped_out_bytes;
} SaltB200Workspace;

/* Experts [expert_begin, expert_end) of every layer live on this device; other
 * experts' weights are not uploaded and their selections are left untouched in
 * grouped_out (expert-parallel sharding).  Pass 0, n_experts for one GPU. */
int salt_b200_stack_create(int max_tokens, int hidden, int inter, int n_experts, int topk, int expert_begin,
                           int expert_end, void **stack_out);
int salt_b200_stack_destroy(void *stack);
int salt_b200_stack_add_q4_layer(void *stack, const SaltB200Q4LayerSpec *spec);
/* A layer whose experts are NVFP4 (W4A4: E2M1 codes two per byte, one E4M3FN scale per 16 elements, a
 * stored per-tensor weight divisor and an input global scale; reference src/nvfp4.c:82-130, 228-256).  The
 * device sequence is what models/gemma4-26b-a4b/src/gemma4_text.c:8912-8945 runs from the host: quantise-
 * dequantise the routed rows with each tensor's input global scale, gate and up projections, GeGLU,
 * quantise-dequantise again, down projection; router, grouping and the ordered reduce are those of the
 * affine-Q4 layers.  Expert slot in `pool`: gate codes [inter][hidden/2] | gate scales [inter][hidden/16] |
 * up codes | up scales | down codes [hidden][inter/2] | down scales [hidden][inter/16].
 * weight_divisors, input_globals: [n_experts][3] (gate, up, down).  hidden and inter must be multiples of 256. */
typedef struct SaltB200Nvfp4LayerSpec {
    int hidden, inter, n_experts, topk;
    float eps;
    const float *router_w, *router_scale, *per_expert_scale;
    const void *pool;
    size_t expert_stride;
    const float *weight_divisors, *input_globals;
    const float *norm_weight;       /* [hidden] or NULL */
} SaltB200Nvfp4LayerSpec;
int salt_b200_stack_add_nvfp4_layer(void *stack, const SaltB200Nvfp4LayerSpec *spec);
int salt_b200_stack_workspace(void *stack, SaltB200Workspace *out);
/* Intermediate buffers of the NVFP4 layers after salt_b200_layer_experts (for inspection and stage-wise
 * checks): the gate and up projection outputs [rows][inter] in grouped order, and the quantised GeGLU
 * output that feeds the down projection, packed E2M1 codes [rows][inter/2] and E4M3 block scales
 * [rows][inter/16].  -1 when the stack holds no NVFP4 layer. */
typedef struct SaltB200Nvfp4Buffers {
    const float *gate, *up;
    const uint8_t *chain_codes, *chain_scales;
} SaltB200Nvfp4Buffers;
int salt_b200_stack_nvfp4_buffers(void *stack, SaltB200Nvfp4Buffers *out);
/* Batches of up to 4 tokens run gate/up, GeGLU and down of all selected experts in ONE launch
 * (one persistent block per SM, weights of both phases in flight from the start; the reference
 * runs the three projections as separate calls, models/gemma4-26b-a4b/src/gemma4_text.c:7971-7997).
 * A forward pass of ONE token over affine-Q4 layers goes further: level 1 (the default) runs each layer
 * (reduce, norm, router, top-k, experts) as one launch; level 2 runs ALL layers of the pass in one launch
 * whose blocks stay resident, a layer ending with an arrival counter instead of a kernel boundary (one
 * launch per pass for hosts where launches are the cost; on a B200 with graph replay it measured 49.1 us
 * per layer against 46.3 us for level 1, whose programmatic dependent launches overlap a layer's prologue
 * with the previous layer's tail).  enable = 0 makes every later forward pass of this stack use the phase
 * kernels instead; all levels produce the same bits. */
int salt_b200_stack_set_fused_decode(void *stack, int enable);
/* Replace the grouped-output buffer by caller-owned device memory (for example
 * a buffer registered with a communication library). */
int salt_b200_stack_set_grouped_out(void *stack, void *device_buffer, size_t nbytes);

/* The dense branch and the norms that make a MoE layer the reference model's whole feed-forward
 * block (models/gemma4-26b-a4b/src/gemma4_text.c:8293-8385; combine: src/gemma4.c:215-276):
 *   norm_a  = RMSNorm(residual) * pre_ffn_norm;   dense  = down(GeGLU(gate(norm_a), up(norm_a)))
 *   router input, logits, top-k from the residual
 *   norm_b  = RMSNorm(residual) * pre_ffn_norm_2; routed = ordered reduce of the experts on norm_b
 *   out     = (residual + RMSNorm(RMSNorm(dense)*post_ffn_norm_1 + RMSNorm(routed)*post_ffn_norm_2)
 *                         * post_ffn_norm) * layer_scalar
 * dense_gate / dense_up are affine-Q4 tensors [dense_inter][hidden], dense_down is
 * [hidden][dense_inter], each laid out values | scales | biases.  Attach once per layer after
 * salt_b200_stack_add_q4_layer; no reference counterpart as ONE call (the reference runs these
 * steps from the host, with exact cells and projection batches in between). */
typedef struct SaltB200FfnBlockSpec {
    int dense_inter;
    const void *dense_gate, *dense_up, *dense_down;
    const float *pre_ffn_norm, *pre_ffn_norm_2, *post_ffn_norm_1, *post_ffn_norm_2, *post_ffn_norm;
    float layer_scalar;
} SaltB200FfnBlockSpec;
int salt_b200_stack_attach_ffn_block(void *stack, int layer, const SaltB200FfnBlockSpec *spec);
/* d_residual, d_out: [B][hidden] device memory (distinct buffers); every launch goes to `stream`. */
int salt_b200_ffn_block_forward(void *stack, int layer, const float *d_residual, int B, float *d_out, void *stream);

/* Phase A of one layer on `stream` (a cudaStream_t, NULL = default stream):
 * router input, logits, top-k, grouping, gate/up + GeGLU, down for the local
 * experts.  d_x is [B][hidden] in device memory.  flags:
 *   SALT_B200_EXPERTS_ZERO_REMOTE         clear grouped_out first, so rows of remote experts read as +0
 *   SALT_B200_EXPERTS_ROUTER_INPUT_READY  the previous layer's combine already prepared the router input */
#define SALT_B200_EXPERTS_ZERO_REMOTE 1
#define SALT_B200_EXPERTS_ROUTER_INPUT_READY 2
/*   SALT_B200_EXPERTS_TENSOR_CORE         run the expert projections as fp16 GEMMs on the tensor cores
 *                                          (tcgen05/TMEM, fp32 accumulate) with every operand carried as
 *                                          hi + lo fp16 halves: a TOLERANCE path for prefill-sized batches,
 *                                          max |err| / max(|ref|, row rms) <= 1e-3; router and reduce stay exact
 *   SALT_B200_EXPERTS_TENSOR_CORE_SINGLE  same with operands rounded to fp16 once (a third of the tensor work):
 *                                          max |err| <= 1e-3 of the row maximum, about 2e-3 of the row rms
 *                                          Both need hidden and inter to be multiples of 64; a size that is no
 *                                          multiple of 256 must not exceed 960 (hi + lo) or 3520 (single).
 *                                          Otherwise the call returns -1. */
#define SALT_B200_EXPERTS_TENSOR_CORE 4
#define SALT_B200_EXPERTS_TENSOR_CORE_SINGLE 8
/*   SALT_B200_EXPERTS_TWO_LAUNCHES        run gate/up + GeGLU and down as two launches even where the
 *                                          one-launch decode kernel applies (same bits; for comparison) */
#define SALT_B200_EXPERTS_TWO_LAUNCHES 16
int salt_b200_layer_experts(void *stack, int layer, const float *d_x, int B, int flags, void *stream);
/* Phase B: ordered weighted reduce of grouped_out into d_y [B][hidden].  flags:
 *   SALT_B200_COMBINE_NORM          d_y = RMSNorm(reduce) when the layer has a norm weight
 *   SALT_B200_COMBINE_PREPARE_NEXT  also form the router input of layer + 1 from d_y (same launch) */
#define SALT_B200_COMBINE_NORM 1
#define SALT_B200_COMBINE_PREPARE_NEXT 2
int salt_b200_layer_combine(void *stack, int layer, int B, float *d_y, int flags, void *stream);
/* Expert parallelism by token dispatch (tokens partitioned by home rank; rows travel only to the rank that
 * owns their expert and results only back to the home rank - any all-to-all moves them, e.g. NCCL's).  A layer
 * is three calls, no state is kept between them except the router input prepared by _combine_rows:
 *   _layer_route           home rank: router input (unless SALT_B200_EXPERTS_ROUTER_INPUT_READY), in-order logits,
 *                          softmax top-k of its B tokens -> d_selected [B][topk] (expert ids, ascending within a
 *                          token), d_weights [B][topk]; both caller-owned device memory
 *   _layer_experts_routed  owner rank: d_out[i] = expert d_experts[i] (one of THIS stack's experts) applied to
 *                          d_rows[i] (gate | up, GeGLU, down), i < n_rows <= max_tokens * topk, any order; the
 *                          rows are grouped by expert as reference src/moe_group.c:83-182 groups them and every
 *                          row's result depends only on (expert weights, row), so it is the same whichever rank
 *                          computes it and whatever else is in the call.  flags: the TENSOR_CORE flags
 *   _layer_combine_rows    home rank: the returned rows d_rows [B * topk][hidden]; selection (token t, rank k) is
 *                          row d_row_index[t * topk + k], or row t * topk + k when d_row_index is NULL
 *                          -> ordered weighted reduce (src/moe_group.c:211-224), then as salt_b200_layer_combine */
int salt_b200_layer_route(void *stack, int layer, const float *d_x, int B, int32_t *d_selected, float *d_weights,
                          int flags, void *stream);
/* The send order of a home rank's n = B * topk selections (device arrays): rank r of `world` owns experts
 * [r * n_experts / world, (r + 1) * n_experts / world); selections are grouped by owner, canonical order inside
 * a group.  d_order[p] = canonical index of the p-th row sent, d_pos = its inverse (the row of selection i),
 * d_ids[p] = that row's expert, d_counts[r] = rows for rank r.  world <= 8. */
int salt_b200_dispatch_plan(const int32_t *d_selected, int n, int n_experts, int world, int32_t *d_order,
                            int32_t *d_pos, int32_t *d_ids, int32_t *d_counts, void *stream);
int salt_b200_layer_experts_routed(void *stack, int layer, const float *d_rows, const int32_t *d_experts, int n_rows,
                                   float *d_out, int flags, void *stream);
int salt_b200_layer_combine_rows(void *stack, int layer, const float *d_rows, const int32_t *d_row_index,
                                 const float *d_weights, int B, float *d_y, int flags, void *stream);
/* Expert-parallel exchange over peer memory (no reference counterpart: the reference is
 * single-device; the sharding rule follows from its expert independence,
 * models/gemma4-26b-a4b/src/gemma4.c:154-186 reduces per-selection outputs in rank order).
 * Each rank (one process per GPU, or several stacks of one process) owns experts
 * [expert_begin, expert_end) and runs the same tokens through a replicated router.
 *   _ep_region   allocates this stack's landing region and returns its CUDA IPC handle
 *                (64 bytes) and its device address
 *   _ep_connect  takes the handles of all `world` ranks in rank order (entry `rank` is ignored),
 *                or, with ipc_handles == NULL, `regions`: the device addresses themselves when
 *                the ranks live in one process.  world <= 8.
 *   _ep_exchange after salt_b200_layer_experts: pushes this rank's rows of grouped_out into every
 *                peer's region, waits (bounded, a few seconds; a timeout sets the device error
 *                word) for the peers' rows and copies them into grouped_out.  After it,
 *                salt_b200_layer_combine sees the complete buffer.  phase = PUSH | PULL; the two
 *                halves may be launched separately only when all ranks share one device and
 *                every rank's PUSH is enqueued before any PULL.
 * Once connected, salt_b200_stack_forward_device (and a graph captured from it) runs the
 * exchange between the two phases of every layer.  All ranks must run the same sequence of
 * exchanges; start the first one only after every rank has connected (host barrier). */
#define SALT_B200_EP_PUSH 1
#define SALT_B200_EP_PULL 2
int salt_b200_stack_ep_region(void *stack, void *ipc_handle_out, void **region_out);
int salt_b200_stack_ep_connect(void *stack, int rank, int world, const void *ipc_handles, void *const *regions);
int salt_b200_stack_ep_exchange(void *stack, int B, int phase, void *stream);
/* Bounded waits of the exchange: a slot that has not arrived after `polls` polls (about half a
 * microsecond each; default 2^23, a few seconds) makes the kernel give up, set the timeout bit of the
 * device error word (salt_b200_stack_status returns it) and return; the device stays usable.  After a
 * timeout the ranks' exchange counters may differ: call salt_b200_stack_ep_reset on EVERY rank while no
 * exchange is in flight anywhere (it clears the landing region, its counter and the error word), then
 * exchange again.  No reference counterpart (the reference is single-device). */
int salt_b200_stack_ep_set_poll_limit(void *stack, int polls);
int salt_b200_stack_ep_reset(void *stack);
/* Back to the unconnected state (peer mappings closed); call only between exchanges, after a host barrier. */
int salt_b200_stack_ep_disconnect(void *stack);

/* Layers [first, first+count) back to back (phase A + B each), chained through
 * the layers' RMSNorm; d_x and d_y are device pointers and may alias. */
int salt_b200_stack_forward_device(void *stack, int first, int count, const float *d_x, int B, float *d_y,
                                   void *stream);
/* Same with HOST input/output: copies in, runs, copies out, synchronises, and
 * returns -1 if the device error word is set. */
int salt_b200_stack_forward_host(void *stack, int first, int count, const float *h_x, int B, float *h_y);
/* Capture layers [first, first+count) into a CUDA graph on `stream` (not the
 * legacy default stream); pointers and B are baked in.  Replay with
 * salt_b200_stack_graph_launch. */
int salt_b200_stack_graph_capture(void *stack, int first, int count, const float *d_x, int B, float *d_y,
                                  void *stream);
int salt_b200_stack_graph_launch(void *stack, void *stream);
/* Per-kernel-class device timing: while enabled every launch of a forward pass
 * is bracketed by CUDA events (at most max_launches launches between reads).
 * _read returns summed milliseconds and launch counts for the 8 classes
 * router input, logits, top-k, plan, gate/up+GeGLU, down, reduce, RMSNorm. */
int salt_b200_stack_profile(void *stack, int enable, int max_launches);
int salt_b200_stack_profile_read(void *stack, float *ms_by_class, int *launches_by_class, int n_classes);
/* Synchronise `stream`, read and clear the device error word.  0 = clean. */
int salt_b200_stack_status(void *stack, void *stream);
/* Number of kernel launches issued by this library since load. */
uint64_t salt_b200_launch_count(void);

/* Debug tap: synchronise the device and copy nbytes of device memory to the host. */
int salt_b200_read_device(void *host_dst, const void *device_src, size_t nbytes);

/* Stand-alone device-pointer forms of the building blocks (tests, profiling). */
int salt_b200_q4_matvec_device(const void *d_vals, const void *d_scales, const void *d_biases, int R, int C,
                               const float *d_x, int B, float *d_y, void *stream);
int salt_b200_route_group_device(const int32_t *d_selected, int rows, int topk, int n_experts,
                                 int32_t *d_group_offsets, int32_t *d_grouped_to_canonical,
                                 int32_t *d_canonical_to_grouped, void *stream);

/* One expert's chain y = down(gelu_tanh(gate x) * up x) for ntok activation rows,
 * all pointers in DEVICE memory (16-byte aligned), asynchronous on `stream`.
 * No counterpart in the reference: this entry point exists for callers that
 * cannot allocate device memory -- an engine whose own allocator already owns
 * the whole device, a plugin that must keep a pre-sized budget, a loop that
 * cannot afford the synchronisation an allocation implies.  It calls no
 * allocation routine; its
 * intermediate rows live in a fixed 256 KiB array inside the library image
 * that every GPU loading the library holds until the process exits.
 *   - limit: ntok * inter <= 65536 floats (e.g. 93 rows at inter = 704); larger
 *     calls are rejected with -1 and a message on stderr.  hidden and inter
 *     must be positive multiples of 64.
 *   - the first call on a device looks the array's address up; make that call
 *     before any stream capture.
 *   - all calls on a device share the array, which keeps the previous call's
 *     contents (nothing in it needs clearing: each call writes what it reads);
 *     two calls whose kernels overlap on the GPU race on it -- issue them on
 *     one stream or order them yourself.
 * Results are bit-identical to salt_gpu_q4_moe_chain on the same data. */
int salt_b200_q4_expert_chain_static(const void *d_gate_vals, const void *d_gate_scales,
                                     const void *d_gate_biases, const void *d_up_vals,
                                     const void *d_up_scales, const void *d_up_biases,
                                     const void *d_down_vals, const void *d_down_scales,
                                     const void *d_down_biases, int hidden, int inter, const float *d_x,
                                     int ntok, float *d_y, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* SALT_GPU_B200_H */
