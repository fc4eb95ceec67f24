// Host side of libsalt_gpu_b200.so, part 2: a device-resident stack of MoE
// feed-forward layers (salt_b200_*).  Weights are uploaded once; a forward pass
// is a fixed sequence of kernel launches on the caller's stream with no host
// round trip: router input -> logits -> top-k -> grouping/plan -> fused
// gate/up + GeGLU -> down -> ordered weighted reduce [-> RMSNorm].
//
// Expert parallelism: a stack created with a sub-range of experts uploads only
// those experts.  Every device computes the (replicated, deterministic)
// routing for all tokens and writes the down-projection rows of ITS experts at
// their positions in the global grouped order; rows of other devices' experts
// arrive through whatever exchange the caller runs between the two phases.
#include <cuda_runtime.h>
#include <cmath>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "../../include/salt_gpu_b200.h"
#include "backend_state.h"
#include "internal.h"
#include "q4_core.cuh"

namespace sb {

struct Layer {
    float* router_w = nullptr;
    float* router_scale = nullptr;
    float* per_expert_scale = nullptr;
    float* norm_weight = nullptr;
    uint8_t* pool = nullptr;   // local experts only; slot of expert e at pool + (e - expert_begin) * stride
    uint8_t* sb_tables = nullptr;   // derived copy for the fused decode kernels: (scale << 16) | bias words, [local][3][groups]
    int* lit_flags = nullptr;       // [local] bit k: tensor k of the expert has a scale that needs the two-rounding form
    size_t expert_stride = 0;
    float eps = 0.0f;
    bool q4_tc_ok = false;          // tiled maps of the tensor-core path over pool and sb_tables
    TcWeightMaps q4_tc;
    // NVFP4 experts (W4A4: E2M1 codes + E4M3 block scales; reference src/nvfp4.c) instead of affine-Q4 ones
    bool nvfp4 = false;
    Fp4ExpertDesc* fp4_experts = nullptr;      // [local experts] device
    bool fp4_tc_ok = false;                    // every block scale is an unsigned finite E4M3 code: the tensor core can take it
    CUtensorMap fp4_w_gu, fp4_w_dn;            // weight maps of the tensor-core form (gate | up rows; down rows)
    CUtensorMap fp4_ws_gu, fp4_ws_dn;          // ... and of their block scales
    // optional dense branch and norms of the whole feed-forward block
    bool ffn = false;
    int dense_inter = 0;
    float layer_scalar = 1.0f;
    float *pre_ffn_norm = nullptr, *pre_ffn_norm_2 = nullptr;
    float *post_ffn_norm_1 = nullptr, *post_ffn_norm_2 = nullptr, *post_ffn_norm = nullptr;
    uint8_t* dense = nullptr;          // gate | up | down affine-Q4 tensors
    Q4Job* dense_jobs = nullptr;       // [2] device: fused gate/up job, down job
};

struct Stack {
    int max_tokens = 0, hidden = 0, inter = 0, n_experts = 0, topk = 0;
    int expert_begin = 0, expert_end = 0;
    std::vector<Layer> layers;
    // workspace
    float *rin = nullptr, *logits = nullptr, *weights = nullptr, *chain = nullptr, *grouped_out = nullptr;
    float *reduced = nullptr, *act_a = nullptr, *act_b = nullptr, *io_in = nullptr, *io_out = nullptr;
    int32_t *selected = nullptr, *group_offsets = nullptr, *g2c = nullptr, *c2g = nullptr, *counters = nullptr;
    int32_t* identity = nullptr;               // 0, 1, 2, ...: the rank table of rows that arrive in canonical order
    int32_t* status = nullptr;
    Q4Job *gateup_jobs = nullptr, *down_jobs = nullptr;
    FusedJob* fused_jobs = nullptr;            // descriptors and arrival counters of the fused decode kernel
    int32_t* fused_done = nullptr;
    // one-launch decode layers (one token): buffers of the other parity and per-layer arrival counters
    float *grouped_alt = nullptr, *weights_alt = nullptr;
    int32_t* layer_counters = nullptr;         // [layers_cap][FUSED_MAX_JOBS + 1], then [layers_cap] "layer finished" counters
    LayerDecodeArgs* d_layer_args = nullptr;   // [layers_cap] arguments of the whole-stack decode launch
    std::vector<LayerDecodeArgs> h_layer_args;
    int layers_cap = 0;
    bool any_nvfp4 = false;
    // workspace of NVFP4 layers (allocated with the first one): quantise-dequantised activations of the
    // gate / up inputs [2J][H] and of the down inputs [J][M], the codes and block scales the quantisation
    // also produces, gate / up outputs [J][M], per-row input global scales, projection jobs
    float *fp4_dq_gu = nullptr, *fp4_dq_dn = nullptr, *fp4_gate = nullptr, *fp4_up = nullptr;
    float *fp4_ig_gu = nullptr, *fp4_ig_dn = nullptr;
    uint8_t *fp4_packed = nullptr, *fp4_scales = nullptr;
    Fp4Job *fp4_gu_jobs = nullptr, *fp4_dn_jobs = nullptr;
    Fp4TcJob *fp4_tc_gu = nullptr, *fp4_tc_dn = nullptr;
    int* fp4_live = nullptr;                   // [2 + 3E]: counts and indices of the projection jobs that have tokens
    CUtensorMap fp4_x_gu[3], fp4_x_dn[3];      // packed activations as [2J][H/2] and as [J][M/2]
    CUtensorMap fp4_xs_gu[3], fp4_xs_dn[3];    // their block scales as [2J][H/16] and as [J][M/16]
    bool fp4_maps_ok = false;
    int fused_decode = 1;                      // 0: phase kernels; 1: one-launch expert kernel (B <= 4) and one launch per decode layer (B = 1); 2: all layers of a B = 1 pass in one launch (measured slower than 1)
    void *xh = nullptr, *xl = nullptr, *chain_h = nullptr, *chain_l = nullptr;   // fp16 operands (hi, lo) of the tensor-core path
    bool tc_ready = false;                     // tensor maps built and the geometry fits the single-precision tensor-core kernel
    bool tc_split_ready = false;               // ... and the hi + lo form
    TcMaps x_maps, chain_maps;                 // TMA descriptors of (xh, xl) and (chain_h, chain_l)
    void *tc_items_fused = nullptr, *tc_items_plain = nullptr;   // work lists of the tensor-core launches (device-written)
    int* tc_work = nullptr;                    // {items, next, largest pass, -} of the fused launch, then of the plain one
    // workspace of the whole feed-forward block (allocated by the first attach)
    float *norm_a = nullptr, *norm_b = nullptr, *dense_chain = nullptr, *dense_out = nullptr;
    float *routed_out = nullptr, *combine_scratch = nullptr;
    int dense_cap = 0;
    bool own_grouped = true;
    size_t grouped_bytes = 0;
    float *h_in = nullptr, *h_out = nullptr;  // pinned staging for the host entry point
    // optional per-kernel-class timing: event pairs recorded around every launch
    bool profile = false;
    std::vector<cudaEvent_t> ev;          // pairs (begin, end)
    std::vector<int> ev_class;
    size_t ev_used = 0;
    cudaGraphExec_t graph = nullptr;
    // expert-parallel exchange over peer memory
    uint8_t* ep_region = nullptr;              // this stack's landing region
    uint8_t* ep_peer[EP_MAX_WORLD] = {};       // all ranks' regions (own included) once connected
    bool ep_opened[EP_MAX_WORLD] = {};         // mapped through a CUDA IPC handle
    int ep_rank = 0, ep_world = 0;
    int ep_spin_limit = EP_DEFAULT_SPIN_LIMIT;
};

enum KernelClass { KC_ROUTER_INPUT = 0, KC_LOGITS, KC_TOPK, KC_PLAN, KC_GATE_UP, KC_DOWN, KC_REDUCE, KC_NORM, KC_COUNT };

struct Timed {
    Stack* s; cudaStream_t st; bool on;
    Timed(Stack* s_, int cls, cudaStream_t st_) : s(s_), st(st_), on(false) {
        if (!s->profile || s->ev_used + 2 > s->ev.size()) return;
        on = true;
        s->ev_class[s->ev_used / 2] = cls;
        cudaEventRecord(s->ev[s->ev_used], st);
    }
    ~Timed() {
        if (!on) return;
        cudaEventRecord(s->ev[s->ev_used + 1], st);
        s->ev_used += 2;
    }
};

static void free_stack(Stack* s) {
    for (auto& l : s->layers) {
        cudaFree(l.router_w); cudaFree(l.router_scale); cudaFree(l.per_expert_scale);
        cudaFree(l.norm_weight); cudaFree(l.pool); cudaFree(l.sb_tables); cudaFree(l.lit_flags); cudaFree(l.fp4_experts);
        cudaFree(l.pre_ffn_norm); cudaFree(l.pre_ffn_norm_2); cudaFree(l.post_ffn_norm_1);
        cudaFree(l.post_ffn_norm_2); cudaFree(l.post_ffn_norm); cudaFree(l.dense); cudaFree(l.dense_jobs);
    }
    cudaFree(s->norm_a); cudaFree(s->norm_b); cudaFree(s->dense_chain); cudaFree(s->dense_out);
    cudaFree(s->routed_out); cudaFree(s->combine_scratch);
    cudaFree(s->rin); cudaFree(s->logits); cudaFree(s->weights); cudaFree(s->chain);
    if (s->own_grouped) cudaFree(s->grouped_out);
    cudaFree(s->reduced); cudaFree(s->act_a); cudaFree(s->act_b); cudaFree(s->io_in); cudaFree(s->io_out);
    cudaFree(s->selected); cudaFree(s->identity); cudaFree(s->group_offsets); cudaFree(s->g2c); cudaFree(s->c2g);
    cudaFree(s->counters); cudaFree(s->status); cudaFree(s->gateup_jobs); cudaFree(s->down_jobs);
    cudaFree(s->fused_jobs); cudaFree(s->fused_done);
    cudaFree(s->grouped_alt); cudaFree(s->weights_alt); cudaFree(s->layer_counters); cudaFree(s->d_layer_args);
    cudaFree(s->fp4_dq_gu); cudaFree(s->fp4_dq_dn); cudaFree(s->fp4_gate); cudaFree(s->fp4_up); cudaFree(s->fp4_ig_gu);
    cudaFree(s->fp4_ig_dn); cudaFree(s->fp4_packed); cudaFree(s->fp4_scales); cudaFree(s->fp4_gu_jobs); cudaFree(s->fp4_dn_jobs);
    cudaFree(s->fp4_tc_gu); cudaFree(s->fp4_tc_dn); cudaFree(s->fp4_live);
    cudaFree(s->xh); cudaFree(s->xl); cudaFree(s->chain_h); cudaFree(s->chain_l);
    cudaFree(s->tc_items_fused); cudaFree(s->tc_items_plain); cudaFree(s->tc_work);
    if (s->h_in) cudaFreeHost(s->h_in);
    if (s->h_out) cudaFreeHost(s->h_out);
    for (auto e : s->ev) cudaEventDestroy(e);
    if (s->graph) cudaGraphExecDestroy(s->graph);
    for (int p = 0; p < EP_MAX_WORLD; p++)
        if (s->ep_opened[p]) cudaIpcCloseMemHandle(s->ep_peer[p]);
    cudaFree(s->ep_region);
    delete s;
}

template <typename T>
static bool dev_alloc(T** p, size_t count) {
    return cuda_ok(cudaMalloc((void**)p, count * sizeof(T) + 16), "stack alloc");
}

template <typename T>
static bool upload(T** dst, const T* src, size_t count) {
    return dev_alloc(dst, count) &&
           cuda_ok(cudaMemcpy(*dst, src, count * sizeof(T), cudaMemcpyHostToDevice), "stack upload");
}

}  // namespace sb

using namespace sb;

extern "C" {

int salt_b200_stack_create(int max_tokens, int hidden, int inter, int n_experts, int topk, int expert_begin,
                           int expert_end, void** stack_out) {
    if (!stack_out || max_tokens < 1 || hidden < 64 || inter < 64 || (hidden % 64) || (inter % 64) ||
        n_experts < 1 || n_experts > 1024 || topk < 1 || topk > n_experts || topk > 64 || expert_begin < 0 ||
        expert_end > n_experts || expert_begin >= expert_end)
        return -1;
    int ndev = 0;
    cudaDeviceProp prop;
    int dev = 0;
    if (!cuda_ok(cudaGetDeviceCount(&ndev), "device count") || ndev < 1 || !cuda_ok(cudaGetDevice(&dev), "device") ||
        !cuda_ok(cudaGetDeviceProperties(&prop, dev), "props") || prop.major != 10)
        return -1;  // sm_100a binary: nothing else can run it, and nothing else is tried
    Stack* s = new Stack();
    s->max_tokens = max_tokens; s->hidden = hidden; s->inter = inter; s->n_experts = n_experts; s->topk = topk;
    s->expert_begin = expert_begin; s->expert_end = expert_end;
    const size_t T = (size_t)max_tokens, J = T * (size_t)topk;
    s->grouped_bytes = J * (size_t)hidden * sizeof(float);
    bool ok = dev_alloc(&s->rin, T * hidden) && dev_alloc(&s->logits, T * n_experts) && dev_alloc(&s->weights, J) &&
              dev_alloc(&s->chain, J * inter) && dev_alloc(&s->grouped_out, J * hidden) &&
              dev_alloc(&s->reduced, T * hidden) && dev_alloc(&s->act_a, T * hidden) &&
              dev_alloc(&s->act_b, T * hidden) && dev_alloc(&s->io_in, T * hidden) &&
              dev_alloc(&s->io_out, T * hidden) && dev_alloc(&s->selected, J) &&
              dev_alloc(&s->group_offsets, (size_t)n_experts + 1) && dev_alloc(&s->g2c, J) &&
              dev_alloc(&s->c2g, J) && dev_alloc(&s->counters, 4) && dev_alloc(&s->status, 1) &&
              dev_alloc(&s->gateup_jobs, (size_t)n_experts) && dev_alloc(&s->down_jobs, (size_t)n_experts) &&
              dev_alloc(&s->fused_jobs, (size_t)FUSED_MAX_JOBS) && dev_alloc(&s->fused_done, (size_t)FUSED_MAX_JOBS) &&
              dev_alloc(&s->grouped_alt, (size_t)topk * hidden) && dev_alloc(&s->weights_alt, (size_t)topk) &&
              dev_alloc((uint16_t**)&s->xh, J * hidden) && dev_alloc((uint16_t**)&s->chain_h, J * inter) &&
              dev_alloc((uint16_t**)&s->xl, J * hidden) && dev_alloc((uint16_t**)&s->chain_l, J * inter) &&
              cuda_ok(cudaMemset(s->status, 0, sizeof(int32_t)), "status") &&
              cuda_ok(cudaHostAlloc((void**)&s->h_in, T * hidden * sizeof(float), cudaHostAllocDefault), "pinned") &&
              cuda_ok(cudaHostAlloc((void**)&s->h_out, T * hidden * sizeof(float), cudaHostAllocDefault), "pinned");
    if (!ok) {
        free_stack(s);
        return -1;
    }
    {
        const size_t items = q4_tc_work_items_max(n_experts, (int)J, hidden, inter);
        if (!dev_alloc((uint8_t**)&s->tc_items_fused, items * 16) || !dev_alloc((uint8_t**)&s->tc_items_plain, items * 16) ||
            !dev_alloc(&s->tc_work, 8)) {
            free_stack(s);
            return -1;
        }
    }
    s->tc_ready = q4_tc_supported(hidden, inter, false) && make_tc_maps(&s->x_maps, s->xh, s->xl, (int)J, hidden) == cudaSuccess &&
                  make_tc_maps(&s->chain_maps, s->chain_h, s->chain_l, (int)J, inter) == cudaSuccess;
    s->tc_split_ready = s->tc_ready && q4_tc_supported(hidden, inter, true);
    *stack_out = s;
    return 0;
}

int salt_b200_stack_destroy(void* stack) {
    if (!stack) return -1;
    cudaDeviceSynchronize();
    free_stack((Stack*)stack);
    return 0;
}

int salt_b200_stack_add_q4_layer(void* stack, const SaltB200Q4LayerSpec* spec) {
    Stack* s = (Stack*)stack;
    if (!s || !spec || spec->hidden != s->hidden || spec->inter != s->inter || spec->n_experts != s->n_experts ||
        spec->topk != s->topk || !spec->router_w || !spec->router_scale || !spec->per_expert_scale || !spec->pool)
        return -1;
    const size_t elems = (size_t)s->hidden * s->inter;
    const size_t tensor_bytes = elems / 2 + 2 * (elems / 64 * 2);
    if (spec->expert_stride < 3 * tensor_bytes || (spec->expert_stride % 16) != 0) return -1;
    Layer l;
    l.eps = spec->eps;
    l.expert_stride = spec->expert_stride;
    const size_t local = (size_t)(s->expert_end - s->expert_begin);
    const uint8_t* src = (const uint8_t*)spec->pool + (size_t)s->expert_begin * spec->expert_stride;
    bool ok = upload(&l.router_w, spec->router_w, (size_t)s->n_experts * s->hidden) &&
              upload(&l.router_scale, spec->router_scale, (size_t)s->hidden) &&
              upload(&l.per_expert_scale, spec->per_expert_scale, (size_t)s->n_experts) &&
              upload(&l.pool, src, local * spec->expert_stride) &&
              (!spec->norm_weight || upload(&l.norm_weight, spec->norm_weight, (size_t)s->hidden));
    const size_t groups = elems / 64;
    ok = ok && dev_alloc(&l.sb_tables, local * 3 * groups * 4) && dev_alloc(&l.lit_flags, local) &&
         cuda_ok(launch_q4_interleave_tables(l.pool, l.expert_stride, tensor_bytes, elems / 2, groups, (int)local,
                                             (uint32_t*)l.sb_tables, l.lit_flags, 0), "scale tables") &&
         cuda_ok(cudaDeviceSynchronize(), "scale tables");
    if (!ok) {
        cudaFree(l.router_w); cudaFree(l.router_scale); cudaFree(l.per_expert_scale); cudaFree(l.pool);
        cudaFree(l.norm_weight); cudaFree(l.sb_tables); cudaFree(l.lit_flags);
        return -1;
    }
    l.q4_tc_ok = s->tc_ready && make_q4_tc_weight_maps(&l.q4_tc, l.pool, l.expert_stride, (const uint32_t*)l.sb_tables,
                                                        s->hidden, s->inter, (int)local) == cudaSuccess;
    s->layers.push_back(l);
    return (int)s->layers.size() - 1;
}

int salt_b200_stack_add_nvfp4_layer(void* stack, const SaltB200Nvfp4LayerSpec* spec) {
    Stack* s = (Stack*)stack;
    if (!s || !spec || spec->hidden != s->hidden || spec->inter != s->inter || spec->n_experts != s->n_experts ||
        spec->topk != s->topk || !spec->router_w || !spec->router_scale || !spec->per_expert_scale || !spec->pool ||
        !spec->weight_divisors || !spec->input_globals || (s->hidden % 256) || (s->inter % 256))
        return -1;
    const size_t elems = (size_t)s->hidden * s->inter;
    const size_t code_bytes = elems / 2, scale_bytes = elems / 16, tensor_bytes = code_bytes + scale_bytes;
    if (spec->expert_stride < 3 * tensor_bytes || (spec->expert_stride % 16) != 0) return -1;
    const size_t T = (size_t)s->max_tokens, J = T * (size_t)s->topk;
    const int E = s->n_experts;
    if (!s->fp4_dq_gu &&
        !(dev_alloc(&s->fp4_dq_gu, 2 * J * s->hidden) && dev_alloc(&s->fp4_dq_dn, J * s->inter) &&
          dev_alloc(&s->fp4_gate, J * s->inter) && dev_alloc(&s->fp4_up, J * s->inter) && dev_alloc(&s->fp4_ig_gu, 2 * J) &&
          dev_alloc(&s->fp4_ig_dn, J) && dev_alloc(&s->fp4_packed, 2 * J * (size_t)s->hidden / 2) &&
          dev_alloc(&s->fp4_scales, 2 * J * (size_t)s->hidden / 16) && dev_alloc(&s->fp4_gu_jobs, (size_t)2 * E) &&
          dev_alloc(&s->fp4_dn_jobs, (size_t)E) && dev_alloc(&s->fp4_tc_gu, (size_t)2 * E) &&
          dev_alloc(&s->fp4_tc_dn, (size_t)E) && dev_alloc(&s->fp4_live, (size_t)(2 + 3 * E))))
        return -1;
    if (!s->fp4_maps_ok)
        s->fp4_maps_ok = make_fp4_act_maps(s->fp4_x_gu, s->fp4_packed, s->hidden, (int)(2 * J)) == cudaSuccess &&
                         make_fp4_act_maps(s->fp4_x_dn, s->fp4_packed, s->inter, (int)J) == cudaSuccess &&
                         make_fp4_act_scale_maps(s->fp4_xs_gu, s->fp4_scales, s->hidden, (int)(2 * J)) == cudaSuccess &&
                         make_fp4_act_scale_maps(s->fp4_xs_dn, s->fp4_scales, s->inter, (int)J) == cudaSuccess;
    Layer l;
    l.eps = spec->eps;
    l.expert_stride = spec->expert_stride;
    l.nvfp4 = true;
    const size_t local = (size_t)(s->expert_end - s->expert_begin);
    const uint8_t* src = (const uint8_t*)spec->pool + (size_t)s->expert_begin * spec->expert_stride;
    bool ok = upload(&l.router_w, spec->router_w, (size_t)E * s->hidden) &&
              upload(&l.router_scale, spec->router_scale, (size_t)s->hidden) &&
              upload(&l.per_expert_scale, spec->per_expert_scale, (size_t)E) &&
              upload(&l.pool, src, local * spec->expert_stride) &&
              (!spec->norm_weight || upload(&l.norm_weight, spec->norm_weight, (size_t)s->hidden));
    std::vector<Fp4ExpertDesc> desc(local);
    for (size_t i = 0; ok && i < local; i++) {
        const size_t e = (size_t)s->expert_begin + i;
        for (int k = 0; k < 3; k++) {
            const float div = spec->weight_divisors[e * 3 + k], ig = spec->input_globals[e * 3 + k];
            if (!std::isfinite(div) || div == 0.0f || !std::isfinite(ig) || !(ig > 0.0f)) ok = false;
            desc[i].codes[k] = l.pool + i * spec->expert_stride + (size_t)k * tensor_bytes;
            desc[i].scales[k] = desc[i].codes[k] + code_bytes;
            desc[i].wg[k] = 1.0f / div;              // fl(1 / stored divisor), as reference src/nvfp4.c:228-256 forms it
            desc[i].ig[k] = ig;
        }
    }
    ok = ok && upload(&l.fp4_experts, desc.data(), local);
    if (ok) {
        // the tensor-core form reads the block scales as UNSIGNED E4M3: a negative or NaN scale code (legal in
        // the stored format, never produced by a quantiser) keeps the layer on the exact kernels
        bool plain = s->fp4_maps_ok && (s->inter % 8) == 0;
        for (size_t i = 0; plain && i < local; i++)
            for (int k = 0; plain && k < 3; k++) {
                const uint8_t* sc = src + i * spec->expert_stride + (size_t)k * tensor_bytes + code_bytes;
                for (size_t b = 0; b < scale_bytes; b++)
                    if (sc[b] >= 0x7f) { plain = false; break; }
            }
        const int M = s->inter, H = s->hidden;
        l.fp4_tc_ok = plain &&
                      make_fp4_weight_map(&l.fp4_w_gu, l.pool, H, 2 * M + M / 8, (int)local, spec->expert_stride) == cudaSuccess &&
                      make_fp4_weight_map(&l.fp4_w_dn, l.pool + 2 * tensor_bytes, M, H, (int)local, spec->expert_stride) == cudaSuccess &&
                      make_fp4_weight_scale_map(&l.fp4_ws_gu, l.pool + code_bytes, H, 10 * M, (int)local,
                                                spec->expert_stride) == cudaSuccess &&
                      make_fp4_weight_scale_map(&l.fp4_ws_dn, l.pool + 2 * tensor_bytes + code_bytes, M, H, (int)local,
                                                spec->expert_stride) == cudaSuccess;
    }
    if (!ok) {
        cudaFree(l.router_w); cudaFree(l.router_scale); cudaFree(l.per_expert_scale); cudaFree(l.pool);
        cudaFree(l.norm_weight); cudaFree(l.fp4_experts);
        return -1;
    }
    s->any_nvfp4 = true;
    s->layers.push_back(l);
    return (int)s->layers.size() - 1;
}

int salt_b200_stack_set_fused_decode(void* stack, int enable) {
    Stack* s = (Stack*)stack;
    if (!s) return -1;
    s->fused_decode = enable < 0 ? 0 : (enable > 2 ? 2 : enable);
    return 0;
}

int salt_b200_stack_workspace(void* stack, SaltB200Workspace* out) {
    Stack* s = (Stack*)stack;
    if (!s || !out) return -1;
    out->grouped_out = s->grouped_out;
    out->group_offsets = s->group_offsets;
    out->selected = s->selected;
    out->weights = s->weights;
    out->canonical_to_grouped = s->c2g;
    out->grouped_to_canonical = s->g2c;
    out->logits = s->logits;
    out->status = s->status;
    out->grouped_out_bytes = s->grouped_bytes;
    return 0;
}

int salt_b200_stack_nvfp4_buffers(void* stack, SaltB200Nvfp4Buffers* out) {
    Stack* s = (Stack*)stack;
    if (!s || !out || !s->any_nvfp4) return -1;
    out->gate = s->fp4_gate;
    out->up = s->fp4_up;
    out->chain_codes = s->fp4_packed;
    out->chain_scales = s->fp4_scales;
    return 0;
}

int salt_b200_stack_set_grouped_out(void* stack, void* device_buffer, size_t nbytes) {
    Stack* s = (Stack*)stack;
    if (!s || !device_buffer || nbytes < s->grouped_bytes || ((uintptr_t)device_buffer & 15)) return -1;
    if (s->own_grouped) cudaFree(s->grouped_out);
    s->grouped_out = (float*)device_buffer;
    s->own_grouped = false;
    return 0;
}

// flags for salt_b200_layer_experts / salt_b200_layer_combine
enum { SB_EXPERTS_ZERO_REMOTE = 1, SB_EXPERTS_ROUTER_INPUT_READY = 2, SB_EXPERTS_TENSOR_CORE = 4,
       SB_EXPERTS_TENSOR_CORE_SINGLE = 8, SB_EXPERTS_TWO_LAUNCHES = 16 };
enum { SB_COMBINE_NORM = 1, SB_COMBINE_PREPARE_NEXT = 2 };

// Router of a layer for B tokens: router input (unless already prepared), in-order logits and, unless the plan
// kernel will do it (fused_topk), the softmax top-k into sel_out / w_out.
static int layer_router(Stack* s, const Layer& l, const float* d_router_src, int B, int flags, bool fused_topk,
                        int32_t* sel_out, float* w_out, cudaStream_t st) {
    const int H = s->hidden, E = s->n_experts, K = s->topk;
    if (!(flags & SB_EXPERTS_ROUTER_INPUT_READY)) {
        Timed t(s, KC_ROUTER_INPUT, st);
        GlueArgs g;
        memset(&g, 0, sizeof g);
        g.x_in = d_router_src; g.router_scale = l.router_scale; g.eps_router = l.eps; g.rin = s->rin; g.n = H;
        g.status = s->status;
        if (!cuda_ok(launch_glue(g, B, st), "router in")) return -1;
        count_launches(1);
    }
    {
        Timed t(s, KC_LOGITS, st);
        if (!cuda_ok(launch_router_logits(l.router_w, nullptr, s->rin, s->logits, B, E, H, st), "logits")) return -1;
    }
    if (!fused_topk) {
        Timed t(s, KC_TOPK, st);
        if (!cuda_ok(launch_router_topk(s->logits, l.per_expert_scale, sel_out, w_out, B, E, K, 1, s->status, st), "topk"))
            return -1;
        count_launches(1);
    }
    return 0;
}

static int experts_run(Stack* s, const Layer& l, const float* d_x, int B, int K, const int32_t* selected, bool fused_topk,
                       int flags, cudaStream_t st);

// d_router_src feeds the router input (unless it is already prepared), d_x the expert projections.
static int layer_experts_impl(Stack* s, int layer, const float* d_router_src, const float* d_x, int B, int flags,
                              cudaStream_t st) {
    if (!s || layer < 0 || layer >= (int)s->layers.size() || !d_x || !d_router_src || B < 1 || B > s->max_tokens)
        return -1;
    const Layer& l = s->layers[(size_t)layer];
    if ((flags & SB_EXPERTS_ZERO_REMOTE) &&
        !cuda_ok(cudaMemsetAsync(s->grouped_out, 0, (size_t)B * s->topk * s->hidden * sizeof(float), st), "zero grouped"))
        return -1;
    const bool fused_topk = B <= 8;
    if (layer_router(s, l, d_router_src, B, flags, fused_topk, s->selected, s->weights, st) != 0) return -1;
    return experts_run(s, l, d_x, B, s->topk, s->selected, fused_topk, flags, st);
}

// Grouping and expert projections for `B` rows with K selections each (`selected`: [B][K] expert ids; with
// fused_topk the plan kernel derives them from the logits first).  Results land in grouped_out in grouped order.
static int experts_run(Stack* s, const Layer& l, const float* d_x, int B, int K, const int32_t* selected, bool fused_topk,
                       int flags, cudaStream_t st) {
    const int H = s->hidden, M = s->inter, E = s->n_experts;
    const int jobs = B * K;
    const size_t elems = (size_t)H * M;
    MoePlanArgs a;
    memset(&a, 0, sizeof a);
    if (fused_topk) {
        a.logits = s->logits; a.per_expert_scale = l.per_expert_scale;
        a.selected_out = s->selected; a.weights_out = s->weights;
    }
    a.selected = selected; a.rows = B; a.topk = K; a.n_experts = E;
    a.expert_begin = s->expert_begin; a.expert_end = s->expert_end;
    a.group_offsets = s->group_offsets; a.grouped_to_canonical = s->g2c; a.canonical_to_grouped = s->c2g;
    a.n_active = s->counters; a.max_group = s->counters + 1;
    // the plan indexes experts globally; local slot 0 is expert_begin
    a.pool = l.pool - (size_t)s->expert_begin * l.expert_stride;
    a.expert_stride = l.expert_stride;
    a.value_bytes = elems / 2; a.group_bytes = elems / 64 * 2;
    a.tensor_bytes = a.value_bytes + 2 * a.group_bytes;
    a.hidden = H; a.inter = M; a.x = d_x; a.chain = s->chain; a.grouped_out = s->grouped_out;
    a.gateup_jobs = s->gateup_jobs; a.down_jobs = s->down_jobs; a.status = s->status;
    const int local = s->expert_end - s->expert_begin;
    const int njobs_max = jobs < local ? jobs : local;
    // decode batches: gate/up, GeGLU and down of all selected experts in one launch
    const bool fused = !l.nvfp4 && s->fused_decode && !(flags & (SB_EXPERTS_TENSOR_CORE | SB_EXPERTS_TENSOR_CORE_SINGLE |
                                                     SB_EXPERTS_TWO_LAUNCHES)) &&
                       B <= FUSED_MAX_TOKENS && njobs_max <= FUSED_MAX_JOBS &&
                       ((((uintptr_t)d_x) | ((uintptr_t)l.pool) | l.expert_stride) & 15) == 0 &&
                       q4_fused_plan(H, M, B, njobs_max, nullptr);
    if (fused) {
        a.fused_jobs = s->fused_jobs; a.fused_done = s->fused_done;
        a.fused_tables = l.sb_tables - (size_t)s->expert_begin * 6 * a.group_bytes;
        a.fused_lit = l.lit_flags - s->expert_begin;
    }
    {
        Timed t(s, KC_PLAN, st);
        if (!cuda_ok(launch_moe_plan(a, st), "plan")) return -1;
    }
    if (l.nvfp4 && (flags & SB_EXPERTS_TENSOR_CORE)) {
        // block-scaled tensor-core form (tolerance path): same plan, same bit-exact quantiser, the two
        // projection batches as tcgen05.mma.kind::mxf4nvf4 GEMMs
        if (!l.fp4_tc_ok) return -1;
        Timed t(s, KC_GATE_UP, st);
        Fp4TcMaps mg, md;
        mg.w = l.fp4_w_gu; md.w = l.fp4_w_dn;
        mg.ws = l.fp4_ws_gu; md.ws = l.fp4_ws_dn;
        for (int v = 0; v < 3; v++) {
            mg.x[v] = s->fp4_x_gu[v]; md.x[v] = s->fp4_x_dn[v];
            mg.xs[v] = s->fp4_xs_gu[v]; md.xs[v] = s->fp4_xs_dn[v];
        }
        if (!cuda_ok(launch_nvfp4_moe_plan(s->group_offsets, E, s->expert_begin, s->expert_end, jobs, l.fp4_experts, H, M,
                                           s->fp4_dq_gu, s->fp4_gate, s->fp4_up, s->fp4_dq_dn, s->grouped_out,
                                           s->fp4_gu_jobs, s->fp4_dn_jobs, s->fp4_ig_gu, s->fp4_ig_dn, st, s->fp4_tc_gu,
                                           s->fp4_tc_dn), "nvfp4 plan") ||
            !cuda_ok(launch_nvfp4_qdq(d_x, 2 * jobs, H, s->fp4_ig_gu, s->fp4_packed, s->fp4_scales, nullptr,
                                      s->status, st, s->g2c, jobs, K), "nvfp4 qdq x") ||
            !cuda_ok(launch_nvfp4_gemm_tc(s->fp4_tc_gu, 2 * E, M, H, mg, s->status, st), "nvfp4 tc gate/up") ||
            !cuda_ok(launch_nvfp4_qdq(s->fp4_gate, jobs, M, s->fp4_ig_dn, s->fp4_packed, s->fp4_scales, nullptr,
                                      s->status, st, nullptr, 1, 1, s->fp4_up), "nvfp4 geglu + qdq") ||
            !cuda_ok(launch_nvfp4_gemm_tc(s->fp4_tc_dn, E, H, M, md, s->status, st), "nvfp4 tc down"))
            return -1;
        count_launches(6);
        return 0;
    }
    if (l.nvfp4) {
        if (flags & SB_EXPERTS_TENSOR_CORE_SINGLE) return -1;
        Timed t(s, KC_GATE_UP, st);
        const int live_max = std::min(s->expert_end - s->expert_begin, jobs);   // experts that can have tokens
        const int typical = std::max(1, (jobs + E - 1) / E);                    // selections per expert, evenly routed
        if (!cuda_ok(launch_nvfp4_moe_plan(s->group_offsets, E, s->expert_begin, s->expert_end, jobs, l.fp4_experts, H, M,
                                           s->fp4_dq_gu, s->fp4_gate, s->fp4_up, s->fp4_dq_dn, s->grouped_out,
                                           s->fp4_gu_jobs, s->fp4_dn_jobs, s->fp4_ig_gu, s->fp4_ig_dn, st, nullptr, nullptr,
                                           s->fp4_live), "nvfp4 plan") ||
            !cuda_ok(launch_nvfp4_qdq(d_x, 2 * jobs, H, s->fp4_ig_gu, s->fp4_packed, s->fp4_scales, s->fp4_dq_gu,
                                      s->status, st, s->g2c, jobs, K), "nvfp4 qdq x") ||
            !cuda_ok(launch_nvfp4_jobs(s->fp4_gu_jobs, 2 * live_max, M, B, H, true, st, s->fp4_live + 2, s->fp4_live,
                                       typical), "nvfp4 gate/up") ||
            !cuda_ok(launch_nvfp4_qdq(s->fp4_gate, jobs, M, s->fp4_ig_dn, s->fp4_packed, s->fp4_scales, s->fp4_dq_dn,
                                      s->status, st, nullptr, 1, 1, s->fp4_up), "nvfp4 geglu + qdq") ||
            !cuda_ok(launch_nvfp4_jobs(s->fp4_dn_jobs, live_max, H, B, M, true, st, s->fp4_live + 2 + 2 * E,
                                       s->fp4_live + 1, typical), "nvfp4 down"))
            return -1;
        count_launches(6);
        return 0;
    }
    if (fused) {
        FusedArgs f;
        memset(&f, 0, sizeof f);
        f.jobs = s->fused_jobs; f.n_jobs_dev = s->counters; f.n_jobs_max = njobs_max; f.done = s->fused_done;
        f.x = d_x; f.x_stride = H; f.n_x = B; f.chain = s->chain; f.out = s->grouped_out; f.H = H; f.M = M;
        f.status = s->status;
        Timed t(s, KC_GATE_UP, st);
        if (!cuda_ok(launch_q4_fused(f, st), "fused experts")) return -1;
        count_launches(3);
        return 0;
    }
    // tokens per expert group: at most B (the tile kernels loop over a group's tokens and use the bound
    // only to pick their token block; the any-shape kernel takes one grid row per token)
    const int tok_hint = B;
    if (flags & (SB_EXPERTS_TENSOR_CORE | SB_EXPERTS_TENSOR_CORE_SINGLE)) {
        const bool split = (flags & SB_EXPERTS_TENSOR_CORE) != 0;
        if (!s->tc_ready || !l.q4_tc_ok || (split && !s->tc_split_ready)) {
            fprintf(stderr, "salt_b200: tensor-core path unavailable for this geometry\n");
            return -1;
        }
        // tolerance path: fp16 operands on tcgen05, fp32 accumulation in TMEM
        {
            Timed t(s, KC_ROUTER_INPUT, st);
            if (!cuda_ok(launch_gather_convert(d_x, s->g2c, s->xh, split ? s->xl : nullptr, jobs, K, H, st), "gather/convert")) return -1;
            if (!cuda_ok(launch_q4_tc_work_list(s->gateup_jobs, s->counters, njobs_max, s->chain, M, l.q4_tc, H, M,
                                                s->tc_items_fused, s->tc_items_plain, s->tc_work, st), "tc work list"))
                return -1;
        }
        {
            Timed t(s, KC_GATE_UP, st);
            if (!cuda_ok(launch_q4_gemm_tc(true, split, s->tc_items_fused, s->tc_work, s->x_maps, l.q4_tc, s->chain_h,
                                           s->chain_l, nullptr, M, H, s->status, st), "tc gate/up"))
                return -1;
        }
        {
            Timed t(s, KC_DOWN, st);
            if (!cuda_ok(launch_q4_gemm_tc(false, split, s->tc_items_plain, s->tc_work + 4, s->chain_maps, l.q4_tc, nullptr,
                                           nullptr, s->grouped_out, H, M, s->status, st), "tc down"))
                return -1;
        }
        count_launches(6);
        return 0;
    }
    {
        Timed t(s, KC_GATE_UP, st);
        if (!cuda_ok(launch_q4_jobs(s->gateup_jobs, njobs_max, s->counters, M, tok_hint, H, 2, true, st, 0), "gate/up"))
            return -1;
    }
    {
        Timed t(s, KC_DOWN, st);
        if (!cuda_ok(launch_q4_jobs(s->down_jobs, njobs_max, s->counters, H, tok_hint, M, 1, true, st, 1), "down"))
            return -1;
    }
    count_launches(4);
    return 0;
}

int salt_b200_layer_experts(void* stack, int layer, const float* d_x, int B, int flags, void* stream_) {
    return layer_experts_impl((Stack*)stack, layer, d_x, d_x, B, flags, (cudaStream_t)stream_);
}

// ---- expert parallelism by token dispatch: the three steps of a layer as separate calls -----------------
// Send order of a home rank's n selections: grouped by the rank that owns each selection's expert, canonical
// order inside a group (a stable counting sort over at most EP_MAX_WORLD destinations, one block).
__global__ void __launch_bounds__(1024)
dispatch_plan_kernel(const int32_t* __restrict__ sel, int n, int E, int world, int32_t* __restrict__ order,
                     int32_t* __restrict__ pos, int32_t* __restrict__ ids, int32_t* __restrict__ counts) {
    __shared__ int warp_tot[EP_MAX_WORLD][32];
    __shared__ int s_start[EP_MAX_WORLD + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = (n + 1023) / 1024;
    const int i0 = min(n, tid * chunk), i1 = min(n, i0 + chunk);
    auto owner = [&](int e) {
        int d = 0;
        for (int r = 1; r < world; r++) d += e >= (int)((long long)r * E / world) ? 1 : 0;
        return d;                                     // ids outside [0, E) travel to rank 0 or the last rank, which flags them
    };
    int cnt[EP_MAX_WORLD], base[EP_MAX_WORLD];
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; d++) cnt[d] = 0;
    for (int i = i0; i < i1; i++) {
        const int o = owner(sel[i]);
#pragma unroll
        for (int d = 0; d < EP_MAX_WORLD; d++) cnt[d] += o == d ? 1 : 0;
    }
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; d++) {
        int inc = cnt[d];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        base[d] = inc - cnt[d];                       // exclusive inside the warp
        if (lane == 31) warp_tot[d][warp] = inc;
    }
    __syncthreads();
    if (warp == 0) {
        int run = 0;
        for (int d = 0; d < EP_MAX_WORLD; d++) {
            int inc = warp_tot[d][lane];
            const int own = inc;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            warp_tot[d][lane] = inc - own;            // exclusive prefix of the warp totals
            const int total = __shfl_sync(0xffffffffu, inc, 31);
            if (lane == 0) {
                s_start[d] = run;
                if (d < world) counts[d] = total;
            }
            run += total;
        }
    }
    __syncthreads();
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; d++) base[d] += s_start[d] + warp_tot[d][warp];
    for (int i = i0; i < i1; i++) {
        const int e = sel[i], o = owner(e);
        int p = 0;
#pragma unroll
        for (int d = 0; d < EP_MAX_WORLD; d++)
            if (o == d) p = base[d]++;
        pos[i] = p;
        order[p] = i;
        ids[p] = e;
    }
}

int salt_b200_dispatch_plan(const int32_t* d_selected, int n, int n_experts, int world, int32_t* d_order, int32_t* d_pos,
                            int32_t* d_ids, int32_t* d_counts, void* stream_) {
    if (n < 0 || n_experts < 1 || world < 1 || world > EP_MAX_WORLD || world > n_experts || !d_counts) return -1;
    if (n > 0 && (!d_selected || !d_order || !d_pos || !d_ids)) return -1;
    dispatch_plan_kernel<<<1, 1024, 0, (cudaStream_t)stream_>>>(d_selected, n, n_experts, world, d_order, d_pos, d_ids, d_counts);
    return cuda_ok(cudaGetLastError(), "dispatch plan") ? 0 : -1;
}

// home rank: router of its own tokens -> caller-owned selected / weights
int salt_b200_layer_route(void* stack, int layer, const float* d_x, int B, int32_t* d_selected, float* d_weights, int flags,
                          void* stream_) {
    Stack* s = (Stack*)stack;
    if (!s || layer < 0 || layer >= (int)s->layers.size() || !d_x || !d_selected || !d_weights || B < 1 || B > s->max_tokens)
        return -1;
    return layer_router(s, s->layers[(size_t)layer], d_x, B, flags & SB_EXPERTS_ROUTER_INPUT_READY, false, d_selected,
                        d_weights, (cudaStream_t)stream_);
}

// out[row] = grouped[c2g[row]]; a row whose expert is not one of this rank's gets zeros and sets the error word
// (its slot in the grouped buffer was never computed, or, for an id outside the table, never assigned)
__global__ void __launch_bounds__(256)
ungroup_rows_kernel(const float4* __restrict__ grouped, const int* __restrict__ c2g, const int32_t* __restrict__ experts,
                    int expert_begin, int expert_end, int n_rows, float4* __restrict__ out, int n4, int* status) {
    const int row = blockIdx.x;
    const int e = experts[row];
    const bool mine = e >= expert_begin && e < expert_end;
    const int g = mine ? c2g[row] : -1;
    if ((g < 0 || g >= n_rows) && blockIdx.y == 0 && threadIdx.x == 0 && status) atomicOr(status, SB_ERR_INDEX);
    const float4* src = grouped + (size_t)(g >= 0 && g < n_rows ? g : 0) * n4;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n4; i += gridDim.y * blockDim.x)
        out[(size_t)row * n4 + i] = (g >= 0 && g < n_rows) ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

// owner rank: rows that other ranks (and this one) routed to ITS experts -> d_out[i] = expert d_experts[i] applied
// to d_rows[i], in the order given.  Every id must be one of this stack's experts (others set the status word).
int salt_b200_layer_experts_routed(void* stack, int layer, const float* d_rows, const int32_t* d_experts, int n_rows,
                                   float* d_out, int flags, void* stream_) {
    Stack* s = (Stack*)stack;
    cudaStream_t st = (cudaStream_t)stream_;
    if (!s || layer < 0 || layer >= (int)s->layers.size() || n_rows < 0 || n_rows > s->max_tokens * s->topk ||
        (s->hidden % 4) != 0)
        return -1;
    if (n_rows == 0) return 0;
    if (!d_rows || !d_experts || !d_out || ((uintptr_t)d_out & 15)) return -1;
    const Layer& l = s->layers[(size_t)layer];
    flags &= (SB_EXPERTS_TENSOR_CORE | SB_EXPERTS_TENSOR_CORE_SINGLE);
    if (experts_run(s, l, d_rows, n_rows, 1, d_experts, false, flags | SB_EXPERTS_TWO_LAUNCHES, st) != 0) return -1;
    const int n4 = s->hidden / 4;
    ungroup_rows_kernel<<<dim3(n_rows, (n4 + 255) / 256), 256, 0, st>>>((const float4*)s->grouped_out, s->c2g, d_experts,
                                                                      s->expert_begin, s->expert_end, n_rows,
                                                                      (float4*)d_out, n4, s->status);
    count_launches(1);
    return cuda_ok(cudaGetLastError(), "ungroup") ? 0 : -1;
}

// home rank: the returned rows in canonical order (token-major, rank order) -> ordered weighted reduce, norm,
// next router input, exactly as salt_b200_layer_combine does from the grouped buffer
int salt_b200_layer_combine_rows(void* stack, int layer, const float* d_rows, const int32_t* d_row_index,
                                 const float* d_weights, int B, float* d_y, int flags, void* stream_) {
    Stack* s = (Stack*)stack;
    cudaStream_t st = (cudaStream_t)stream_;
    if (!s || layer < 0 || layer >= (int)s->layers.size() || !d_rows || !d_weights || !d_y || B < 1 || B > s->max_tokens)
        return -1;
    const int J = s->max_tokens * s->topk;
    if (!d_row_index && !s->identity) {
        std::vector<int32_t> id((size_t)J);
        for (int i = 0; i < J; i++) id[(size_t)i] = i;
        if (!upload(&s->identity, id.data(), (size_t)J)) return -1;
    }
    const Layer& l = s->layers[(size_t)layer];
    const bool next = (flags & SB_COMBINE_PREPARE_NEXT) && layer + 1 < (int)s->layers.size();
    GlueArgs g;
    memset(&g, 0, sizeof g);
    g.weights = d_weights; g.c2g = d_row_index ? d_row_index : s->identity; g.grouped = d_rows; g.topk = s->topk;
    g.jobs = B * s->topk; g.y_out = d_y; g.n = s->hidden; g.status = s->status;
    g.tables_late = 1;                  // weights and row table may come from the kernel right before this one
    if ((flags & SB_COMBINE_NORM) && l.norm_weight) { g.norm_w = l.norm_weight; g.eps_norm = l.eps; }
    if (next) {
        const Layer& nl = s->layers[(size_t)layer + 1];
        g.router_scale = nl.router_scale; g.eps_router = nl.eps; g.rin = s->rin;
    }
    {
        Timed t(s, KC_REDUCE, st);
        if (!cuda_ok(launch_glue(g, B, st), "combine rows")) return -1;
    }
    count_launches(1);
    return 0;
}

// Ordered weighted reduce of grouped_out into d_y; SB_COMBINE_NORM applies the
// layer's RMSNorm (if it has one) to the result; SB_COMBINE_PREPARE_NEXT also
// forms the router input of layer + 1 from it, so that layer's
// salt_b200_layer_experts can be called with SB_EXPERTS_ROUTER_INPUT_READY.
int salt_b200_layer_combine(void* stack, int layer, int B, float* d_y, int flags, void* stream_) {
    Stack* s = (Stack*)stack;
    cudaStream_t st = (cudaStream_t)stream_;
    if (!s || layer < 0 || layer >= (int)s->layers.size() || !d_y || B < 1 || B > s->max_tokens) return -1;
    const Layer& l = s->layers[(size_t)layer];
    const bool next = (flags & SB_COMBINE_PREPARE_NEXT) && layer + 1 < (int)s->layers.size();
    GlueArgs g;
    memset(&g, 0, sizeof g);
    g.weights = s->weights; g.c2g = s->c2g; g.grouped = s->grouped_out; g.topk = s->topk; g.jobs = B * s->topk;
    g.y_out = d_y; g.n = s->hidden; g.status = s->status;
    if ((flags & SB_COMBINE_NORM) && l.norm_weight) { g.norm_w = l.norm_weight; g.eps_norm = l.eps; }
    if (next) {
        const Layer& nl = s->layers[(size_t)layer + 1];
        g.router_scale = nl.router_scale; g.eps_router = nl.eps; g.rin = s->rin;
    }
    {
        Timed t(s, KC_REDUCE, st);
        if (!cuda_ok(launch_glue(g, B, st), "combine")) return -1;
    }
    count_launches(1);
    return 0;
}

// ---- expert-parallel exchange over peer memory ------------------------------------------------
int salt_b200_stack_ep_region(void* stack, void* ipc_handle_out, void** region_out) {
    Stack* s = (Stack*)stack;
    if (!s || !ipc_handle_out) return -1;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    if (!s->ep_region) {
        const size_t bytes = ep_region_bytes(s->max_tokens * s->topk, s->hidden);
        if (!cuda_ok(cudaMalloc((void**)&s->ep_region, bytes), "ep region") ||
            !cuda_ok(cudaMemset(s->ep_region, 0, bytes), "ep region clear") ||
            !cuda_ok(cudaDeviceSynchronize(), "ep region sync"))
            return -1;
    }
    cudaIpcMemHandle_t h;
    if (!cuda_ok(cudaIpcGetMemHandle(&h, s->ep_region), "ipc handle")) return -1;
    memcpy(ipc_handle_out, &h, sizeof h);
    if (region_out) *region_out = s->ep_region;
    return 0;
}

int salt_b200_stack_ep_connect(void* stack, int rank, int world, const void* ipc_handles, void* const* regions) {
    Stack* s = (Stack*)stack;
    if (!s || !s->ep_region || s->ep_world || world < 2 || world > EP_MAX_WORLD || rank < 0 || rank >= world ||
        (!ipc_handles && !regions))
        return -1;
    for (int p = 0; p < world; p++) {
        if (p == rank) {
            s->ep_peer[p] = s->ep_region;
            continue;
        }
        if (ipc_handles) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const uint8_t*)ipc_handles + (size_t)p * sizeof h, sizeof h);
            void* ptr = nullptr;
            if (!cuda_ok(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "ipc open")) {
                for (int q = 0; q < p; q++)
                    if (s->ep_opened[q]) { cudaIpcCloseMemHandle(s->ep_peer[q]); s->ep_opened[q] = false; }
                return -1;
            }
            s->ep_peer[p] = (uint8_t*)ptr;
            s->ep_opened[p] = true;
        } else {
            if (!regions[p]) return -1;
            s->ep_peer[p] = (uint8_t*)regions[p];
        }
    }
    s->ep_rank = rank;
    s->ep_world = world;
    return 0;
}

int salt_b200_stack_ep_disconnect(void* stack) {
    Stack* s = (Stack*)stack;
    if (!s) return -1;
    cudaDeviceSynchronize();
    for (int p = 0; p < EP_MAX_WORLD; p++) {
        if (s->ep_opened[p]) cudaIpcCloseMemHandle(s->ep_peer[p]);
        s->ep_opened[p] = false;
        s->ep_peer[p] = nullptr;
    }
    s->ep_world = 0;
    return 0;
}

int salt_b200_stack_ep_set_poll_limit(void* stack, int polls) {
    Stack* s = (Stack*)stack;
    if (!s || polls < 1) return -1;
    s->ep_spin_limit = polls;
    return 0;
}

// Clears this stack's landing region (epoch and both buffers) and its error word.  To be called on
// every rank, with no exchange in flight anywhere, before the ranks exchange again.
int salt_b200_stack_ep_reset(void* stack) {
    Stack* s = (Stack*)stack;
    if (!s || !s->ep_region) return -1;
    const size_t bytes = ep_region_bytes(s->max_tokens * s->topk, s->hidden);
    return cuda_ok(cudaDeviceSynchronize(), "ep reset sync") && cuda_ok(cudaMemset(s->ep_region, 0, bytes), "ep reset") &&
                   cuda_ok(cudaMemset(s->status, 0, sizeof(int32_t)), "ep reset status") &&
                   cuda_ok(cudaDeviceSynchronize(), "ep reset sync") ? 0 : -1;
}

int salt_b200_stack_ep_exchange(void* stack, int B, int phase, void* stream) {
    Stack* s = (Stack*)stack;
    if (!s || s->ep_world < 2 || B < 1 || B > s->max_tokens) return -1;
    EpExchangeArgs a;
    memset(&a, 0, sizeof a);
    for (int p = 0; p < s->ep_world; p++) a.region[p] = s->ep_peer[p];
    a.rank = s->ep_rank; a.world = s->ep_world;
    a.group_offsets = s->group_offsets;
    a.expert_begin = s->expert_begin; a.expert_end = s->expert_end; a.n_experts = s->n_experts;
    a.grouped = s->grouped_out; a.width = s->hidden; a.rows_cap = s->max_tokens * s->topk;
    a.phase = phase; a.status = s->status; a.spin_limit = s->ep_spin_limit;
    Timed t(s, KC_NORM, (cudaStream_t)stream);
    if (!cuda_ok(launch_ep_exchange(a, B * s->topk, (cudaStream_t)stream), "ep exchange")) return -1;
    count_launches(1);
    return 0;
}

// ---- the whole feed-forward block ------------------------------------------------------------
__global__ void patch_job_tokens_kernel(Q4Job* jobs, int n, int ntok) {
    if ((int)threadIdx.x < n) jobs[threadIdx.x].ntok = ntok;
}

static size_t q4_blob_bytes(int R, int C) {
    const size_t elems = (size_t)R * C;
    return elems / 2 + 2 * (elems / 64 * 2);
}

int salt_b200_stack_attach_ffn_block(void* stack, int layer, const SaltB200FfnBlockSpec* spec) {
    Stack* s = (Stack*)stack;
    if (!s || !spec || layer < 0 || layer >= (int)s->layers.size() || spec->dense_inter < 64 ||
        (spec->dense_inter % 64) != 0 || (s->hidden % 64) != 0 || !spec->dense_gate || !spec->dense_up ||
        !spec->dense_down || !spec->pre_ffn_norm || !spec->pre_ffn_norm_2 || !spec->post_ffn_norm_1 ||
        !spec->post_ffn_norm_2 || !spec->post_ffn_norm || !std::isfinite(spec->layer_scalar))
        return -1;
    Layer& l = s->layers[(size_t)layer];
    if (l.ffn || l.nvfp4) return -1;
    const int H = s->hidden, D = spec->dense_inter;
    const size_t T = (size_t)s->max_tokens;
    if (D > s->dense_cap) {
        cudaFree(s->dense_chain);
        s->dense_chain = nullptr;
        if (!dev_alloc(&s->dense_chain, T * D)) return -1;
        s->dense_cap = D;
    }
    if (!s->norm_a &&
        !(dev_alloc(&s->norm_a, T * H) && dev_alloc(&s->norm_b, T * H) && dev_alloc(&s->dense_out, T * H) &&
          dev_alloc(&s->routed_out, T * H) && dev_alloc(&s->combine_scratch, 2 * T * H)))
        return -1;
    const size_t gu = q4_blob_bytes(D, H), dn = q4_blob_bytes(H, D);      // equal, kept apart for clarity
    bool ok = dev_alloc(&l.dense, 2 * gu + dn) &&
              cuda_ok(cudaMemcpy(l.dense, spec->dense_gate, gu, cudaMemcpyHostToDevice), "dense gate") &&
              cuda_ok(cudaMemcpy(l.dense + gu, spec->dense_up, gu, cudaMemcpyHostToDevice), "dense up") &&
              cuda_ok(cudaMemcpy(l.dense + 2 * gu, spec->dense_down, dn, cudaMemcpyHostToDevice), "dense down") &&
              upload(&l.pre_ffn_norm, spec->pre_ffn_norm, (size_t)H) &&
              upload(&l.pre_ffn_norm_2, spec->pre_ffn_norm_2, (size_t)H) &&
              upload(&l.post_ffn_norm_1, spec->post_ffn_norm_1, (size_t)H) &&
              upload(&l.post_ffn_norm_2, spec->post_ffn_norm_2, (size_t)H) &&
              upload(&l.post_ffn_norm, spec->post_ffn_norm, (size_t)H);
    if (!ok) return -1;
    const size_t vb = (size_t)D * H / 2, gb = (size_t)D * H / 64 * 2;
    Q4Job jobs[2];
    memset(jobs, 0, sizeof jobs);
    Q4Job& a = jobs[0];
    a.vals = l.dense; a.scales = l.dense + vb; a.biases = l.dense + vb + gb;
    a.vals2 = l.dense + gu; a.scales2 = a.vals2 + vb; a.biases2 = a.scales2 + gb;
    a.x = s->norm_a; a.y = s->dense_chain; a.x_rows = nullptr; a.x_div = 1;
    a.R = D; a.C = H; a.ntok = 1; a.x_stride = H; a.y_stride = D;
    Q4Job& b = jobs[1];
    b.vals = l.dense + 2 * gu; b.scales = b.vals + vb; b.biases = b.scales + gb;
    b.x = s->dense_chain; b.y = s->dense_out; b.x_rows = nullptr; b.x_div = 1;
    b.R = H; b.C = D; b.ntok = 1; b.x_stride = D; b.y_stride = H;
    if (!upload(&l.dense_jobs, jobs, (size_t)2)) return -1;
    l.dense_inter = D;
    l.layer_scalar = spec->layer_scalar;
    l.ffn = true;
    return 0;
}

int salt_b200_ffn_block_forward(void* stack, int layer, const float* d_residual, int B, float* d_out,
                                void* stream_) {
    Stack* s = (Stack*)stack;
    cudaStream_t st = (cudaStream_t)stream_;
    if (!s || layer < 0 || layer >= (int)s->layers.size() || !d_residual || !d_out || B < 1 || B > s->max_tokens)
        return -1;
    const Layer& l = s->layers[(size_t)layer];
    if (!l.ffn) return -1;
    const int H = s->hidden, D = l.dense_inter;
    const int tok_hint = B;            // see layer_experts_impl
    auto norm = [&](const float* w, float* y) {
        GlueArgs g;
        memset(&g, 0, sizeof g);
        g.x_in = d_residual; g.norm_w = w; g.eps_norm = l.eps; g.y_out = y; g.n = H; g.status = s->status;
        return cuda_ok(launch_glue(g, B, st), "ffn pre-norm");
    };
    // dense branch: norm_a -> gate/up + GeGLU -> down
    patch_job_tokens_kernel<<<1, 32, 0, st>>>(l.dense_jobs, 2, B);
    if (!norm(l.pre_ffn_norm, s->norm_a) ||
        !cuda_ok(launch_q4_jobs(l.dense_jobs, 1, nullptr, D, tok_hint, H, 2, true, st), "dense gate/up") ||
        !cuda_ok(launch_q4_jobs(l.dense_jobs + 1, 1, nullptr, H, tok_hint, D, 1, true, st), "dense down"))
        return -1;
    // routed branch: router on the residual, experts on norm_b
    if (!norm(l.pre_ffn_norm_2, s->norm_b)) return -1;
    count_launches(5);
    if (layer_experts_impl(s, layer, d_residual, s->norm_b, B, 0, st) != 0) return -1;
    if (s->ep_world > 1 && salt_b200_stack_ep_exchange(stack, B, EP_PHASE_PUSH | EP_PHASE_PULL, stream_) != 0) return -1;
    {
        GlueArgs g;
        memset(&g, 0, sizeof g);
        g.weights = s->weights; g.c2g = s->c2g; g.grouped = s->grouped_out; g.topk = s->topk; g.jobs = B * s->topk;
        g.y_out = s->routed_out; g.n = H; g.status = s->status;
        if (!cuda_ok(launch_glue(g, B, st), "routed reduce")) return -1;
    }
    if (!cuda_ok(launch_parallel_combine(d_residual, s->dense_out, s->routed_out, l.post_ffn_norm_1,
                                         l.post_ffn_norm_2, l.post_ffn_norm, s->combine_scratch,
                                         s->combine_scratch + (size_t)s->max_tokens * H, d_out, B, H, l.eps,
                                         l.layer_scalar, s->status, st), "parallel combine"))
        return -1;
    count_launches(2);
    return 0;
}

// Keeps the stream busy for a fixed number of clock cycles (bounded loop, nothing is waited
// for).  Used only while profiling: with the device occupied for about a millisecond the
// host enqueues a whole pass of launches and event records ahead of it, so the event pairs
// measure kernels that run back to back instead of kernels that wait for the host.
__global__ void profile_head_start_kernel(long long cycles) {
    const long long t0 = clock64();
    for (int i = 0; i < (1 << 24) && clock64() - t0 < cycles; i++) { }
}

// One token, one device: every layer is ONE launch (reduce + norm of the previous layer, router,
// top-k, experts), then one launch for the last reduce.
static bool decode_layers_apply(Stack* s, int B) {
    const int local = s->expert_end - s->expert_begin;
    return s->fused_decode && !s->any_nvfp4 && B == 1 && s->ep_world == 0 && s->topk <= FUSED_MAX_JOBS &&
           q4_layer_decode_plan(s->hidden, s->inter, s->n_experts, s->topk, s->topk < local ? s->topk : local, nullptr);
}

static int forward_decode_layers(Stack* s, int first, int count, const float* d_x, float* d_y, cudaStream_t st) {
    const int H = s->hidden, M = s->inter, K = s->topk;
    // per layer: the logits arrival counter and FUSED_MAX_JOBS job counters; after all layers' blocks of those,
    // one "layer finished" counter per layer (the whole-stack launch)
    const int stride = FUSED_MAX_JOBS + 1;
    if (count > s->layers_cap) {       // set-up, not part of a captured pass: forward passes are not captured before one has run
        cudaFree(s->layer_counters);
        cudaFree(s->d_layer_args);
        s->layer_counters = nullptr;
        s->d_layer_args = nullptr;
        if (!dev_alloc(&s->layer_counters, (size_t)count * (stride + 1)) || !dev_alloc(&s->d_layer_args, (size_t)count))
            return -1;
        s->h_layer_args.reserve((size_t)count);
        s->layers_cap = count;
    }
    if (!cuda_ok(cudaMemsetAsync(s->layer_counters, 0, (size_t)count * (stride + 1) * sizeof(int32_t), st), "layer counters"))
        return -1;
    const size_t elems = (size_t)H * M;
    const int local = s->expert_end - s->expert_begin;
    const int n_jobs_max = K < local ? K : local;
    const bool stacked = s->fused_decode >= 2;
    float* gbuf[2] = {s->grouped_out, s->grouped_alt};
    float* wbuf[2] = {s->weights, s->weights_alt};
    if (stacked) s->h_layer_args.resize((size_t)count);
    for (int i = 0; i < count; i++) {
        const Layer& l = s->layers[(size_t)first + i];
        LayerDecodeArgs a;
        memset(&a, 0, sizeof a);
        a.f.H = H; a.f.M = M; a.f.chain = s->chain; a.f.out = gbuf[i & 1];
        a.f.done = s->layer_counters + (size_t)i * stride + 1; a.f.status = s->status;
        a.f.n_jobs_max = n_jobs_max;
        a.logits_count = s->layer_counters + (size_t)i * stride;
        if (i == 0) {
            a.x_in = d_x;
        } else {
            const Layer& pl = s->layers[(size_t)first + i - 1];
            a.prev_grouped = gbuf[(i - 1) & 1]; a.prev_weights = wbuf[(i - 1) & 1];
            a.norm_w = pl.norm_weight; a.eps_norm = pl.eps;
        }
        a.router_scale = l.router_scale; a.eps_router = l.eps; a.router_w = l.router_w;
        a.per_expert_scale = l.per_expert_scale; a.logits = s->logits;
        a.E = s->n_experts; a.topk = K; a.expert_begin = s->expert_begin; a.expert_end = s->expert_end;
        a.selected = s->selected; a.weights_out = wbuf[i & 1]; a.c2g = s->c2g; a.g2c = s->g2c;
        a.group_offsets = s->group_offsets;
        a.pool = l.pool; a.tables = l.sb_tables; a.lit_flags = l.lit_flags; a.expert_stride = l.expert_stride;
        a.value_bytes = elems / 2; a.group_bytes = elems / 64 * 2; a.tensor_bytes = a.value_bytes + 2 * a.group_bytes;
        if (stacked) {
            a.f.jobs_per_round = q4_layer_decode_jobs_per_round(H, M, s->n_experts, K, n_jobs_max);
            a.f.n_x = 1;
            s->h_layer_args[(size_t)i] = a;
            continue;
        }
        Timed t(s, KC_GATE_UP, st);
        if (!cuda_ok(launch_q4_layer_decode(a, a.f.n_jobs_max, st), "decode layer")) return -1;
    }
    if (stacked) {
        // the arguments travel with every pass (a captured pass replays the copy from this host vector, whose
        // storage stays put while the capacity holds: set-up, like the counters above)
        if (!cuda_ok(cudaMemcpyAsync(s->d_layer_args, s->h_layer_args.data(), (size_t)count * sizeof(LayerDecodeArgs),
                                     cudaMemcpyHostToDevice, st), "layer arguments"))
            return -1;
        Timed t(s, KC_GATE_UP, st);
        if (!cuda_ok(launch_q4_stack_decode(s->d_layer_args, count, s->layer_counters + (size_t)count * stride, H, M,
                                            s->n_experts, K, n_jobs_max, st), "decode stack"))
            return -1;
    }
    const int last = count - 1;
    GlueArgs g;
    memset(&g, 0, sizeof g);
    g.weights = wbuf[last & 1]; g.c2g = s->c2g; g.grouped = gbuf[last & 1]; g.topk = K; g.jobs = K;
    g.y_out = d_y; g.n = H; g.status = s->status; g.tables_late = 1;
    {
        Timed t(s, KC_REDUCE, st);
        if (!cuda_ok(launch_glue(g, 1, st), "last reduce")) return -1;
    }
    count_launches(count + 1);
    return 0;
}

int salt_b200_stack_forward_device(void* stack, int first, int count, const float* d_x, int B, float* d_y,
                                   void* stream) {
    Stack* s = (Stack*)stack;
    if (!s || first < 0 || count < 1 || first + count > (int)s->layers.size() || !d_x || !d_y) return -1;
    if (s->profile) profile_head_start_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(80000LL * count + 400000LL);
    if (decode_layers_apply(s, B)) return forward_decode_layers(s, first, count, d_x, d_y, (cudaStream_t)stream);
    const float* in = d_x;
    for (int i = 0; i < count; i++) {
        const bool last = i == count - 1;
        float* out = last ? d_y : ((i & 1) ? s->act_b : s->act_a);
        if (salt_b200_layer_experts(stack, first + i, in, B, i > 0 ? SB_EXPERTS_ROUTER_INPUT_READY : 0,
                                    stream) != 0 ||
            (s->ep_world > 1 && salt_b200_stack_ep_exchange(stack, B, EP_PHASE_PUSH | EP_PHASE_PULL, stream) != 0) ||
            salt_b200_layer_combine(stack, first + i, B, out,
                                    last ? 0 : (SB_COMBINE_NORM | SB_COMBINE_PREPARE_NEXT), stream) != 0)
            return -1;
        in = out;
    }
    return 0;
}

// Per-kernel-class device timing.  While enabled, every launch of a forward pass
// is bracketed by a pair of CUDA events on the launching stream.
int salt_b200_stack_profile(void* stack, int enable, int max_launches) {
    Stack* s = (Stack*)stack;
    if (!s || max_launches < 0) return -1;
    s->profile = enable != 0;
    s->ev_used = 0;
    while (s->ev.size() < (size_t)2 * max_launches) {
        cudaEvent_t e;
        if (!cuda_ok(cudaEventCreate(&e), "event")) return -1;
        s->ev.push_back(e);
    }
    s->ev_class.assign(s->ev.size() / 2 + 1, 0);
    return 0;
}

// Sum of elapsed milliseconds and launch count per kernel class since the last
// call (classes: 0 router input, 1 logits, 2 top-k, 3 plan, 4 gate/up+GeGLU,
// 5 down, 6 weighted reduce, 7 RMSNorm).  Synchronises the device.
int salt_b200_stack_profile_read(void* stack, float* ms_by_class, int* launches_by_class, int n_classes) {
    Stack* s = (Stack*)stack;
    if (!s || !ms_by_class || !launches_by_class || n_classes < KC_COUNT) return -1;
    if (!cuda_ok(cudaDeviceSynchronize(), "profile sync")) return -1;
    for (int i = 0; i < n_classes; i++) { ms_by_class[i] = 0.0f; launches_by_class[i] = 0; }
    for (size_t i = 0; i + 1 < s->ev_used; i += 2) {
        float ms = 0.0f;
        if (!cuda_ok(cudaEventElapsedTime(&ms, s->ev[i], s->ev[i + 1]), "elapsed")) return -1;
        ms_by_class[s->ev_class[i / 2]] += ms;
        launches_by_class[s->ev_class[i / 2]]++;
    }
    s->ev_used = 0;
    return 0;
}

// Capture layers [first, first+count) as one CUDA graph on `stream` (which must
// not be the legacy default stream), for replay with salt_b200_stack_graph_launch.
// The pointers and B are baked into the graph.
int salt_b200_stack_graph_capture(void* stack, int first, int count, const float* d_x, int B, float* d_y,
                                  void* stream) {
    Stack* s = (Stack*)stack;
    cudaStream_t st = (cudaStream_t)stream;
    if (!s || !st || s->profile) return -1;
    // one uncaptured pass first: it performs the one-time function attribute setup
    if (salt_b200_stack_forward_device(stack, first, count, d_x, B, d_y, stream) != 0 ||
        !cuda_ok(cudaStreamSynchronize(st), "pre-capture sync"))
        return -1;
    if (s->graph) { cudaGraphExecDestroy(s->graph); s->graph = nullptr; }
    cudaGraph_t graph = nullptr;
    if (!cuda_ok(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "begin capture")) return -1;
    const int rc = salt_b200_stack_forward_device(stack, first, count, d_x, B, d_y, stream);
    const bool ended = cuda_ok(cudaStreamEndCapture(st, &graph), "end capture");
    if (rc != 0 || !ended || !graph) {
        if (graph) cudaGraphDestroy(graph);
        return -1;
    }
    const bool ok = cuda_ok(cudaGraphInstantiate(&s->graph, graph, 0), "instantiate");
    cudaGraphDestroy(graph);
    return ok ? 0 : -1;
}

int salt_b200_stack_graph_launch(void* stack, void* stream) {
    Stack* s = (Stack*)stack;
    if (!s || !s->graph) return -1;
    return cuda_ok(cudaGraphLaunch(s->graph, (cudaStream_t)stream), "graph launch") ? 0 : -1;
}

int salt_b200_stack_status(void* stack, void* stream) {
    Stack* s = (Stack*)stack;
    if (!s) return -1;
    int32_t status = 0;
    if (!cuda_ok(cudaStreamSynchronize((cudaStream_t)stream), "status sync") ||
        !cuda_ok(cudaMemcpy(&status, s->status, sizeof status, cudaMemcpyDeviceToHost), "status read"))
        return -1;
    if (status) cudaMemset(s->status, 0, sizeof status);
    return status;
}

int salt_b200_stack_forward_host(void* stack, int first, int count, const float* h_x, int B, float* h_y) {
    Stack* s = (Stack*)stack;
    if (!s || !h_x || !h_y || B < 1 || B > s->max_tokens) return -1;
    const size_t bytes = (size_t)B * s->hidden * sizeof(float);
    memcpy(s->h_in, h_x, bytes);
    if (!cuda_ok(cudaMemcpyAsync(s->io_in, s->h_in, bytes, cudaMemcpyHostToDevice, 0), "x upload")) return -1;
    if (salt_b200_stack_forward_device(stack, first, count, s->io_in, B, s->io_out, 0) != 0) return -1;
    if (!cuda_ok(cudaMemcpyAsync(s->h_out, s->io_out, bytes, cudaMemcpyDeviceToHost, 0), "y download")) return -1;
    if (salt_b200_stack_status(stack, 0) != 0) return -1;
    memcpy(h_y, s->h_out, bytes);
    return 0;
}

int salt_b200_read_device(void* host_dst, const void* device_src, size_t nbytes) {
    if (!host_dst || !device_src) return -1;
    return cuda_ok(cudaDeviceSynchronize(), "read sync") &&
                   cuda_ok(cudaMemcpy(host_dst, device_src, nbytes, cudaMemcpyDeviceToHost), "read") ? 0 : -1;
}

int salt_b200_q4_matvec_device(const void* d_vals, const void* d_scales, const void* d_biases, int R, int C,
                               const float* d_x, int B, float* d_y, void* stream) {
    if (!d_vals || !d_scales || !d_x || !d_y || R < 1 || C < 1 || B < 1) return -1;
    Q4Job j;
    memset(&j, 0, sizeof j);
    j.vals = (const uint8_t*)d_vals; j.scales = (const uint8_t*)d_scales; j.biases = (const uint8_t*)d_biases;
    j.x = d_x; j.y = d_y; j.x_div = 1; j.R = R; j.C = C; j.ntok = B; j.x_stride = C; j.y_stride = R;
    // a ring of descriptor slots per device: calls in flight on different streams do not share one
    constexpr int RING = 64, MAXDEV = 64;
    static Q4Job* rings[MAXDEV] = {};
    static unsigned cursor[MAXDEV] = {};
    static std::mutex mu;
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev), "device") || dev < 0 || dev >= MAXDEV) return -1;
    Q4Job* d_job;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!rings[dev] && !cuda_ok(cudaMalloc((void**)&rings[dev], RING * sizeof(Q4Job)), "job ring")) return -1;
        d_job = rings[dev] + (cursor[dev]++ % RING);
    }
    const bool aligned = (C % 64) == 0 &&
                         ((((uintptr_t)d_vals | (uintptr_t)d_scales | (uintptr_t)d_biases | (uintptr_t)d_x) & 15) == 0);
    if (!cuda_ok(cudaMemcpyAsync(d_job, &j, sizeof j, cudaMemcpyHostToDevice, (cudaStream_t)stream), "job upload") ||
        !cuda_ok(launch_q4_jobs(d_job, 1, nullptr, R, B, C, 1, aligned, (cudaStream_t)stream), "launch"))
        return -1;
    count_launches(1);
    return 0;
}

int salt_b200_route_group_device(const int32_t* d_selected, int rows, int topk, int n_experts,
                                 int32_t* d_group_offsets, int32_t* d_grouped_to_canonical,
                                 int32_t* d_canonical_to_grouped, void* stream) {
    if (!d_selected || !d_group_offsets || !d_grouped_to_canonical || !d_canonical_to_grouped || rows < 1 ||
        topk < 1 || n_experts < 1 || n_experts > 1024 || topk > n_experts)
        return -1;
    // scratch per device (n_active, max_group, status, unused descriptors); the call synchronises the
    // stream before it returns, and callers serialise (one calling thread at a time)
    constexpr int MAXDEV = 64;
    static int32_t* scratch_dev[MAXDEV] = {};
    static Q4Job* jobs_dev[MAXDEV] = {};
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev), "device") || dev < 0 || dev >= MAXDEV) return -1;
    if (!scratch_dev[dev] && (!cuda_ok(cudaMalloc((void**)&scratch_dev[dev], 4 * sizeof(int32_t)), "scratch") ||
                              !cuda_ok(cudaMalloc((void**)&jobs_dev[dev], 2 * 1024 * sizeof(Q4Job)), "scratch")))
        return -1;
    int32_t* scratch = scratch_dev[dev];
    Q4Job* jobs = jobs_dev[dev];
    MoePlanArgs a;
    memset(&a, 0, sizeof a);
    a.selected = d_selected; a.rows = rows; a.topk = topk; a.n_experts = n_experts;
    a.expert_begin = 0; a.expert_end = 0;  // no descriptors wanted
    a.group_offsets = d_group_offsets; a.grouped_to_canonical = d_grouped_to_canonical;
    a.canonical_to_grouped = d_canonical_to_grouped;
    a.n_active = scratch; a.max_group = scratch + 1; a.status = scratch + 2;
    a.gateup_jobs = jobs; a.down_jobs = jobs + 1024;
    if (!cuda_ok(cudaMemsetAsync(scratch, 0, 4 * sizeof(int32_t), (cudaStream_t)stream), "scratch") ||
        !cuda_ok(launch_moe_plan(a, (cudaStream_t)stream), "plan"))
        return -1;
    count_launches(1);
    int32_t status = 0;
    if (!cuda_ok(cudaStreamSynchronize((cudaStream_t)stream), "sync") ||
        !cuda_ok(cudaMemcpy(&status, scratch + 2, sizeof status, cudaMemcpyDeviceToHost), "status"))
        return -1;
    return status ? -1 : 0;
}

}  // extern "C"
