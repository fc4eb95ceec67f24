// Host side of libsalt_gpu_b200.so, part 1: the reference operator surface
// (salt_gpu_*) for the quantized MoE feed-forward path.
//
// Weight resources are byte ranges of caller memory that are copied into HBM
// when activated; tensors are (key -> resource, byte offsets, shape) records,
// as in the reference backends (reference src/gpu_cuda.cu:2714-2745,
// 3142-3217).  Compute calls with host pointers are synchronous: inputs are
// staged through pinned memory, the kernels of q4_kernels.cu run on one
// internal stream, and results are copied back before returning.  There is no
// CPU execution path in this file: a call that cannot run on the device
// returns -1.
#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <utility>
#include <cmath>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <unordered_map>
#include <vector>

#include "../../include/salt_gpu_b200.h"
#include "backend_state.h"
#include "internal.h"
#include "q4_core.cuh"

namespace sb {

void fp4_release();
Backend g_backend;
static uint64_t g_launches = 0;
void count_launches(int n) { g_launches += (uint64_t)n; }

cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, size_t> done;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    size_t& have = done[std::make_pair(dev, kernel)];
    if (have >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) have = bytes;
    return e;
}
uint64_t launch_count() { return g_launches; }

bool cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    if (getenv("SALT_GPU_DIAG")) fprintf(stderr, "salt-b200: %s: %s\n", what, cudaGetErrorString(e));
    return false;
}

static Resource* find_resource(uint32_t kind, uint32_t id) {
    for (auto& r : g_backend.resources)
        if (r.kind == kind && r.id == id) return &r;
    return nullptr;
}

static Resource* live_resource(uint32_t kind, uint32_t id) {
    Resource* r = find_resource(kind, id);
    return (r && r->active && r->dev) ? r : nullptr;
}

static bool in_range(const Resource& r, const void* p, size_t nbytes, uint64_t* off) {
    uintptr_t base = (uintptr_t)r.host, v = (uintptr_t)p;
    if (!p || v < base || v - base > r.nbytes || nbytes > r.nbytes - (v - base)) return false;
    *off = (uint64_t)(v - base);
    return true;
}

static bool q4_sizes(int bits, int R, int C, size_t* vbytes, size_t* gbytes) {
    if ((bits != 4 && bits != 8) || R < 1 || C < 1) return false;
    uint64_t elems = (uint64_t)(uint32_t)R * (uint64_t)(uint32_t)C;
    *vbytes = bits == 4 ? (size_t)(((elems + 7) / 8) * 4) : (size_t)(((elems + 3) / 4) * 4);
    *gbytes = (size_t)(((elems + 63) / 64) * 2);
    return true;
}

static void release_tensor(Tensor& t) {
    for (void* p : t.owned) cudaFree(p);
    t.owned.clear();
}

// Device views of a registered tensor.  Views that are not 16-byte aligned get
// a private aligned copy once, so every kernel sees aligned operands.
static bool materialize(Tensor& t, const Resource& r) {
    if (t.dv) return true;
    const uint64_t offs[3] = {t.voff, t.soff, t.boff};
    const size_t sizes[3] = {t.vbytes, t.gbytes, t.gbytes};
    const uint8_t* out[3];
    for (int i = 0; i < 3; i++) {
        const uint8_t* p = r.dev + offs[i];
        if (((uintptr_t)p & 15) != 0) {
            void* copy = nullptr;
            if (!cuda_ok(cudaMalloc(&copy, sizes[i] + 16), "cudaMalloc realign") ||
                !cuda_ok(cudaMemcpy(copy, p, sizes[i], cudaMemcpyDeviceToDevice), "realign copy"))
                return false;
            t.owned.push_back(copy);
            p = (const uint8_t*)copy;
        }
        out[i] = p;
    }
    t.dv = out[0]; t.ds = out[1]; t.db = out[2];
    return true;
}

// Resolve a projection's weights to device pointers.  Order: registered key;
// first sight of a tensor lying inside an active resource (registers it); in
// non-mapped-only mode, a private device copy keyed by id ("arena").
static Tensor* resolve_q4(const void* key, const void* vals, const void* scales, const void* biases, int R, int C,
                          int* kind_out, int bits = 4) {
    Backend& B = g_backend;
    size_t vb, gb;
    if (!key || !vals || !scales || !q4_sizes(bits, R, C, &vb, &gb)) return nullptr;
    auto it = B.tensors.find(key);
    if (it != B.tensors.end()) {
        Tensor& t = it->second;
        Resource* r = live_resource(t.kind, t.id);
        if (!r || t.bits != bits || t.R != R || t.C != C || r->host + t.voff != (const uint8_t*)vals ||
            r->host + t.soff != (const uint8_t*)scales || (biases && r->host + t.boff != (const uint8_t*)biases))
            return nullptr;
        if (!materialize(t, *r)) return nullptr;
        *kind_out = (int)t.kind;
        return &t;
    }
    for (auto& r : B.resources) {
        uint64_t vo, so, bo;
        if (!r.active || !r.dev || !in_range(r, vals, vb, &vo) || !in_range(r, scales, gb, &so) ||
            !biases || !in_range(r, biases, gb, &bo))
            continue;
        Tensor t;
        t.kind = r.kind; t.id = r.id; t.bits = bits; t.R = R; t.C = C;
        t.voff = vo; t.soff = so; t.boff = bo; t.vbytes = vb; t.gbytes = gb;
        Tensor& slot = B.tensors[key] = t;
        if (!materialize(slot, r)) { B.tensors.erase(key); return nullptr; }
        *kind_out = (int)r.kind;
        return &slot;
    }
    if (B.mapped_only || !biases) return nullptr;
    auto at = B.arena.find(key);
    if (at == B.arena.end() || at->second.R != R || at->second.C != C || at->second.bits != bits) {
        Tensor t;
        t.kind = SALT_GPU_RESOURCE_ARENA; t.bits = bits; t.R = R; t.C = C; t.vbytes = vb; t.gbytes = gb;
        void* dv = nullptr; void* ds = nullptr; void* db = nullptr;
        if (!cuda_ok(cudaMalloc(&dv, vb + 16), "arena") || !cuda_ok(cudaMalloc(&ds, gb + 16), "arena") ||
            !cuda_ok(cudaMalloc(&db, gb + 16), "arena") ||
            !cuda_ok(cudaMemcpy(dv, vals, vb, cudaMemcpyHostToDevice), "arena copy") ||
            !cuda_ok(cudaMemcpy(ds, scales, gb, cudaMemcpyHostToDevice), "arena copy") ||
            !cuda_ok(cudaMemcpy(db, biases, gb, cudaMemcpyHostToDevice), "arena copy")) {
            cudaFree(dv); cudaFree(ds); cudaFree(db);
            return nullptr;
        }
        t.owned = {dv, ds, db};
        t.dv = (const uint8_t*)dv; t.ds = (const uint8_t*)ds; t.db = (const uint8_t*)db;
        if (at != B.arena.end()) release_tensor(at->second);
        B.arena[key] = t;
        B.copied_bytes += vb + 2 * gb;
        at = B.arena.find(key);
    }
    *kind_out = SALT_GPU_RESOURCE_ARENA;
    return &at->second;
}

static void count_kinds(bool trunk, bool expert, bool arena) {
    Backend& B = g_backend;
    if (trunk) B.stats.trunk_batches++;
    if (expert) B.stats.expert_layer_batches++;
    if (arena) B.stats.arena_batches++;
}

bool stage_reserve(size_t x_floats, size_t y_floats, size_t mid_floats, size_t jobs) {
    Backend& B = g_backend;
    return x_floats <= B.stage_floats && y_floats <= B.stage_floats && mid_floats <= B.stage_floats &&
           jobs <= B.job_cap;
}

// Run descriptor jobs (already in B.h_jobs[0..n)) and wait.
static bool run_jobs(int njobs, int max_rows, int max_tok, int C, int nmat, bool aligned, int bits = 4) {
    Backend& B = g_backend;
    if (!cuda_ok(cudaMemcpyAsync(B.d_jobs, B.h_jobs, (size_t)njobs * sizeof(Q4Job), cudaMemcpyHostToDevice,
                                 B.stream), "job upload"))
        return false;
    if (bits == 8) {
        if (!cuda_ok(launch_q8_jobs(B.d_jobs, njobs, max_rows, max_tok, C, B.stream), "q8 launch")) return false;
    } else if (!cuda_ok(launch_q4_jobs(B.d_jobs, njobs, nullptr, max_rows, max_tok, C, nmat, aligned, B.stream),
                        "q4 launch"))
        return false;
    count_launches(1);
    return true;
}

static bool fill_job(Q4Job& j, const Tensor& t, const float* x, float* y, int ntok, int x_stride, int y_stride) {
    memset(&j, 0, sizeof j);
    j.vals = t.dv; j.scales = t.ds; j.biases = t.db;
    j.x = x; j.y = y; j.x_rows = nullptr; j.x_div = 1;
    j.R = t.R; j.C = t.C; j.ntok = ntok; j.x_stride = x_stride; j.y_stride = y_stride;
    return true;
}

}  // namespace sb

using namespace sb;

extern "C" {

// ------------------------------------------------------------------------
// lifecycle
// ------------------------------------------------------------------------
int salt_gpu_startup_requirements(SaltGpuStartupRequirements* r, size_t n) {
    if (!r || n != sizeof *r) return -1;
    memset(r, 0, sizeof *r);
    const uint64_t stage = (uint64_t)SB_STAGE_FLOATS * sizeof(float);
    r->fixed_device_bytes = 3 * stage + (uint64_t)SB_MAX_JOBS * sizeof(Q4Job) + sizeof(int);
    r->fixed_pinned_host_bytes = 2 * stage + (uint64_t)SB_MAX_JOBS * sizeof(Q4Job);
    r->descriptor_bytes = 2ull * SB_MAX_JOBS * sizeof(Q4Job);
    r->max_output_floats = (uint32_t)SB_STAGE_FLOATS;
    r->max_batch_jobs = SB_MAX_JOBS;
    return 0;
}

int salt_gpu_init(void) {
    Backend& B = g_backend;
    if (B.ready) return 0;
    int ndev = 0;
    if (!cuda_ok(cudaGetDeviceCount(&ndev), "cudaGetDeviceCount") || ndev < 1) return -1;
    cudaDeviceProp prop;
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice") ||
        !cuda_ok(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties"))
        return -1;
    if (prop.major != 10) {  // built for sm_100a only; there is no other code path
        if (getenv("SALT_GPU_DIAG")) fprintf(stderr, "salt-b200: device is sm_%d%d, need sm_100\n", prop.major, prop.minor);
        return -1;
    }
    const size_t stage = (size_t)SB_STAGE_FLOATS * sizeof(float);
    bool ok = cuda_ok(cudaStreamCreateWithFlags(&B.stream, cudaStreamNonBlocking), "stream") &&
              cuda_ok(cudaMalloc((void**)&B.d_x, stage), "stage x") &&
              cuda_ok(cudaMalloc((void**)&B.d_y, stage), "stage y") &&
              cuda_ok(cudaMalloc((void**)&B.d_mid, stage), "stage mid") &&
              cuda_ok(cudaMalloc((void**)&B.d_jobs, (size_t)SB_MAX_JOBS * sizeof(Q4Job)), "jobs") &&
              cuda_ok(cudaMalloc((void**)&B.d_status, sizeof(int)), "status") &&
              cuda_ok(cudaMemset(B.d_status, 0, sizeof(int)), "status") &&
              cuda_ok(cudaHostAlloc((void**)&B.h_x, stage, cudaHostAllocDefault), "pinned x") &&
              cuda_ok(cudaHostAlloc((void**)&B.h_y, stage, cudaHostAllocDefault), "pinned y") &&
              cuda_ok(cudaHostAlloc((void**)&B.h_jobs, (size_t)SB_MAX_JOBS * sizeof(Q4Job), cudaHostAllocDefault),
                      "pinned jobs");
    B.stage_floats = SB_STAGE_FLOATS;
    B.job_cap = SB_MAX_JOBS;
    if (!ok) {
        salt_gpu_free();
        return -1;
    }
    B.ready = true;
    return 0;
}

int salt_gpu_free(void) {
    Backend& B = g_backend;
    if (B.stream) cudaStreamSynchronize(B.stream);
    cudaDeviceSynchronize();
    for (auto& kv : B.tensors) release_tensor(kv.second);
    for (auto& kv : B.arena) release_tensor(kv.second);
    B.tensors.clear();
    B.arena.clear();
    for (auto& r : B.resources)
        if (r.dev) cudaFree(r.dev);
    B.resources.clear();
    for (auto& s : B.selected)
        if (s.own) cudaFree(s.own);
    residency_shutdown();
    B.selected.clear();
    B.logical_to_slot.clear();
    cudaFree(B.d_x); cudaFree(B.d_y); cudaFree(B.d_mid); cudaFree(B.d_jobs); cudaFree(B.d_status);
    if (B.h_x) cudaFreeHost(B.h_x);
    if (B.h_y) cudaFreeHost(B.h_y);
    if (B.h_jobs) cudaFreeHost(B.h_jobs);
    if (B.stream) cudaStreamDestroy(B.stream);
    fp4_release();
    const SaltGpuBatchStatsV2 keep = B.stats;
    const int mapped_only = B.mapped_only;
    B = Backend();
    B.stats = keep;  // counters are process-lifetime (tests compare deltas across re-init)
    B.mapped_only = mapped_only;
    return 0;
}

int salt_gpu_set_defer(int on) {
    Backend& B = g_backend;
    int rc = 0;
    if (!on && B.defer) rc = salt_gpu_sync();
    B.defer = on ? 1 : 0;
    return rc;
}
int salt_gpu_defer(void) { return g_backend.defer; }

int salt_gpu_sync(void) {
    Backend& B = g_backend;
    if (!B.ready) return 0;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "sync")) return -1;
    B.x_cursor = 0;
    int status = 0;
    if (!cuda_ok(cudaMemcpy(&status, B.d_status, sizeof status, cudaMemcpyDeviceToHost), "status")) return -1;
    if (status) {
        cudaMemset(B.d_status, 0, sizeof(int));
        return -1;
    }
    return 0;
}

void salt_gpu_set_mapped_only(int on) { g_backend.mapped_only = on ? 1 : 0; }
int salt_gpu_mapped_only(void) { return g_backend.mapped_only; }

void salt_gpu_batch_stats_get(SaltGpuBatchStats* s) {
    if (!s) return;
    const SaltGpuBatchStatsV2& v = g_backend.stats;
    s->arena_batches = v.arena_batches;
    s->trunk_batches = v.trunk_batches;
    s->expert_layer_batches = v.expert_layer_batches;
    s->mapped_only_misses = v.mapped_only_misses;
    s->direct_output_batches = v.direct_output_batches;
    s->direct_output_jobs = v.direct_output_jobs;
}

int salt_gpu_batch_stats_get_v2(SaltGpuBatchStatsV2* s, size_t n) {
    if (!s || n != sizeof *s) return -1;
    *s = g_backend.stats;
    return 0;
}

const SaltGpuDispatch* salt_dispatch_get(void) { return nullptr; }
int salt_gpu_cuda_present(void) { return 1; }
int salt_gpu_rocm_present(void) { return 0; }
int salt_gpu_pageable_mmap_active(void) { return 0; }
const struct SaltTextGpuProgramOps* salt_gpu_tensor_program_ops(void) { return nullptr; }

// ------------------------------------------------------------------------
// weight resources
// ------------------------------------------------------------------------
int salt_gpu_weight_resource_describe(uint32_t kind, uint32_t id, const void* base, size_t nbytes) {
    Backend& B = g_backend;
    if (!B.ready || !base || nbytes < 1 || find_resource(kind, id)) return -1;
    Resource r;
    r.kind = kind; r.id = id; r.host = (const uint8_t*)base; r.nbytes = nbytes;
    B.resources.push_back(r);
    return 0;
}

// Any explicit policy results in the same thing here: a byte-identical copy of
// the described range in HBM at a 256-byte aligned base.
int salt_gpu_weight_resource_activate(uint32_t kind, uint32_t id, SaltGpuWeightAddressability policy) {
    Backend& B = g_backend;
    Resource* r = find_resource(kind, id);
    if (!r || r->active || r->dev || policy == SALT_GPU_WEIGHT_ADDRESS_AUTO ||
        policy == SALT_GPU_WEIGHT_ADDRESS_BOUNDED_WINDOW)
        return -1;
    void* dev = nullptr;
    if (!cuda_ok(cudaMalloc(&dev, r->nbytes + 16), "resource alloc")) return -1;
    if (!cuda_ok(cudaMemcpy(dev, r->host, r->nbytes, cudaMemcpyHostToDevice), "resource copy")) {
        cudaFree(dev);
        return -1;
    }
    r->dev = (uint8_t*)dev;
    r->active = true;
    r->policy = (int)policy;
    B.copied_bytes += r->nbytes;
    return 0;
}

int salt_gpu_weight_resource_pool_bind(uint32_t, uint32_t) { return -1; }

int salt_gpu_weight_resource_deactivate(uint32_t kind, uint32_t id) {
    Backend& B = g_backend;
    Resource* r = find_resource(kind, id);
    if (!r || !r->active) return -1;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "deactivate fence") ||
        !cuda_ok(cudaDeviceSynchronize(), "deactivate fence"))
        return -1;
    for (auto& kv : B.tensors)
        if (kv.second.kind == kind && kv.second.id == id) {
            release_tensor(kv.second);
            kv.second.dv = kv.second.ds = kv.second.db = nullptr;
        }
    cudaFree(r->dev);
    r->dev = nullptr;
    r->active = false;
    r->policy = 0;
    r->window_off = r->window_bytes = 0;
    return 0;
}

int salt_gpu_weight_resource_usage(SaltGpuWeightResourceUsage* u, size_t n) {
    Backend& B = g_backend;
    if (!u || n != sizeof *u) return -1;
    memset(u, 0, sizeof *u);
    for (auto& r : B.resources) {
        u->described_resources++;
        u->described_bytes += r.nbytes;
        if (!r.active) continue;
        u->active_resources++;
        if (r.window_bytes) {
            u->active_windows++;
            u->active_window_bytes += r.window_bytes;
        }
    }
    u->peak_window_bytes = B.peak_window;
    u->device_copied_weight_bytes = B.copied_bytes;
    return 0;
}

int salt_gpu_weight_resource_bind(uint32_t kind, uint32_t id, const void* base, size_t nbytes) {
    Backend& B = g_backend;
    if (salt_gpu_weight_resource_describe(kind, id, base, nbytes) != 0) return -1;
    if (salt_gpu_weight_resource_activate(kind, id, SALT_GPU_WEIGHT_ADDRESS_REGISTERED_PERSISTENT) != 0) {
        for (size_t i = 0; i < B.resources.size(); i++)
            if (B.resources[i].kind == kind && B.resources[i].id == id) {
                B.resources.erase(B.resources.begin() + (long)i);
                break;
            }
        return -1;
    }
    return 0;
}

int salt_gpu_weight_window_bind(uint32_t kind, uint32_t id, uint64_t offset, size_t nbytes) {
    Backend& B = g_backend;
    Resource* r = find_resource(kind, id);
    if (!r || !r->active || r->window_bytes || nbytes < 1 || offset > r->nbytes || nbytes > r->nbytes - offset)
        return -1;
    r->window_off = offset;
    r->window_bytes = nbytes;
    B.peak_window = std::max<uint64_t>(B.peak_window, nbytes);
    return 0;
}

int salt_gpu_weight_window_unbind(uint32_t kind, uint32_t id) {
    Resource* r = find_resource(kind, id);
    if (!r || !r->active || !r->window_bytes) return -1;
    if (!cuda_ok(cudaDeviceSynchronize(), "window fence")) return -1;
    r->window_off = r->window_bytes = 0;
    return 0;
}

int salt_gpu_weight_resource_slot(uint32_t kind, uint32_t id, const void* key, const uint32_t* vals,
                                  const uint16_t* scales, const uint16_t* biases, int bits, int R, int C) {
    Backend& B = g_backend;
    Resource* r = live_resource(kind, id);
    size_t vb, gb;
    uint64_t vo, so, bo;
    if (!r || !key || !vals || !scales || !biases || !q4_sizes(bits, R, C, &vb, &gb) ||
        !in_range(*r, vals, vb, &vo) || !in_range(*r, scales, gb, &so) || !in_range(*r, biases, gb, &bo))
        return -1;
    auto it = B.tensors.find(key);
    if (it != B.tensors.end()) {
        const Tensor& t = it->second;
        return (t.kind == kind && t.id == id && t.bits == bits && t.R == R && t.C == C && t.voff == vo &&
                t.soff == so && t.boff == bo) ? 0 : -1;
    }
    Tensor t;
    t.kind = kind; t.id = id; t.bits = bits; t.R = R; t.C = C;
    t.voff = vo; t.soff = so; t.boff = bo; t.vbytes = vb; t.gbytes = gb;
    B.tensors[key] = t;
    return 0;
}

// BF16 matrices (router / head projections of packages that keep them in bf16; reference
// include/salt/gpu.h:60-66, src/gpu_cuda.cu:3267-3300): registered inside a described, active resource.
int salt_gpu_bf16_resource_slot(uint32_t kind, uint32_t id, const void* key, const uint16_t* weights, int R, int C) {
    Backend& B = g_backend;
    Resource* r = live_resource(kind, id);
    uint64_t vo;
    if (!r || !key || !weights || R < 1 || C < 8 || (C & 7) != 0) return -1;
    const uint64_t elems = (uint64_t)(uint32_t)R * (uint64_t)(uint32_t)C;
    if (elems > SIZE_MAX / 2u || !in_range(*r, weights, (size_t)(elems * 2u), &vo)) return -1;
    auto it = B.tensors.find(key);
    if (it != B.tensors.end()) {
        const Tensor& t = it->second;
        return (t.kind == kind && t.id == id && t.bits == 16 && t.R == R && t.C == C && t.voff == vo) ? 0 : -1;
    }
    Tensor t;
    t.kind = kind; t.id = id; t.bits = 16; t.R = R; t.C = C; t.voff = vo; t.vbytes = (size_t)(elems * 2u);
    B.tensors[key] = t;
    return 0;
}

// Device view of a registered bf16 matrix (2-byte alignment is all its kernels need).
static const uint16_t* bf16_view(const void* key, int R, int C) {
    Backend& B = g_backend;
    if (!B.ready || !key) return nullptr;
    auto it = B.tensors.find(key);
    if (it == B.tensors.end()) return nullptr;
    const Tensor& t = it->second;
    Resource* r = live_resource(t.kind, t.id);
    if (!r || t.bits != 16 || t.R != R || t.C != C) return nullptr;
    return (const uint16_t*)(r->dev + t.voff);
}

static int bf16_run(const void* key, int R, int C, int Bt, const float* in, float* out, bool serial) {
    Backend& B = g_backend;
    const uint16_t* W = bf16_view(key, R, C);
    if (!W) {
        if (B.ready && B.mapped_only) B.stats.mapped_only_misses++;
        return -1;
    }
    const size_t nin = (size_t)Bt * C, nout = (size_t)Bt * R;
    if (!in || !out || nin > B.stage_floats || nout > B.stage_floats) return -1;
    if (!cuda_ok(cudaMemcpyAsync(B.d_x, in, nin * sizeof(float), cudaMemcpyHostToDevice, B.stream), "bf16 x upload"))
        return -1;
    const cudaError_t e = serial ? launch_bf16_batch(W, B.d_x, B.d_y, R, C, Bt, B.stream)
                                 : launch_bf16_matvec(W, B.d_x, B.d_y, R, C, B.stream);
    if (!cuda_ok(e, "bf16 launch")) return -1;
    count_launches(1);
    if (!cuda_ok(cudaMemcpyAsync(out, B.d_y, nout * sizeof(float), cudaMemcpyDeviceToHost, B.stream), "bf16 y download") ||
        !cuda_ok(cudaStreamSynchronize(B.stream), "bf16 sync"))
        return -1;
    return 0;
}

int salt_gpu_bf16_matvec(const void* key, int R, int C, const float* input, float* output) {
    return bf16_run(key, R, C, 1, input, output, false);
}

// every (token, row) keeps the serial column order of the reference's portable loop
int salt_gpu_bf16_matvec_batch(const void* key, int R, int C, int Bt, const float* inputs, float* outputs) {
    if (Bt < 1) return -1;
    return bf16_run(key, R, C, Bt, inputs, outputs, true);
}

int salt_gpu_weight_resource_unbind(uint32_t kind, uint32_t id) {
    Backend& B = g_backend;
    Resource* r = find_resource(kind, id);
    if (!r) return -1;
    if (r->active && salt_gpu_weight_resource_deactivate(kind, id) != 0) return -1;
    for (auto it = B.tensors.begin(); it != B.tensors.end();) {
        if (it->second.kind == kind && it->second.id == id) {
            release_tensor(it->second);
            it = B.tensors.erase(it);
        } else {
            ++it;
        }
    }
    for (size_t i = 0; i < B.resources.size(); i++)
        if (B.resources[i].kind == kind && B.resources[i].id == id) {
            B.resources.erase(B.resources.begin() + (long)i);
            break;
        }
    return 0;
}

int salt_gpu_resident_trunk_map(const void* base, size_t nbytes) {
    return salt_gpu_weight_resource_bind(SALT_GPU_RESOURCE_TRUNK, 0, base, nbytes);
}
int salt_gpu_resident_trunk_unmap(void) { return salt_gpu_weight_resource_unbind(SALT_GPU_RESOURCE_TRUNK, 0); }
int salt_gpu_expert_resource_bind(uint32_t id, const void* base, size_t nbytes) {
    return salt_gpu_weight_resource_bind(SALT_GPU_RESOURCE_EXPERT_LAYER, id, base, nbytes);
}
int salt_gpu_expert_resource_slot(uint32_t id, const void* key, const uint32_t* vals, const uint16_t* scales,
                                  const uint16_t* biases, int R, int C) {
    return salt_gpu_weight_resource_slot(SALT_GPU_RESOURCE_EXPERT_LAYER, id, key, vals, scales, biases, 4, R, C);
}
int salt_gpu_expert_resource_unbind(uint32_t id) {
    return salt_gpu_weight_resource_unbind(SALT_GPU_RESOURCE_EXPERT_LAYER, id);
}
int salt_gpu_resident_pool_map(const void* base, size_t nbytes) {
    return salt_gpu_expert_resource_bind(0, base, nbytes);
}
int salt_gpu_resident_slot(const void* key, const uint32_t* vals, const uint16_t* scales, const uint16_t* biases,
                           int R, int C) {
    for (auto& r : g_backend.resources) {
        uint64_t off;
        if (r.kind == SALT_GPU_RESOURCE_EXPERT_LAYER && in_range(r, vals, 1, &off))
            return salt_gpu_expert_resource_slot(r.id, key, vals, scales, biases, R, C);
    }
    return -1;
}

// ------------------------------------------------------------------------
// selected-expert table: each bound slot owns an HBM copy of its payload
// ------------------------------------------------------------------------
int salt_gpu_selected_resources_prepare(int capacity, int logical_capacity) {
    Backend& B = g_backend;
    if (!B.ready || capacity < 1 || logical_capacity < 1) return -1;
    if (!B.selected.empty())
        return ((int)B.selected.size() == capacity && (int)B.logical_to_slot.size() == logical_capacity) ? 0 : -1;
    B.selected.assign((size_t)capacity, Selected());
    B.logical_to_slot.assign((size_t)logical_capacity, -1);
    return 0;
}

int salt_gpu_selected_resource_bind(int slot, uint64_t logical_id, const void* base, size_t nbytes,
                                    const void* payload) {
    Backend& B = g_backend;
    if (!B.ready || B.selected.empty() || slot < 0 || slot >= (int)B.selected.size() ||
        logical_id >= B.logical_to_slot.size() || !base || !payload || nbytes < 1)
        return -1;
    const uintptr_t b = (uintptr_t)base, p = (uintptr_t)payload;
    if (p < b || p - b >= nbytes) return -1;
    Selected& s = B.selected[(size_t)slot];
    if (s.active)
        return (s.logical_id == logical_id && s.base == base && s.payload == payload && s.nbytes == nbytes &&
                B.logical_to_slot[logical_id] == slot) ? 0 : -1;
    if (B.logical_to_slot[logical_id] != -1) return -1;
    const size_t payload_bytes = nbytes - (size_t)(p - b);
    if (s.own_cap < payload_bytes) {
        if (s.own) cudaFree(s.own);
        s.own = nullptr;
        s.own_cap = 0;
        void* d = nullptr;
        if (!cuda_ok(cudaMalloc(&d, payload_bytes + 16), "selected slot")) return -1;
        s.own = (uint8_t*)d;
        s.own_cap = payload_bytes;
    }
    if (!cuda_ok(cudaMemcpy(s.own, payload, payload_bytes, cudaMemcpyHostToDevice), "selected copy")) return -1;
    B.copied_bytes += payload_bytes;
    s.dev = s.own;
    s.resident = false;
    s.generation = 0;
    s.active = true;
    s.logical_id = logical_id;
    s.base = base; s.payload = payload; s.nbytes = nbytes;
    B.logical_to_slot[logical_id] = slot;
    B.selected_fenced = false;
    return 0;
}

// Publish a payload that the residency engine has already populated into seat `slot` of its arena
// (reference gpu.h:339-342; caller models/gemma4-26b-a4b/src/gemma4_text.c:1886-1940): no copy, the slot
// views the seat.  `payload` is only the host identity that later tensor pointers are measured from.
int salt_gpu_selected_resource_bind_resident(int slot, uint64_t logical_id, const void* payload, size_t nbytes,
                                             uintptr_t device_address, uint64_t generation) {
    Backend& B = g_backend;
    if (!B.ready || B.selected.empty() || slot < 0 || slot >= (int)B.selected.size() ||
        logical_id >= B.logical_to_slot.size() || !payload || nbytes < 1 || !device_address || generation == 0)
        return -1;
    if (residency_seat_address(slot, nbytes) != device_address) return -1;
    Selected& s = B.selected[(size_t)slot];
    if (s.active)
        return (s.resident && s.logical_id == logical_id && s.generation == generation && s.payload == payload &&
                s.nbytes == nbytes && s.dev == (uint8_t*)device_address && B.logical_to_slot[logical_id] == slot)
                   ? 0 : -1;
    if (B.logical_to_slot[logical_id] != -1) return -1;
    s.active = true;
    s.resident = true;
    s.generation = generation;
    s.logical_id = logical_id;
    s.base = payload; s.payload = payload; s.nbytes = nbytes;
    s.dev = (uint8_t*)device_address;
    B.logical_to_slot[logical_id] = slot;
    B.selected_fenced = false;
    return 0;
}

int salt_gpu_selected_resources_fence(void) {
    Backend& B = g_backend;
    if (!B.ready || B.selected.empty()) return -1;
    if (!cuda_ok(cudaDeviceSynchronize(), "selected fence")) return -1;
    B.selected_fenced = true;
    return 0;
}

int salt_gpu_selected_resource_unbind(int slot, uint64_t logical_id) {
    Backend& B = g_backend;
    if (B.selected.empty() || slot < 0 || slot >= (int)B.selected.size() || logical_id >= B.logical_to_slot.size())
        return -1;
    Selected& s = B.selected[(size_t)slot];
    if (!s.active) return 0;
    if (s.logical_id != logical_id || B.logical_to_slot[logical_id] != slot) return -1;
    if (!B.selected_fenced && !cuda_ok(cudaDeviceSynchronize(), "selected unbind fence")) return -1;
    B.logical_to_slot[logical_id] = -1;
    s.active = false;  // the device allocation is kept for the next occupant of the slot
    return 0;
}

// ------------------------------------------------------------------------
// affine-Q4 compute with host pointers
// ------------------------------------------------------------------------
static int q4_same_weight(const void* key, const uint32_t* vals, const uint16_t* scales, const uint16_t* biases,
                          int R, int C, int Bt, const float* const* xs, float* const* ys, int bits = 4) {
    Backend& B = g_backend;
    int kind = 0;
    if (!B.ready || R < 1 || C < 1 || Bt < 1 || !xs || !ys) return -1;
    Tensor* t = resolve_q4(key, vals, scales, biases, R, C, &kind, bits);
    if (!t) {
        if (B.mapped_only) B.stats.mapped_only_misses++;
        return -1;
    }
    if (!stage_reserve((size_t)Bt * C, (size_t)Bt * R, 0, 1)) return -1;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "fence")) return -1;
    for (int b = 0; b < Bt; b++) {
        if (!xs[b] || !ys[b]) return -1;
        memcpy(B.h_x + (size_t)b * C, xs[b], (size_t)C * sizeof(float));
    }
    if (!cuda_ok(cudaMemcpyAsync(B.d_x, B.h_x, (size_t)Bt * C * sizeof(float), cudaMemcpyHostToDevice, B.stream),
                 "x upload"))
        return -1;
    fill_job(B.h_jobs[0], *t, B.d_x, B.d_y, Bt, C, R);
    const bool aligned = (C % 64) == 0;
    if (!run_jobs(1, R, Bt, C, 1, aligned, bits) ||
        !cuda_ok(cudaMemcpyAsync(B.h_y, B.d_y, (size_t)Bt * R * sizeof(float), cudaMemcpyDeviceToHost, B.stream),
                 "y download") ||
        !cuda_ok(cudaStreamSynchronize(B.stream), "sync"))
        return -1;
    for (int b = 0; b < Bt; b++) memcpy(ys[b], B.h_y + (size_t)b * R, (size_t)R * sizeof(float));
    count_kinds(kind == SALT_GPU_RESOURCE_TRUNK, kind == SALT_GPU_RESOURCE_EXPERT_LAYER,
                kind == SALT_GPU_RESOURCE_ARENA);
    B.stats.direct_output_batches++;
    B.stats.direct_output_jobs += (uint64_t)Bt;
    return 0;
}

int salt_gpu_q4_matvec(const uint32_t* vals, const uint16_t* scales, const uint16_t* biases, int R, int C,
                       const float* x, float* y) {
    if (!x || !y) return -1;
    const float* xs[1] = {x};
    float* ys[1] = {y};
    return q4_same_weight(vals, vals, scales, biases, R, C, 1, xs, ys);
}

int salt_gpu_proj_batch(const uint32_t* vals, const uint16_t* scales, const uint16_t* biases, int R, int C, int Bt,
                        const float* const* xs, float* const* ys, const void* id) {
    return q4_same_weight(id ? id : vals, vals, scales, biases, R, C, Bt, xs, ys);
}

static int q_batch(int bits, const uint32_t* const* vals, const uint16_t* const* scales,
                   const uint16_t* const* biases, const float* const* xs, float* const* ys, const void* const* ids,
                   const int* Rj, int C, int njobs) {
    Backend& B = g_backend;
    if (!B.ready || !vals || !scales || !biases || !xs || !ys || !ids || !Rj || C < 1 || njobs < 1 ||
        (size_t)njobs > B.job_cap)
        return -1;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "fence")) return -1;
    size_t x_floats = 0, y_floats = 0;
    int max_rows = 0, ndesc = 0, max_tok = 1;
    bool trunk = false, expert = false, arena = false;
    std::vector<size_t> yoff((size_t)njobs);
    const float* last_x = nullptr;
    size_t last_x_off = 0;
    int last_run = 0;
    for (int j = 0; j < njobs;) {
        if (!vals[j] || !scales[j] || !biases[j] || !xs[j] || !ys[j] || Rj[j] < 1) return -1;
        int kind = 0;
        Tensor* t = resolve_q4(ids[j], vals[j], scales[j], biases[j], Rj[j], C, &kind, bits);
        if (!t) {
            if (B.mapped_only) B.stats.mapped_only_misses++;
            return -1;
        }
        // consecutive jobs on the same weights with contiguous rows become one multi-token job
        int run = 1;
        while (j + run < njobs && ids[j + run] == ids[j] && vals[j + run] == vals[j] && Rj[j + run] == Rj[j] &&
               xs[j + run] == xs[j] + (size_t)run * C && ys[j + run] == ys[j] + (size_t)run * Rj[j])
            run++;
        const bool reuse = last_x == xs[j] && last_run == run;
        if ((!reuse && x_floats + (size_t)run * C > B.stage_floats) ||
            y_floats + (size_t)run * Rj[j] > B.stage_floats)
            return -1;
        size_t xo = reuse ? last_x_off : x_floats;
        if (!reuse) {
            memcpy(B.h_x + x_floats, xs[j], (size_t)run * C * sizeof(float));
            last_x = xs[j]; last_x_off = x_floats; last_run = run;
            x_floats += (size_t)run * C;
        }
        fill_job(B.h_jobs[ndesc++], *t, B.d_x + xo, B.d_y + y_floats, run, C, Rj[j]);
        for (int i = 0; i < run; i++) yoff[(size_t)(j + i)] = y_floats + (size_t)i * Rj[j];
        y_floats += (size_t)run * Rj[j];
        max_rows = std::max(max_rows, Rj[j]);
        max_tok = std::max(max_tok, run);
        trunk |= kind == SALT_GPU_RESOURCE_TRUNK;
        expert |= kind == SALT_GPU_RESOURCE_EXPERT_LAYER;
        arena |= kind == SALT_GPU_RESOURCE_ARENA;
        j += run;
    }
    if (!cuda_ok(cudaMemcpyAsync(B.d_x, B.h_x, x_floats * sizeof(float), cudaMemcpyHostToDevice, B.stream),
                 "x upload") ||
        !run_jobs(ndesc, max_rows, max_tok, C, 1, (C % 64) == 0, bits) ||
        !cuda_ok(cudaMemcpyAsync(B.h_y, B.d_y, y_floats * sizeof(float), cudaMemcpyDeviceToHost, B.stream),
                 "y download") ||
        !cuda_ok(cudaStreamSynchronize(B.stream), "sync"))
        return -1;
    for (int j = 0; j < njobs; j++) memcpy(ys[j], B.h_y + yoff[(size_t)j], (size_t)Rj[j] * sizeof(float));
    count_kinds(trunk, expert, arena);
    B.stats.direct_output_batches++;
    B.stats.direct_output_jobs += (uint64_t)njobs;
    return 0;
}

int salt_gpu_q4_batch(const uint32_t* const* vals, const uint16_t* const* scales, const uint16_t* const* biases,
                      const float* const* xs, float* const* ys, const void* const* ids, const int* Rj, int C,
                      int njobs) {
    return q_batch(4, vals, scales, biases, xs, ys, ids, Rj, C, njobs);
}

// Affine 8-bit (reference src/kernels.c:343-369): same registry, staging and statistics as the
// 4-bit entry points; the values are one byte per element.
int salt_gpu_q8_matvec(const uint32_t* vals, const uint16_t* scales, const uint16_t* biases, int R, int C,
                       const float* x, float* y) {
    if (!x || !y) return -1;
    const float* xs[1] = {x};
    float* ys[1] = {y};
    return q4_same_weight(vals, vals, scales, biases, R, C, 1, xs, ys, 8);
}

int salt_gpu_q8_batch(const uint32_t* const* vals, const uint16_t* const* scales, const uint16_t* const* biases,
                      const float* const* xs, float* const* ys, const void* const* ids, const int* Rj, int C,
                      int njobs) {
    return q_batch(8, vals, scales, biases, xs, ys, ids, Rj, C, njobs);
}

// Jobs [first_job, first_job+job_count) of a [B][C] batch, written straight into
// a shared buffer (device alias of pinned host memory); asynchronous, fenced by
// salt_gpu_sync (reference gpu.h:349-362).
int salt_gpu_proj_batch_indexed(const uint32_t* vals, const uint16_t* scales, const uint16_t* biases, int R, int C,
                                int Bt, int first_job, int job_count, const float* xs, SaltGpuSharedBuffer* output,
                                size_t y_float_offset, const void* id) {
    Backend& B = g_backend;
    if (!B.ready || !vals || !scales || !xs || !output || !output->contents || !output->backend || !id || R < 1 ||
        C < 1 || Bt < 1 || first_job < 0 || job_count < 1 || first_job > Bt - job_count)
        return -1;
    const uint64_t span = (uint64_t)(uint32_t)Bt * (uint32_t)R;
    const uint64_t cap = output->nbytes / sizeof(float);
    if (span > UINT32_MAX || (uint64_t)y_float_offset > (uint64_t)UINT32_MAX - span ||
        (uint64_t)y_float_offset > cap || span > cap - (uint64_t)y_float_offset)
        return -1;
    int kind = 0;
    Tensor* t = resolve_q4(id, vals, scales, biases, R, C, &kind);
    if (!t) {
        if (B.mapped_only) B.stats.mapped_only_misses++;
        return -1;
    }
    const size_t need = (size_t)job_count * C;
    if (need > B.stage_floats) return -1;
    if (B.x_cursor + need > B.stage_floats) {
        if (!cuda_ok(cudaStreamSynchronize(B.stream), "stage wrap")) return -1;
        B.x_cursor = 0;
    }
    float* dx = B.d_x + B.x_cursor;
    B.x_cursor += need;
    if (!cuda_ok(cudaMemcpyAsync(dx, xs + (size_t)first_job * C, need * sizeof(float), cudaMemcpyHostToDevice,
                                 B.stream), "x upload"))
        return -1;
    // descriptor ring: one slot per outstanding call
    if (B.job_cursor >= B.job_cap) {
        if (!cuda_ok(cudaStreamSynchronize(B.stream), "job wrap")) return -1;
        B.job_cursor = 0;
    }
    Q4Job* hj = B.h_jobs + B.job_cursor;
    Q4Job* dj = B.d_jobs + B.job_cursor;
    B.job_cursor++;
    fill_job(*hj, *t, dx, (float*)output->backend + y_float_offset + (size_t)first_job * R, job_count, C, R);
    if (!cuda_ok(cudaMemcpyAsync(dj, hj, sizeof(Q4Job), cudaMemcpyHostToDevice, B.stream), "job upload") ||
        !cuda_ok(launch_q4_jobs(dj, 1, nullptr, R, job_count, C, 1, (C % 64) == 0, B.stream), "launch"))
        return -1;
    count_launches(1);
    count_kinds(kind == SALT_GPU_RESOURCE_TRUNK, kind == SALT_GPU_RESOURCE_EXPERT_LAYER,
                kind == SALT_GPU_RESOURCE_ARENA);
    B.stats.direct_output_batches++;
    B.stats.direct_output_jobs += (uint64_t)job_count;
    if (!B.defer) {
        // host pointers may be reused by the caller right away; the result is
        // still only published by salt_gpu_sync().
    }
    return 0;
}

int salt_gpu_proj_batch_indexed_exact_views(const uint32_t* vals, const uint16_t* scales, const uint16_t* biases,
                                            int R, int C, int Bt, int first_job, int job_count, const float* xs,
                                            SaltGpuSharedBuffer* output, size_t y_float_offset, const void* id) {
    return salt_gpu_proj_batch_indexed(vals, scales, biases, R, C, Bt, first_job, job_count, xs, output,
                                       y_float_offset, id);
}

// One expert tensor of a MoE chain: a registered key, or a view into a bound
// selected-resource slot (reference src/gpu_cuda.cu:4630-4700).
static bool chain_tensor(const uint32_t* vals, const uint16_t* scales, const uint16_t* biases, const void* id, int R,
                         int C, int slot, uint64_t logical_id, bool require_selected, Tensor* out, int* kind) {
    Backend& B = g_backend;
    size_t vb, gb;
    if (!vals || !scales || !biases || !id || !q4_sizes(4, R, C, &vb, &gb)) return false;
    if (!require_selected && B.tensors.find(id) != B.tensors.end()) slot = -1;  // a registered key wins
    if (slot < 0) {
        Tensor* t = resolve_q4(id, vals, scales, biases, R, C, kind);
        if (!t) return false;
        *out = *t;
        out->owned.clear();
        return true;
    }
    if (slot < 0 || slot >= (int)B.selected.size()) return false;
    const Selected& s = B.selected[(size_t)slot];
    if (!s.active || !s.dev || s.logical_id != logical_id || logical_id >= B.logical_to_slot.size() ||
        B.logical_to_slot[logical_id] != slot)
        return false;
    const uintptr_t p0 = (uintptr_t)s.payload, p1 = (uintptr_t)s.base + s.nbytes;
    const uintptr_t v = (uintptr_t)vals, sc = (uintptr_t)scales, bi = (uintptr_t)biases, ident = (uintptr_t)id;
    if (v < p0 || sc < p0 || bi < p0 || ident < p0 || ident >= p1 || v > p1 || sc > p1 || bi > p1 ||
        vb > p1 - v || gb > p1 - sc || gb > p1 - bi)
        return false;
    Tensor t;
    t.kind = SALT_GPU_RESOURCE_EXPERT_LAYER; t.bits = 4; t.R = R; t.C = C; t.vbytes = vb; t.gbytes = gb;
    t.dv = s.dev + (v - p0); t.ds = s.dev + (sc - p0); t.db = s.dev + (bi - p0);
    *out = t;
    *kind = SALT_GPU_RESOURCE_EXPERT_LAYER;
    return true;
}

static bool ptr_aligned16(const Tensor& t) {
    return (((uintptr_t)t.dv | (uintptr_t)t.ds | (uintptr_t)t.db) & 15) == 0;
}

static int moe_chain(const SaltGpuMoeExpert* experts, int count, int hidden, int routed, const float* inputs,
                     float* outputs, float* gate_scratch, float* up_scratch, size_t scratch_cap,
                     bool require_selected) {
    Backend& B = g_backend;
    if (!B.ready || !experts || !inputs || !outputs || !gate_scratch || !up_scratch || scratch_cap < 1 ||
        count < 1 || (size_t)(2 * count) > B.job_cap || hidden < 1 || routed < 1)
        return -1;
    uint64_t total_rows = 0;
    int max_group = 0;
    for (int i = 0; i < count; i++) {
        if (experts[i].group < 1) return -1;
        total_rows += (uint32_t)experts[i].group;
        max_group = std::max(max_group, experts[i].group);
    }
    if (total_rows * (uint64_t)hidden > B.stage_floats || total_rows * (uint64_t)routed > B.stage_floats) return -1;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "fence")) return -1;
    bool aligned = (hidden % 64) == 0 && (routed % 64) == 0;
    size_t row = 0;
    for (int i = 0; i < count; i++) {
        const SaltGpuMoeExpert& e = experts[i];
        Tensor g, u, d;
        int kind = 0;
        if (!chain_tensor(e.gate_vals, e.gate_scales, e.gate_biases, e.gate_id, routed, hidden, e.resource_slot,
                          e.logical_resource_id, require_selected, &g, &kind) ||
            !chain_tensor(e.up_vals, e.up_scales, e.up_biases, e.up_id, routed, hidden, e.resource_slot,
                          e.logical_resource_id, require_selected, &u, &kind) ||
            !chain_tensor(e.down_vals, e.down_scales, e.down_biases, e.down_id, hidden, routed, e.resource_slot,
                          e.logical_resource_id, require_selected, &d, &kind))
            return -1;
        aligned = aligned && ptr_aligned16(g) && ptr_aligned16(u) && ptr_aligned16(d);
        Q4Job& gu = B.h_jobs[i];
        fill_job(gu, g, B.d_x + row * hidden, B.d_mid + row * routed, e.group, hidden, routed);
        gu.vals2 = u.dv; gu.scales2 = u.ds; gu.biases2 = u.db;
        Q4Job& dn = B.h_jobs[count + i];
        fill_job(dn, d, B.d_mid + row * routed, B.d_y + row * hidden, e.group, routed, hidden);
        row += (size_t)e.group;
    }
    const size_t in_bytes = (size_t)total_rows * hidden * sizeof(float);
    if (!cuda_ok(cudaMemcpyAsync(B.d_x, inputs, in_bytes, cudaMemcpyHostToDevice, B.stream), "x upload") ||
        !cuda_ok(cudaMemcpyAsync(B.d_jobs, B.h_jobs, (size_t)(2 * count) * sizeof(Q4Job), cudaMemcpyHostToDevice,
                                 B.stream), "job upload") ||
        !cuda_ok(launch_q4_jobs(B.d_jobs, count, nullptr, routed, max_group, hidden, 2, aligned, B.stream),
                 "gate/up launch") ||
        !cuda_ok(launch_q4_jobs(B.d_jobs + count, count, nullptr, hidden, max_group, routed, 1, aligned, B.stream),
                 "down launch") ||
        !cuda_ok(cudaMemcpyAsync(outputs, B.d_y, in_bytes, cudaMemcpyDeviceToHost, B.stream), "y download") ||
        !cuda_ok(cudaStreamSynchronize(B.stream), "sync"))
        return -1;
    count_launches(2);
    B.stats.expert_layer_batches++;
    B.stats.direct_output_batches++;
    B.stats.direct_output_jobs += (uint64_t)count;
    return 0;
}

int salt_gpu_q4_moe_chain(const SaltGpuMoeExpert* experts, int count, int hidden, int routed, const float* inputs,
                          float* outputs, float* gate_scratch, float* up_scratch, size_t cap) {
    return moe_chain(experts, count, hidden, routed, inputs, outputs, gate_scratch, up_scratch, cap, false);
}

int salt_gpu_q4_moe_chain_selected(const SaltGpuMoeExpert* experts, int count, int hidden, int routed,
                                   const float* inputs, float* outputs, float* gate_scratch, float* up_scratch,
                                   size_t cap) {
    return moe_chain(experts, count, hidden, routed, inputs, outputs, gate_scratch, up_scratch, cap, true);
}

// Heterogeneous projections whose inputs and outputs live inside one shared
// arena (reference gpu.h:311-316); no staging, no output scatter.
int salt_gpu_q4_selected_shared(const SaltGpuSelectedProjectionJob* jobs, int job_count,
                                SaltGpuSharedBuffer* arena) {
    Backend& B = g_backend;
    if (!B.ready || !jobs || job_count < 1 || (size_t)job_count > B.job_cap || !arena || !arena->contents ||
        !arena->backend || arena->nbytes < sizeof(float))
        return -1;
    const uintptr_t a0 = (uintptr_t)arena->contents, a1 = a0 + arena->nbytes;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "fence")) return -1;
    std::vector<int> order((size_t)job_count);
    for (int i = 0; i < job_count; i++) order[(size_t)i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return jobs[a].cols < jobs[b].cols; });
    std::vector<bool> aligned_by_desc((size_t)job_count, true);
    for (int n = 0; n < job_count; n++) {
        const SaltGpuSelectedProjectionJob& j = jobs[order[(size_t)n]];
        Tensor t;
        int kind = 0;
        if (j.rows < 1 || j.cols < 1 || j.batch < 1 || !j.inputs || !j.outputs ||
            !chain_tensor(j.vals, j.scales, j.biases, j.id, j.rows, j.cols, j.resource_slot,
                          j.logical_resource_id, false, &t, &kind))
            return -1;
        const uintptr_t in0 = (uintptr_t)j.inputs, out0 = (uintptr_t)j.outputs;
        const size_t in_bytes = (size_t)j.batch * j.cols * sizeof(float);
        const size_t out_bytes = (size_t)j.batch * j.rows * sizeof(float);
        if (in0 < a0 || in0 > a1 || in_bytes > a1 - in0 || out0 < a0 || out0 > a1 || out_bytes > a1 - out0 ||
            (in0 < out0 + out_bytes && out0 < in0 + in_bytes))
            return -1;
        fill_job(B.h_jobs[n], t, (const float*)((uint8_t*)arena->backend + (in0 - a0)),
                 (float*)((uint8_t*)arena->backend + (out0 - a0)), j.batch, j.cols, j.rows);
        aligned_by_desc[(size_t)n] = ptr_aligned16(t) && (j.cols % 64) == 0 && ((in0 - a0) % 16) == 0;
    }
    if (!cuda_ok(cudaMemcpyAsync(B.d_jobs, B.h_jobs, (size_t)job_count * sizeof(Q4Job), cudaMemcpyHostToDevice,
                                 B.stream), "job upload"))
        return -1;
    for (int n0 = 0; n0 < job_count;) {
        int n1 = n0, max_rows = 0, max_tok = 1;
        bool aligned = true;
        const int C = jobs[order[(size_t)n0]].cols;
        while (n1 < job_count && jobs[order[(size_t)n1]].cols == C) {
            max_rows = std::max(max_rows, jobs[order[(size_t)n1]].rows);
            max_tok = std::max(max_tok, jobs[order[(size_t)n1]].batch);
            aligned = aligned && aligned_by_desc[(size_t)n1];
            n1++;
        }
        if (!cuda_ok(launch_q4_jobs(B.d_jobs + n0, n1 - n0, nullptr, max_rows, max_tok, C, 1, aligned, B.stream),
                     "selected launch"))
            return -1;
        count_launches(1);
        n0 = n1;
    }
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "sync")) return -1;
    B.stats.expert_layer_batches++;
    B.stats.direct_output_batches++;
    B.stats.direct_output_jobs += (uint64_t)job_count;
    return 0;
}

// ------------------------------------------------------------------------
// shared buffers and exact cells
// ------------------------------------------------------------------------
int salt_gpu_shared_buffer_alloc(SaltGpuSharedBuffer* buffer, size_t nbytes) {
    if (!buffer || !g_backend.ready || nbytes < 1) return -1;
    memset(buffer, 0, sizeof *buffer);
    void* host = nullptr;
    void* dev = nullptr;
    if (!cuda_ok(cudaHostAlloc(&host, nbytes, cudaHostAllocMapped), "shared alloc") ||
        !cuda_ok(cudaHostGetDevicePointer(&dev, host, 0), "shared alias")) {
        if (host) cudaFreeHost(host);
        return -1;
    }
    buffer->contents = host;
    buffer->nbytes = nbytes;
    buffer->backend = dev;
    return 0;
}

int salt_gpu_shared_buffer_free(SaltGpuSharedBuffer* buffer) {
    if (!buffer) return -1;
    if (!buffer->contents && !buffer->backend && buffer->nbytes == 0) return 0;
    if (!buffer->contents || !buffer->backend || buffer->nbytes < 1) return -1;
    if (!cuda_ok(cudaDeviceSynchronize(), "shared free fence") || !cuda_ok(cudaFreeHost(buffer->contents), "free"))
        return -1;
    memset(buffer, 0, sizeof *buffer);
    return 0;
}

static bool cell_view(const SaltGpuSharedBuffer* b, size_t offset, size_t elements, void** out) {
    if (!b || !b->contents || !b->backend || b->nbytes < sizeof(float)) return false;
    const size_t cap = b->nbytes / sizeof(float);
    if (offset > cap || elements > cap - offset) return false;
    *out = (uint8_t*)b->backend + offset * sizeof(float);
    return true;
}

int salt_gpu_exact_cells(const SaltGpuExactCell* cells, int count) {
    Backend& B = g_backend;
    if (!B.ready || !cells || count < 1) return -1;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "fence") ||
        !cuda_ok(cudaMemsetAsync(B.d_status, 0, sizeof(int), B.stream), "status"))
        return -1;
    for (int i = 0; i < count; i++) {
        const SaltGpuExactCell& c = cells[i];
        void* v[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
        if (c.n == 0) return -1;
        switch (c.kind) {
            case SALT_GPU_EXACT_RMSNORM:
                if (c.aux > 1u || !cell_view(c.views[0], c.offsets[0], c.n, &v[0]) ||
                    !cell_view(c.views[1], c.offsets[1], c.aux ? c.n : 1u, &v[1]) ||
                    !cell_view(c.views[2], c.offsets[2], c.n, &v[2]))
                    return -1;
                if (!cuda_ok(launch_rmsnorm((const float*)v[0], (const float*)v[1], (float*)v[2], 1, (int)c.n, c.eps,
                                            (int)c.aux, B.d_status, B.stream), "rmsnorm cell"))
                    return -1;
                break;
            case SALT_GPU_EXACT_TOPK:
                if (c.aux == 0 || c.aux > c.n || !cell_view(c.views[0], c.offsets[0], c.n, &v[0]) ||
                    !cell_view(c.views[1], c.offsets[1], c.n, &v[1]) ||
                    !cell_view(c.views[2], c.offsets[2], c.aux, &v[2]) ||
                    !cell_view(c.views[3], c.offsets[3], c.aux, &v[3]))
                    return -1;
                if (!cuda_ok(launch_router_topk((const float*)v[0], (const float*)v[1], (int32_t*)v[2], (float*)v[3],
                                                1, (int)c.n, (int)c.aux, 1, B.d_status, B.stream), "topk cell"))
                    return -1;
                break;
            case SALT_GPU_EXACT_ROUTER_INPUT:
                if (!cell_view(c.views[0], c.offsets[0], c.n, &v[0]) ||
                    !cell_view(c.views[1], c.offsets[1], c.n, &v[1]) ||
                    !cell_view(c.views[2], c.offsets[2], c.n, &v[2]))
                    return -1;
                if (!cuda_ok(launch_router_input((const float*)v[0], (const float*)v[1], (float*)v[2], 1, (int)c.n,
                                                 c.eps, c.scalar, B.d_status, B.stream), "router-input cell"))
                    return -1;
                break;
            case SALT_GPU_EXACT_RESIDUAL_POSTNORM:
                for (int k = 0; k < 4; k++)
                    if (!cell_view(c.views[k], c.offsets[k], c.n, &v[k])) return -1;
                if (!(c.eps >= 0.0f) || !std::isfinite(c.eps) ||
                    !cuda_ok(launch_residual_postnorm((const float*)v[0], (const float*)v[1], (const float*)v[2],
                                                      (float*)v[3], 1, (int)c.n, c.eps, B.d_status, B.stream),
                             "residual cell"))
                    return -1;
                break;
            case SALT_GPU_EXACT_PARALLEL_COMBINE:
                for (int k = 0; k < 8; k++) {
                    const size_t elements = k == 6 ? (size_t)c.n * 2u : c.n;
                    if (!cell_view(c.views[k], c.offsets[k], elements, &v[k])) return -1;
                }
                if (!(c.eps >= 0.0f) || !std::isfinite(c.eps) || !std::isfinite(c.scalar) ||
                    !cuda_ok(launch_parallel_combine((const float*)v[0], (const float*)v[1], (const float*)v[2],
                                                     (const float*)v[3], (const float*)v[4], (const float*)v[5],
                                                     (float*)v[6], (float*)v[6] + c.n, (float*)v[7], 1, (int)c.n,
                                                     c.eps, c.scalar, B.d_status, B.stream),
                             "combine cell"))
                    return -1;
                break;
            case SALT_GPU_EXACT_SOFTCAP:
                if (!(c.scalar > 0.0f) || !std::isfinite(c.scalar) ||
                    !cell_view(c.views[0], c.offsets[0], c.n, &v[0]) ||
                    !cuda_ok(launch_softcap((float*)v[0], (int)c.n, c.scalar, B.d_status, B.stream), "softcap cell"))
                    return -1;
                break;
            default:
                return -1;
        }
        count_launches(1);
    }
    return salt_gpu_sync();
}

uint64_t salt_b200_launch_count(void) { return launch_count(); }

}  // extern "C"
