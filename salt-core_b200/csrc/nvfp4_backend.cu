// NVFP4 entry points of the reference operator surface (reference
// include/salt/gpu.h:41-59, 475-480; reference behaviour src/gpu_cuda.cu:3540-3770).
// A projection is W4A4: the activations go through the dynamic group-16
// quantise/dequantise first (one launch for all rows of the call), then one
// projection launch over all jobs.  Host pointers in, host pointers out,
// synchronous.
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "../../include/salt_gpu_b200.h"
#include "backend_state.h"
#include "internal.h"
#include "q4_core.cuh"

namespace sb {

constexpr int FMT_NVFP4 = 104;

struct Fp4Scratch {
    uint8_t *d_packed = nullptr, *d_scales = nullptr;
    float *d_ig = nullptr, *h_ig = nullptr;
    Fp4Job *d_jobs = nullptr, *h_jobs = nullptr;
    bool ready = false;
};
static Fp4Scratch g_fp4;

// Lazily carved once after salt_gpu_init; sizes follow the fixed staging capacity.
static bool fp4_ready() {
    Backend& B = g_backend;
    if (!B.ready) return false;
    if (g_fp4.ready) return true;
    const size_t rows_cap = SB_MAX_JOBS;
    bool ok = cuda_ok(cudaMalloc((void**)&g_fp4.d_packed, B.stage_floats / 2), "fp4 packed") &&
              cuda_ok(cudaMalloc((void**)&g_fp4.d_scales, B.stage_floats / 16), "fp4 scales") &&
              cuda_ok(cudaMalloc((void**)&g_fp4.d_ig, rows_cap * sizeof(float)), "fp4 ig") &&
              cuda_ok(cudaHostAlloc((void**)&g_fp4.h_ig, rows_cap * sizeof(float), cudaHostAllocDefault), "fp4 ig") &&
              cuda_ok(cudaMalloc((void**)&g_fp4.d_jobs, SB_MAX_JOBS * sizeof(Fp4Job)), "fp4 jobs") &&
              cuda_ok(cudaHostAlloc((void**)&g_fp4.h_jobs, SB_MAX_JOBS * sizeof(Fp4Job), cudaHostAllocDefault),
                      "fp4 jobs");
    g_fp4.ready = ok;
    return ok;
}

void fp4_release() {
    cudaFree(g_fp4.d_packed); cudaFree(g_fp4.d_scales); cudaFree(g_fp4.d_ig); cudaFree(g_fp4.d_jobs);
    if (g_fp4.h_ig) cudaFreeHost(g_fp4.h_ig);
    if (g_fp4.h_jobs) cudaFreeHost(g_fp4.h_jobs);
    g_fp4 = Fp4Scratch();
}

static Tensor* fp4_tensor(const void* key, int R, int C, const Resource** res_out) {
    Backend& B = g_backend;
    auto it = B.tensors.find(key);
    if (it == B.tensors.end()) return nullptr;
    Tensor& t = it->second;
    if (t.bits != FMT_NVFP4 || t.R != R || t.C != C) return nullptr;
    for (auto& r : B.resources)
        if (r.kind == t.kind && r.id == t.id && r.active && r.dev) {
            if (!t.dv) {
                // codes and scales must be 16-byte aligned for the tile kernel; copy if not
                const uint64_t offs[2] = {t.voff, t.soff};
                const size_t sizes[2] = {t.vbytes, t.gbytes};
                const uint8_t* out[2];
                for (int i = 0; i < 2; i++) {
                    const uint8_t* p = r.dev + offs[i];
                    if (((uintptr_t)p & 15) != 0) {
                        void* copy = nullptr;
                        if (!cuda_ok(cudaMalloc(&copy, sizes[i] + 16), "fp4 realign") ||
                            !cuda_ok(cudaMemcpy(copy, p, sizes[i], cudaMemcpyDeviceToDevice), "fp4 realign"))
                            return nullptr;
                        t.owned.push_back(copy);
                        p = (const uint8_t*)copy;
                    }
                    out[i] = p;
                }
                t.dv = out[0];
                t.ds = out[1];
            }
            *res_out = &r;
            return &t;
        }
    return nullptr;
}

// rows of all jobs are staged contiguously in d_x; ig per row in h_ig.
static int fp4_run(const std::vector<Tensor*>& tensors, const float* const* inputs, float* const* outputs,
                   const int* batches, const int* rows_per_job, int C, int njobs) {
    Backend& B = g_backend;
    size_t total_rows = 0, out_floats = 0;
    for (int j = 0; j < njobs; j++) {
        if (batches[j] < 1 || !inputs[j] || !outputs[j]) return -1;
        total_rows += (size_t)batches[j];
        out_floats += (size_t)batches[j] * rows_per_job[j];
    }
    if (total_rows > SB_MAX_JOBS || total_rows * (size_t)C > B.stage_floats || out_floats > B.stage_floats ||
        (size_t)njobs > SB_MAX_JOBS)
        return -1;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "fence")) return -1;
    size_t row = 0, yoff = 0;
    int max_rows = 0, max_tok = 1;
    bool aligned = true;
    uint64_t wbytes = 0, sbytes = 0;
    for (int j = 0; j < njobs; j++) {
        const Tensor& t = *tensors[(size_t)j];
        memcpy(B.h_x + row * C, inputs[j], (size_t)batches[j] * C * sizeof(float));
        for (int b = 0; b < batches[j]; b++) g_fp4.h_ig[row + b] = t.input_global;
        Fp4Job& fj = g_fp4.h_jobs[j];
        fj.codes = t.dv; fj.scales = t.ds; fj.wg = 1.0f / t.weight_divisor;
        fj.x = B.d_mid + row * C; fj.y = B.d_y + yoff;
        fj.R = t.R; fj.C = C; fj.ntok = batches[j]; fj.x_stride = C; fj.y_stride = t.R;
        aligned = aligned && ((((uintptr_t)t.dv | (uintptr_t)t.ds) & 15) == 0);
        max_rows = std::max(max_rows, t.R);
        max_tok = std::max(max_tok, batches[j]);
        wbytes += t.vbytes; sbytes += t.gbytes;
        row += (size_t)batches[j];
        yoff += (size_t)batches[j] * t.R;
    }
    const size_t in_bytes = total_rows * C * sizeof(float);
    if (!cuda_ok(cudaMemcpyAsync(B.d_x, B.h_x, in_bytes, cudaMemcpyHostToDevice, B.stream), "fp4 x") ||
        !cuda_ok(cudaMemcpyAsync(g_fp4.d_ig, g_fp4.h_ig, total_rows * sizeof(float), cudaMemcpyHostToDevice,
                                 B.stream), "fp4 ig") ||
        !cuda_ok(cudaMemcpyAsync(g_fp4.d_jobs, g_fp4.h_jobs, (size_t)njobs * sizeof(Fp4Job), cudaMemcpyHostToDevice,
                                 B.stream), "fp4 jobs") ||
        !cuda_ok(launch_nvfp4_qdq(B.d_x, (int)total_rows, C, g_fp4.d_ig, g_fp4.d_packed, g_fp4.d_scales, B.d_mid,
                                  B.d_status, B.stream), "fp4 qdq") ||
        !cuda_ok(launch_nvfp4_jobs(g_fp4.d_jobs, njobs, max_rows, max_tok, C, aligned, B.stream), "fp4 proj") ||
        !cuda_ok(cudaMemcpyAsync(B.h_y, B.d_y, out_floats * sizeof(float), cudaMemcpyDeviceToHost, B.stream),
                 "fp4 y"))
        return -1;
    count_launches(2);
    if (salt_gpu_sync() != 0) return -1;   // also reports non-finite activations
    yoff = 0;
    for (int j = 0; j < njobs; j++) {
        const size_t n = (size_t)batches[j] * rows_per_job[j];
        memcpy(outputs[j], B.h_y + yoff, n * sizeof(float));
        yoff += n;
    }
    SaltGpuBatchStatsV2& s = B.stats;
    s.nvfp4_logical_packed_weight_bytes += wbytes;
    s.nvfp4_logical_weight_scale_bytes += sbytes;
    s.nvfp4_activation_input_bytes += in_bytes;
    s.nvfp4_activation_qdq_bytes += total_rows * ((size_t)C / 2 + (size_t)C / 16 + (size_t)C * 4);
    s.nvfp4_projection_output_bytes += out_floats * sizeof(float);
    s.nvfp4_kernel_launches += 2;
    s.nvfp4_completion_fences += 1;
    s.direct_output_batches++;
    s.direct_output_jobs += (uint64_t)njobs;
    return 0;
}

}  // namespace sb

using namespace sb;

extern "C" {

int salt_gpu_nvfp4_resource_slot(uint32_t kind, uint32_t id, const void* key, const uint8_t* weight_packed,
                                 const uint8_t* weight_scales, const float* weight_global_scale,
                                 const float* input_global_scale, int R, int C) {
    Backend& B = g_backend;
    if (!B.ready || !key || !weight_packed || !weight_scales || !weight_global_scale || !input_global_scale ||
        R < 1 || C < 16 || (C & 15))
        return -1;
    Resource* res = nullptr;
    for (auto& r : B.resources)
        if (r.kind == kind && r.id == id && r.active && r.dev) res = &r;
    if (!res) return -1;
    const uint64_t elems = (uint64_t)(uint32_t)R * (uint32_t)C;
    const size_t vb = (size_t)(elems / 2), sb_ = (size_t)(elems / 16);
    auto inside = [&](const void* p, size_t n, uint64_t* off) {
        const uintptr_t b = (uintptr_t)res->host, v = (uintptr_t)p;
        if (v < b || v - b > res->nbytes || n > res->nbytes - (v - b)) return false;
        *off = v - b;
        return true;
    };
    uint64_t vo, so, wo, io;
    if (!inside(weight_packed, vb, &vo) || !inside(weight_scales, sb_, &so) ||
        !inside(weight_global_scale, sizeof(float), &wo) || !inside(input_global_scale, sizeof(float), &io))
        return -1;
    auto it = B.tensors.find(key);
    if (it != B.tensors.end()) {
        const Tensor& t = it->second;
        return (t.kind == kind && t.id == id && t.bits == FMT_NVFP4 && t.R == R && t.C == C && t.voff == vo &&
                t.soff == so && t.boff == wo && t.aoff == io) ? 0 : -1;
    }
    Tensor t;
    t.kind = kind; t.id = id; t.bits = FMT_NVFP4; t.R = R; t.C = C;
    t.voff = vo; t.soff = so; t.boff = wo; t.aoff = io; t.vbytes = vb; t.gbytes = sb_;
    memcpy(&t.weight_divisor, weight_global_scale, sizeof(float));
    memcpy(&t.input_global, input_global_scale, sizeof(float));
    if (!isfinite(t.weight_divisor) || t.weight_divisor == 0.0f || !isfinite(t.input_global) ||
        !(t.input_global > 0.0f))
        return -1;
    B.tensors[key] = t;
    return 0;
}

int salt_gpu_nvfp4_qdq(const float* input, int C, float input_global_scale, uint8_t* packed, uint8_t* scales,
                       float* dequant) {
    Backend& B = g_backend;
    if (!fp4_ready() || !input || !packed || !scales || !dequant || C < 16 || (C & 15) ||
        !isfinite(input_global_scale) || !(input_global_scale > 0.0f) || (size_t)C > B.stage_floats)
        return -1;
    if (!cuda_ok(cudaStreamSynchronize(B.stream), "fence")) return -1;
    g_fp4.h_ig[0] = input_global_scale;
    uint8_t* hp = (uint8_t*)B.h_y;                      // pinned scratch for the byte outputs
    if (!cuda_ok(cudaMemcpyAsync(B.d_x, input, (size_t)C * sizeof(float), cudaMemcpyHostToDevice, B.stream), "x") ||
        !cuda_ok(cudaMemcpyAsync(g_fp4.d_ig, g_fp4.h_ig, sizeof(float), cudaMemcpyHostToDevice, B.stream), "ig") ||
        !cuda_ok(launch_nvfp4_qdq(B.d_x, 1, C, g_fp4.d_ig, g_fp4.d_packed, g_fp4.d_scales, B.d_mid, B.d_status,
                                  B.stream), "qdq") ||
        !cuda_ok(cudaMemcpyAsync(hp, g_fp4.d_packed, (size_t)C / 2, cudaMemcpyDeviceToHost, B.stream), "packed") ||
        !cuda_ok(cudaMemcpyAsync(hp + C, g_fp4.d_scales, (size_t)C / 16, cudaMemcpyDeviceToHost, B.stream), "sc") ||
        !cuda_ok(cudaMemcpyAsync(B.h_x, B.d_mid, (size_t)C * sizeof(float), cudaMemcpyDeviceToHost, B.stream), "dq"))
        return -1;
    count_launches(1);
    if (salt_gpu_sync() != 0) return -1;
    memcpy(packed, hp, (size_t)C / 2);
    memcpy(scales, hp + C, (size_t)C / 16);
    memcpy(dequant, B.h_x, (size_t)C * sizeof(float));
    B.stats.nvfp4_kernel_launches += 1;
    B.stats.nvfp4_completion_fences += 1;
    return 0;
}

int salt_gpu_nvfp4_matvec_batch(const void* key, int R, int C, int Bt, const float* inputs, float* outputs) {
    const Resource* res = nullptr;
    if (!fp4_ready() || !inputs || !outputs || Bt < 1) return -1;
    Tensor* t = fp4_tensor(key, R, C, &res);
    if (!t) {
        if (g_backend.mapped_only) g_backend.stats.mapped_only_misses++;
        return -1;
    }
    std::vector<Tensor*> ts = {t};
    const float* in[1] = {inputs};
    float* out[1] = {outputs};
    return fp4_run(ts, in, out, &Bt, &R, C, 1);
}

int salt_gpu_nvfp4_matvec(const void* key, int R, int C, const float* input, float* output) {
    return salt_gpu_nvfp4_matvec_batch(key, R, C, 1, input, output);
}

int salt_gpu_nvfp4_mixed_batch(const void* const* keys, const float* const* inputs, float* const* outputs,
                               const int* batches, const int* rows, int C, int njobs) {
    if (!fp4_ready() || !keys || !inputs || !outputs || !batches || !rows || njobs < 1 || C < 16 || (C & 15))
        return -1;
    std::vector<Tensor*> ts((size_t)njobs);
    for (int j = 0; j < njobs; j++) {
        const Resource* res = nullptr;
        ts[(size_t)j] = fp4_tensor(keys[j], rows[j], C, &res);
        if (!ts[(size_t)j]) {
            if (g_backend.mapped_only) g_backend.stats.mapped_only_misses++;
            return -1;
        }
    }
    return fp4_run(ts, inputs, outputs, batches, rows, C, njobs);
}

int salt_gpu_nvfp4_batch(const void* const* keys, const float* const* inputs, float* const* outputs,
                         const int* batches, int R, int C, int njobs) {
    if (njobs < 1) return -1;
    std::vector<int> rows((size_t)njobs, R);
    return salt_gpu_nvfp4_mixed_batch(keys, inputs, outputs, batches, rows.data(), C, njobs);
}

}  // extern "C"
