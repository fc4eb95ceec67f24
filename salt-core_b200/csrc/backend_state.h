// Process-wide state of the salt_gpu_* backend (one calling thread at a time,
// as the reference surface assumes).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <unordered_map>
#include <vector>

#include "../../include/salt_gpu_b200.h"

namespace sb {

struct Q4Job;

// Fixed capacities, allocated once by salt_gpu_init and never grown by an
// operation: 2048 tokens x top-8 rows of 2816 floats per staging buffer.
constexpr size_t SB_STAGE_FLOATS = (size_t)16384 * 2816;
constexpr uint32_t SB_MAX_JOBS = 16384;

struct Resource {
    uint32_t kind = 0, id = 0;
    const uint8_t* host = nullptr;
    size_t nbytes = 0;
    uint8_t* dev = nullptr;
    bool active = false;
    int policy = 0;
    uint64_t window_off = 0, window_bytes = 0;
};

struct Tensor {
    uint32_t kind = 0, id = 0;
    int bits = 0, R = 0, C = 0;      // bits: 4 = affine Q4, 104 = NVFP4
    uint64_t voff = 0, soff = 0, boff = 0, aoff = 0;
    size_t vbytes = 0, gbytes = 0;
    const uint8_t *dv = nullptr, *ds = nullptr, *db = nullptr;  // device views (16-byte aligned)
    float weight_divisor = 0.0f, input_global = 0.0f;           // NVFP4 per-tensor scalars
    std::vector<void*> owned;                                   // private aligned copies
};

struct Selected {
    bool active = false;
    uint64_t logical_id = 0;
    const void* base = nullptr;
    const void* payload = nullptr;
    size_t nbytes = 0;
    uint8_t* dev = nullptr;          // where the payload lives in HBM: `own`, or a residency seat
    uint8_t* own = nullptr;          // allocation of the copying bind, kept for the slot's next occupant
    size_t own_cap = 0;
    bool resident = false;           // bound by salt_gpu_selected_resource_bind_resident
    uint64_t generation = 0;
};

struct Backend {
    bool ready = false;
    int mapped_only = 0, defer = 0;
    std::vector<Resource> resources;
    std::unordered_map<const void*, Tensor> tensors;
    std::unordered_map<const void*, Tensor> arena;
    std::vector<Selected> selected;
    std::vector<int> logical_to_slot;
    bool selected_fenced = false;
    SaltGpuBatchStatsV2 stats = {};
    uint64_t copied_bytes = 0, peak_window = 0;
    cudaStream_t stream = nullptr;
    float *d_x = nullptr, *d_y = nullptr, *d_mid = nullptr;
    float *h_x = nullptr, *h_y = nullptr;
    Q4Job *d_jobs = nullptr, *h_jobs = nullptr;
    int* d_status = nullptr;
    size_t stage_floats = 0, job_cap = 0, x_cursor = 0, job_cursor = 0;
};

extern Backend g_backend;
bool cuda_ok(cudaError_t e, const char* what);
void count_launches(int n);
uint64_t launch_count();
uintptr_t residency_seat_address(int seat, size_t nbytes);
void residency_shutdown();

}  // namespace sb
