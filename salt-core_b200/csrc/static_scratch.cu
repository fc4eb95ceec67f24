// An expert chain (gate/up + GeGLU, then down) for callers that must not
// allocate device memory.
//
// Some embedders of this library run under a fixed device-memory budget that is
// handed out once at start-up (an engine whose allocator owns all of HBM, a
// plugin loaded into a process where cudaMalloc after initialisation is
// forbidden or would fragment a pre-sized pool, a latency-critical loop that
// cannot afford the device-wide synchronisation an allocation implies).  The
// other entry points of this library keep their intermediate buffers in memory
// obtained from cudaMalloc; this one keeps them in a fixed array that is part of
// the library image itself, so calling it never changes the amount of device
// memory in use.
//
// The price: the array is sized at build time (SB_STATIC_CHAIN_FLOATS), every
// GPU that loads the library carries it until the process exits, and all calls
// on a device share it.
#include <cuda_runtime.h>
#include <stdio.h>

#include "../../include/salt_gpu_b200.h"
#include "backend_state.h"
#include "internal.h"
#include "q4_core.cuh"

namespace sb {

// Layout of the static scratch: two job descriptors, then the GeGLU output
// ("chain") rows that the down projection consumes.
constexpr size_t SB_STATIC_HEADER_BYTES = 512;
constexpr size_t SB_STATIC_CHAIN_FLOATS = 65536;   // 256 KiB: e.g. 93 tokens at inter = 704
constexpr size_t SB_STATIC_BYTES = SB_STATIC_HEADER_BYTES + SB_STATIC_CHAIN_FLOATS * sizeof(float);

static __device__ __align__(256) unsigned char g_static_scratch[SB_STATIC_BYTES];

// In host code the name g_static_scratch is only a handle; the address a kernel
// can use has to be asked for, per device.
constexpr int SB_MAX_DEVICES = 64;
static unsigned char* g_static_ptr[SB_MAX_DEVICES];

static unsigned char* static_scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= SB_MAX_DEVICES) return nullptr;
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) {
            fprintf(stderr, "salt_b200_q4_expert_chain_static: cudaGetSymbolAddress failed: %s\n",
                    cudaGetErrorString(e));
            return nullptr;
        }
        g_static_ptr[dev] = (unsigned char*)p;
    }
    return g_static_ptr[dev];
}

// Descriptors travel as kernel arguments and are stored by the device, which
// may name the array directly.
__global__ void static_write_jobs(Q4Job gate_up, Q4Job down) {
    Q4Job* jobs = (Q4Job*)g_static_scratch;
    if (threadIdx.x == 0) {
        jobs[0] = gate_up;
        jobs[1] = down;
    }
}

}  // namespace sb

using namespace sb;

extern "C" int salt_b200_q4_expert_chain_static(const void* d_gate_vals, const void* d_gate_scales,
                                                const void* d_gate_biases, const void* d_up_vals,
                                                const void* d_up_scales, const void* d_up_biases,
                                                const void* d_down_vals, const void* d_down_scales,
                                                const void* d_down_biases, int hidden, int inter,
                                                const float* d_x, int ntok, float* d_y, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!d_gate_vals || !d_gate_scales || !d_gate_biases || !d_up_vals || !d_up_scales || !d_up_biases ||
        !d_down_vals || !d_down_scales || !d_down_biases || !d_x || !d_y || hidden < 64 || inter < 64 ||
        (hidden % 64) || (inter % 64) || ntok < 1) {
        fprintf(stderr, "salt_b200_q4_expert_chain_static: invalid argument (null pointer, or hidden/inter not a "
                        "positive multiple of 64, or ntok < 1)\n");
        return -1;
    }
    const size_t need = (size_t)ntok * (size_t)inter;
    if (need > SB_STATIC_CHAIN_FLOATS) {
        fprintf(stderr, "salt_b200_q4_expert_chain_static: ntok*inter = %zu floats exceeds the static scratch "
                        "capacity of %zu floats; split the tokens over several calls\n",
                need, (size_t)SB_STATIC_CHAIN_FLOATS);
        return -1;
    }
    const uintptr_t all = (uintptr_t)d_gate_vals | (uintptr_t)d_gate_scales | (uintptr_t)d_gate_biases |
                          (uintptr_t)d_up_vals | (uintptr_t)d_up_scales | (uintptr_t)d_up_biases |
                          (uintptr_t)d_down_vals | (uintptr_t)d_down_scales | (uintptr_t)d_down_biases |
                          (uintptr_t)d_x | (uintptr_t)d_y;
    if (all & 15) {
        fprintf(stderr, "salt_b200_q4_expert_chain_static: every device pointer must be 16-byte aligned\n");
        return -1;
    }
    unsigned char* scratch = static_scratch_for_current_device();
    if (!scratch) return -1;
    Q4Job* jobs = (Q4Job*)scratch;
    float* chain = (float*)(scratch + SB_STATIC_HEADER_BYTES);

    Q4Job gu = {};
    gu.vals = (const uint8_t*)d_gate_vals; gu.scales = (const uint8_t*)d_gate_scales;
    gu.biases = (const uint8_t*)d_gate_biases;
    gu.vals2 = (const uint8_t*)d_up_vals; gu.scales2 = (const uint8_t*)d_up_scales;
    gu.biases2 = (const uint8_t*)d_up_biases;
    gu.x = d_x; gu.y = chain; gu.x_rows = nullptr; gu.x_div = 1;
    gu.R = inter; gu.C = hidden; gu.ntok = ntok; gu.x_stride = hidden; gu.y_stride = inter;
    Q4Job dn = {};
    dn.vals = (const uint8_t*)d_down_vals; dn.scales = (const uint8_t*)d_down_scales;
    dn.biases = (const uint8_t*)d_down_biases;
    dn.x = chain; dn.y = d_y; dn.x_rows = nullptr; dn.x_div = 1;
    dn.R = hidden; dn.C = inter; dn.ntok = ntok; dn.x_stride = inter; dn.y_stride = hidden;

    // Nothing in the scratch has to start at zero: both descriptors and every
    // chain row that the down projection reads are written earlier in this call.
    static_write_jobs<<<1, 32, 0, st>>>(gu, dn);
    if (!cuda_ok(cudaGetLastError(), "static descriptors") ||
        !cuda_ok(launch_q4_jobs(jobs, 1, nullptr, inter, ntok, hidden, 2, true, st), "static gate/up") ||
        !cuda_ok(launch_q4_jobs(jobs + 1, 1, nullptr, hidden, ntok, inter, 1, true, st), "static down"))
        return -1;
    count_launches(3);
    return 0;
}
