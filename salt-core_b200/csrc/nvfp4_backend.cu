// NVFP4 entry points of the operator surface (placeholder until the NVFP4
// kernels land: they fail closed).
#include "../../include/salt_gpu_b200.h"

extern "C" {
int salt_gpu_nvfp4_resource_slot(uint32_t, uint32_t, const void*, const uint8_t*, const uint8_t*, const float*,
                                 const float*, int, int) { return -1; }
int salt_gpu_nvfp4_qdq(const float*, int, float, uint8_t*, uint8_t*, float*) { return -1; }
int salt_gpu_nvfp4_matvec(const void*, int, int, const float*, float*) { return -1; }
int salt_gpu_nvfp4_matvec_batch(const void*, int, int, int, const float*, float*) { return -1; }
int salt_gpu_nvfp4_batch(const void* const*, const float* const*, float* const*, const int*, int, int, int) { return -1; }
int salt_gpu_nvfp4_mixed_batch(const void* const*, const float* const*, float* const*, const int*, const int*, int,
                               int) { return -1; }
}
