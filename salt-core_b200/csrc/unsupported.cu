// Operator-surface entry points outside the quantized MoE feed-forward path.
// They exist so a reference build links; each fails closed exactly as the
// reference's stub backend does (reference src/gpu_stub.c).
#include "../../include/salt_gpu_b200.h"

extern "C" {

int salt_gpu_attention_batch(int, int, int, int, int, const SaltGpuSharedBuffer*, size_t, const SaltGpuSharedBuffer*,
                             size_t, size_t, int, int, int, int, SaltGpuSharedBuffer*, size_t, SaltGpuSharedBuffer*,
                             size_t, size_t, int) { return -1; }
int salt_gpu_attention_prepare(const SaltGpuSharedBuffer*) { return -1; }
int salt_gpu_attention_bind_kv(size_t, size_t, int) { return -1; }
int salt_gpu_attention_materialize(SaltGpuSharedBuffer*, int, uint64_t*) { return -1; }
int salt_gpu_attention_import(SaltGpuSharedBuffer*, int, uint64_t*) { return -1; }
int salt_gpu_attention_rewind(int) { return -1; }
int salt_gpu_attention_transform(int, int, int, int, int, int, int, int, float, SaltGpuSharedBuffer*, size_t,
                                 SaltGpuSharedBuffer*, size_t, SaltGpuSharedBuffer*, size_t, const float*,
                                 const float*, const float*, const float*, int, SaltGpuSharedBuffer*, size_t,
                                 size_t) { return -1; }

}  // extern "C"
