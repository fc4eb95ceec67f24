// BF16 matrix x FP32 vector products, bit-exact against the reference CPU functions:
//   single vector (reference src/kernels.c:139-174, salt_bf16_matvec): eight accumulators, a_j takes
//     the columns c with c % 8 == j in ascending order (product rounded, then added), then
//     y = ((a0 + a2) + (a4 + a6)) + ((a1 + a3) + (a5 + a7)); columns past the last multiple of 8 are
//     added to y one by one;
//   batch (reference models/gemma4-26b-a4b/src/gemma4_vision.c:700-717): per (token, row) one chain
//     sum = fl(sum + fl(w * x)) over the columns in ascending order.
// BF16 -> FP32 is the bit pattern shifted into the top half.
#include "internal.h"

namespace sb {

__device__ __forceinline__ float bf16_at(const uint16_t* w, size_t i) { return __uint_as_float((uint32_t)__ldg(w + i) << 16); }

// Eight lanes per row (lane j = accumulator j), four rows per warp, four warps per block.
__global__ void __launch_bounds__(128)
bf16_matvec8_kernel(const uint16_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int R, int C) {
    const int j = threadIdx.x & 7;
    const int row = blockIdx.x * 16 + (threadIdx.x >> 3);
    const unsigned mask = 0xffu << (threadIdx.x & 24);
    if (row >= R) return;                         // whole groups of eight lanes leave together
    const uint16_t* wr = W + (size_t)row * C;
    const int c8 = C & ~7;
    float acc = 0.0f;
    for (int c = j; c < c8; c += 8) acc = __fadd_rn(acc, __fmul_rn(bf16_at(wr, c), x[c]));
    const int base = (threadIdx.x & 31) & ~7;
    const float a0 = __shfl_sync(mask, acc, base + 0), a1 = __shfl_sync(mask, acc, base + 1);
    const float a2 = __shfl_sync(mask, acc, base + 2), a3 = __shfl_sync(mask, acc, base + 3);
    const float a4 = __shfl_sync(mask, acc, base + 4), a5 = __shfl_sync(mask, acc, base + 5);
    const float a6 = __shfl_sync(mask, acc, base + 6), a7 = __shfl_sync(mask, acc, base + 7);
    if (j == 0) {
        float s = __fadd_rn(__fadd_rn(__fadd_rn(a0, a2), __fadd_rn(a4, a6)), __fadd_rn(__fadd_rn(a1, a3), __fadd_rn(a5, a7)));
        for (int c = c8; c < C; c++) s = __fadd_rn(s, __fmul_rn(bf16_at(wr, c), x[c]));
        y[row] = s;
    }
}

// One thread per (row, token): the serial chain.  The activation row is staged in shared memory.
__global__ void __launch_bounds__(128)
bf16_batch_serial_kernel(const uint16_t* __restrict__ W, const float* __restrict__ xs, float* __restrict__ ys, int R, int C) {
    extern __shared__ __align__(16) float sx[];
    const int tok = blockIdx.y;
    const float* x = xs + (size_t)tok * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) sx[c] = x[c];
    __syncthreads();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= R) return;
    const uint16_t* wr = W + (size_t)row * C;
    float sum = 0.0f;
    for (int c = 0; c < C; c++) sum = __fadd_rn(sum, __fmul_rn(bf16_at(wr, c), sx[c]));
    ys[(size_t)tok * R + row] = sum;
}

cudaError_t launch_bf16_matvec(const uint16_t* W, const float* x, float* y, int R, int C, cudaStream_t stream) {
    if (R < 1 || C < 1) return cudaErrorInvalidValue;
    bf16_matvec8_kernel<<<(R + 15) / 16, 128, 0, stream>>>(W, x, y, R, C);
    return cudaGetLastError();
}

cudaError_t launch_bf16_batch(const uint16_t* W, const float* xs, float* ys, int R, int C, int B, cudaStream_t stream) {
    if (R < 1 || C < 1 || B < 1 || B > 65535) return cudaErrorInvalidValue;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = ensure_dynamic_smem((const void*)bf16_batch_serial_kernel, 200 * 1024);
        if (e != cudaSuccess) return e;
    }
    bf16_batch_serial_kernel<<<dim3((R + 127) / 128, B), 128, smem, stream>>>(W, xs, ys, R, C);
    return cudaGetLastError();
}

}  // namespace sb
