// Deterministic scalar math on the device: the same IEEE operation sequence as
// the reference's src/bitmath.c, with every multiply and add an explicit
// round-to-nearest intrinsic so no contraction can occur whatever the build flags.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb {

// p * 2^n, exact where the result is normal (n in [-126, 128] here, see expf).
__device__ __forceinline__ float scale_pow2(float p, int n) {
    if (n > 127) {
        p = __fmul_rn(p, __int_as_float(0x7F000000));  // 2^127
        n -= 127;
    }
    if (n < -126) {  // not reached by expf; kept correct for completeness
        p = __fmul_rn(p, __int_as_float(0x00800000));  // 2^-126
        n += 126;
        if (n < -126) n = -126;
    }
    return __fmul_rn(p, __int_as_float((n + 127) << 23));
}

// src/bitmath.c:43-64.  n = round(x*log2e) and r = x - n*ln2 in double,
// degree-8 Horner in float, result scaled by 2^n (ldexpf).
__device__ __forceinline__ float expf_exact(float x) {
    if (x != x) return x;
    if (x > 88.722839f) return 3.402823466e+38f;
    if (x < -87.336548f) return 0.0f;
    double n = round(__dmul_rn((double)x, 1.442695040888963407359924681001892137));
    double r = __dsub_rn((double)x, __dmul_rn(n, 0.693147180559945309417232121458176568));
    float rf = (float)r;
    float p = 2.48015873015873e-05f;
    p = __fadd_rn(__fmul_rn(p, rf), 1.98412698412698e-04f);
    p = __fadd_rn(__fmul_rn(p, rf), 1.38888888888889e-03f);
    p = __fadd_rn(__fmul_rn(p, rf), 8.33333333333333e-03f);
    p = __fadd_rn(__fmul_rn(p, rf), 4.16666666666667e-02f);
    p = __fadd_rn(__fmul_rn(p, rf), 1.66666666666667e-01f);
    p = __fadd_rn(__fmul_rn(p, rf), 5.0e-01f);
    p = __fadd_rn(__fmul_rn(p, rf), 1.0f);
    p = __fadd_rn(__fmul_rn(p, rf), 1.0f);
    return scale_pow2(p, (int)n);
}

// src/bitmath.c:102-116: bit-trick seed, six Newton steps in double.
__device__ __forceinline__ double invsqrt64(float x) {
    uint32_t bits = 0x5f3759dfu - (__float_as_uint(x) >> 1);
    double y = (double)__uint_as_float(bits);
    double xd = (double)x;
    double half_x = __dmul_rn(0.5, xd);
#pragma unroll
    for (int i = 0; i < 6; i++) {
        double yy = __dmul_rn(y, y);
        double corr = __dsub_rn(1.5, __dmul_rn(half_x, yy));
        y = __dmul_rn(y, corr);
    }
    return y;
}

// src/bitmath.c:118-126
__device__ __forceinline__ float rsqrtf_exact(float x) {
    if (x != x) return x;
    if (x < 0.0f) return __int_as_float(0x7fc00000);
    if (x == 0.0f) return __int_as_float(0x7f800000);
    if (x == 1.0f) return 1.0f;
    if (x < 1.17549435e-38f) {
        float xs = __fmul_rn(x, 16777216.0f);
        float r = (xs == 1.0f) ? 1.0f : (float)invsqrt64(xs);
        return __fmul_rn(r, 4096.0f);
    }
    return (float)invsqrt64(x);
}

// src/bitmath.c:128-135
__device__ __forceinline__ float sqrtf_exact(float x) {
    if (x != x) return x;
    if (x < 0.0f) return __int_as_float(0x7fc00000);
    if (x == 0.0f || x == 1.0f) return x;
    if (x < 1.17549435e-38f) {
        float xs = __fmul_rn(x, 16777216.0f);
        float r = (xs == 1.0f) ? 1.0f : (float)__dmul_rn((double)xs, invsqrt64(xs));
        return __fmul_rn(r, 0.000244140625f);
    }
    return (float)__dmul_rn((double)x, invsqrt64(x));
}

// src/bitmath.c:95-100 restricted to the exponent -0.5 this path uses.
__device__ __forceinline__ float pow_neg_half(float x) {
    if (x == 1.0f) return 1.0f;
    if (x > 0.0f) return rsqrtf_exact(x);
    return x;
}

// src/bitmath.c:137-147
__device__ __forceinline__ float tanhf_exact(float x) {
    if (x != x) return x;
    if (x >= 10.0f) return 1.0f;
    if (x <= -10.0f) return -1.0f;
    float m = x < 0.0f ? -x : x;
    float e = expf_exact(__fmul_rn(2.0f, m));
    float r = __fdiv_rn(__fsub_rn(e, 1.0f), __fadd_rn(e, 1.0f));
    return x < 0.0f ? -r : r;
}

// models/gemma4-26b-a4b/src/gemma4.c:80-83, evaluated left to right.
__device__ __forceinline__ float gelu_tanh_exact(float x) {
    float cubic = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, x), x), x);
    float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(x, cubic));
    float t = tanhf_exact(inner);
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, t));
}

__device__ __forceinline__ bool finite_f(float v) {
    return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u;
}

}  // namespace sb
