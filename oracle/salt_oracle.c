/* salt_oracle.c -- CPU restatement of the reference algorithms on the
 * quantized MoE feed-forward path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, imports or
 * calls this file; it exists so the CUDA kernels can be compared bit for bit
 * against an independent statement of the same arithmetic.  Only tests/, the
 * smoke check and the CPU-baseline legs of bench.py may load it.
 *
 * Parity status: PINNED.  Every function here is checked (tests/test_oracle_*.py)
 * against the known-answer vectors the reference's own tests hold
 * (tests/test_kernels.c tests 5, 12-16; tests/test_nvfp4.c:28-118;
 * tests/test_text_verify.c:1234-1312) and against outputs of the reference
 * sources themselves compiled into oracle/_ref/libsalt_ref.so, committed as
 * fixtures under tests/golden/.
 *
 * Build with -ffp-contract=off: the whole point is that no multiply is ever
 * fused into an add.  Row ownership is the only thing threads partition; the
 * order of operations inside a row never depends on the thread count.
 *
 * Each function cites the reference file:line whose behaviour it restates.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#include <pthread.h>
#include <stdlib.h>

#define ORC_GROUP 64

/* Minimal static-partition parallel for: thread t owns indices
 * [t*n/T, (t+1)*n/T).  Ownership only; per-index work is order independent. */
typedef void (*orc_range_fn)(void *ctx, int begin, int end);
typedef struct { orc_range_fn fn; void *ctx; int begin, end; } OrcSpan;

static void *orc_span_main(void *arg) {
    OrcSpan *s = (OrcSpan *)arg;
    s->fn(s->ctx, s->begin, s->end);
    return NULL;
}

static void orc_parallel_for(int n, int threads, orc_range_fn fn, void *ctx) {
    pthread_t tid[256];
    OrcSpan span[256];
    unsigned char started[256];
    if (threads > 256) threads = 256;
    if (threads > n) threads = n;
    if (threads <= 1) { fn(ctx, 0, n); return; }
    for (int t = 0; t < threads; t++) {
        span[t].fn = fn; span[t].ctx = ctx;
        span[t].begin = (int)((long long)n * t / threads);
        span[t].end = (int)((long long)n * (t + 1) / threads);
        started[t] = pthread_create(&tid[t], NULL, orc_span_main, &span[t]) == 0;
        if (!started[t]) fn(ctx, span[t].begin, span[t].end);
    }
    for (int t = 0; t < threads; t++)
        if (started[t]) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------ */
/* deterministic scalar math (reference src/bitmath.c)                 */
/* ------------------------------------------------------------------ */

/* src/bitmath.c:43-64: n = round(x*log2e) in double, r = x - n*ln2 in
 * double, degree-8 Horner in float on (float)r, result scaled by 2^n. */
float orc_expf(float x) {
    static const double LOG2E =
        1.442695040888963407359924681001892137426645954152985934135449406931;
    static const double LN2 =
        0.693147180559945309417232121458176568075500134360255254120680009;
    static const float coeff[9] = {
        2.48015873015873e-05f, 1.98412698412698e-04f, 1.38888888888889e-03f,
        8.33333333333333e-03f, 4.16666666666667e-02f, 1.66666666666667e-01f,
        5.0e-01f, 1.0f, 1.0f
    };
    double n, r;
    float rf, p;
    if (x != x) return x;
    if (x > 88.722839f) return 3.402823466e+38f;
    if (x < -87.336548f) return 0.0f;
    n = round((double)x * LOG2E);
    r = (double)x - n * LN2;
    rf = (float)r;
    p = coeff[0];
    for (int i = 1; i < 9; i++) {
        float t = p * rf;
        p = t + coeff[i];
    }
    return ldexpf(p, (int)n);
}

/* src/bitmath.c:102-116: fast-inverse-sqrt seed refined by six Newton
 * steps in double. */
static double orc_invsqrt64(float x) {
    uint32_t bits;
    float seed;
    double y, xd = (double)x;
    memcpy(&bits, &x, 4);
    bits = UINT32_C(0x5f3759df) - (bits >> 1);
    memcpy(&seed, &bits, 4);
    y = (double)seed;
    for (int i = 0; i < 6; i++) {
        double yy = y * y;
        double half_x_yy = 0.5 * xd * yy;   /* (0.5*xd)*yy, left to right */
        double corr = 1.5 - half_x_yy;
        y = y * corr;
    }
    return y;
}

/* src/bitmath.c:118-126 */
float orc_rsqrtf(float x) {
    if (x != x) return x;
    if (x < 0.0f) return NAN;
    if (x == 0.0f) return INFINITY;
    if (x == 1.0f) return 1.0f;
    if (x < 0x1p-126f) return orc_rsqrtf(x * 0x1p24f) * 0x1p12f;
    return (float)orc_invsqrt64(x);
}

/* src/bitmath.c:128-135 */
float orc_sqrtf(float x) {
    if (x != x) return x;
    if (x < 0.0f) return NAN;
    if (x == 0.0f || x == 1.0f) return x;
    if (x < 0x1p-126f) return orc_sqrtf(x * 0x1p24f) * 0x1p-12f;
    return (float)((double)x * orc_invsqrt64(x));
}

/* src/bitmath.c:137-147: tanh via exp(2|x|), saturating at |x| >= 10. */
float orc_tanhf(float x) {
    float m, e, r;
    if (x != x) return x;
    if (x >= 10.0f) return 1.0f;
    if (x <= -10.0f) return -1.0f;
    m = x < 0.0f ? -x : x;
    e = orc_expf(2.0f * m);
    r = (e - 1.0f) / (e + 1.0f);
    return x < 0.0f ? -r : r;
}

/* models/gemma4-26b-a4b/src/gemma4.c:80-83: tanh-GELU, evaluated strictly
 * left to right: ((0.044715*x)*x)*x, x + cubic, k*inner, (0.5*x)*(1+t). */
float orc_gelu_tanh(float x) {
    const float k = 0.7978845608028654f;
    float cubic = 0.044715f * x;
    float inner, t, half;
    cubic = cubic * x;
    cubic = cubic * x;
    inner = x + cubic;
    inner = k * inner;
    t = orc_tanhf(inner);
    half = 0.5f * x;
    t = 1.0f + t;
    return half * t;
}

/* src/bitmath.c:95-100 (salt_powf) restricted to y = -0.5, the only exponent
 * this path uses: 1 -> 1, positive -> rsqrt, anything else is returned as is. */
static float orc_pow_neg_half(float x) {
    if (x == 1.0f) return 1.0f;
    if (x > 0.0f) return orc_rsqrtf(x);
    return x;
}

/* ------------------------------------------------------------------ */
/* affine Q4, group 64 (reference include/salt/kernels.h:117-130)      */
/* ------------------------------------------------------------------ */

static float orc_bf16(const void *base, size_t index) {
    uint16_t h;
    uint32_t bits;
    float f;
    memcpy(&h, (const unsigned char *)base + index * 2, 2);
    bits = (uint32_t)h << 16;
    memcpy(&f, &bits, 4);
    return f;
}

static uint32_t orc_u32(const void *base, size_t index) {
    uint32_t v;
    memcpy(&v, (const unsigned char *)base + index * 4, 4);
    return v;
}

/* src/kernels.c:181-205: element k = (vals[k>>3] >> 4(k&7)) & 15, group k/64,
 * value = q*scale + bias, no implicit offset. */
void orc_q4_decode(const void *vals, const void *scales, const void *biases,
                   size_t n, float *out) {
    for (size_t k = 0; k < n; k++) {
        size_t g = k / ORC_GROUP;
        uint32_t q = (orc_u32(vals, k >> 3) >> (4u * (unsigned)(k & 7u))) & 15u;
        float s = orc_bf16(scales, g);
        float b = biases ? orc_bf16(biases, g) : 0.0f;
        float d = (float)q * s;
        out[k] = d + b;
    }
}

/* The row DAG, src/kernels.c:220-250.  32 accumulators, accumulator c&31
 * receives columns in ascending order: d = fl(q*s), d = fl(d+b),
 * p = fl(d*x[c]), acc = fl(acc+p).  Fold: L_j = sum over a of acc[4a+j]
 * starting from 0, then (L0+L2)+(L1+L3).  Group index is absolute
 * (row*C + c)/64, so rows may straddle groups when C % 64 != 0. */
static float orc_q4_row_general(const void *vals, const void *scales,
                                const void *biases, int C, const float *x,
                                size_t r) {
    float acc[32];
    float lane[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int j = 0; j < 32; j++) acc[j] = 0.0f;
    for (int c = 0; c < C; c++) {
        size_t k = r * (size_t)C + (size_t)c;
        size_t g = k / ORC_GROUP;
        uint32_t q = (orc_u32(vals, k >> 3) >> (4u * (unsigned)(k & 7u))) & 15u;
        float s = orc_bf16(scales, g);
        float b = biases ? orc_bf16(biases, g) : 0.0f;
        float d = (float)q * s;
        float p;
        d = d + b;
        p = d * x[c];
        acc[c & 31] = acc[c & 31] + p;
    }
    for (int a = 0; a < 8; a++)
        for (int j = 0; j < 4; j++) lane[j] = lane[j] + acc[4 * a + j];
    {
        float t0 = lane[0] + lane[2];
        float t1 = lane[1] + lane[3];
        return t0 + t1;
    }
}

/* Same DAG, restructured for C % 64 == 0 so the compiler can vectorise the
 * 32 independent accumulator lanes (no reassociation is involved: lane j of
 * a block only ever touches acc[j]). */
static float orc_q4_row_blocked(const uint8_t *vals, const void *scales,
                                const void *biases, int C, const float *x,
                                size_t r) {
    float acc[32];
    float lane[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint8_t *row = vals + r * (size_t)(C / 2);
    size_t g0 = r * (size_t)(C / ORC_GROUP);
    for (int j = 0; j < 32; j++) acc[j] = 0.0f;
    for (int blk = 0; blk < C / 32; blk++) {
        float s = orc_bf16(scales, g0 + (size_t)(blk >> 1));
        float b = biases ? orc_bf16(biases, g0 + (size_t)(blk >> 1)) : 0.0f;
        const uint8_t *bytes = row + (size_t)blk * 16;
        const float *xb = x + (size_t)blk * 32;
        float q[32];
        for (int i = 0; i < 16; i++) {
            q[2 * i] = (float)(bytes[i] & 15u);
            q[2 * i + 1] = (float)(bytes[i] >> 4);
        }
        for (int j = 0; j < 32; j++) {
            float d = q[j] * s;
            float p;
            d = d + b;
            p = d * xb[j];
            acc[j] = acc[j] + p;
        }
    }
    for (int a = 0; a < 8; a++)
        for (int j = 0; j < 4; j++) lane[j] = lane[j] + acc[4 * a + j];
    {
        float t0 = lane[0] + lane[2];
        float t1 = lane[1] + lane[3];
        return t0 + t1;
    }
}

static float orc_q4_row(const void *vals, const void *scales,
                        const void *biases, int C, const float *x, size_t r) {
    if (C % ORC_GROUP == 0)
        return orc_q4_row_blocked((const uint8_t *)vals, scales, biases, C, x, r);
    return orc_q4_row_general(vals, scales, biases, C, x, r);
}

/* src/kernels.c:283-335 (salt_q4_matvec): y[r] = row DAG.  Threads own rows. */
typedef struct {
    const void *vals, *scales, *biases;
    int R, C, B;
    const float *xs;
    float *ys;
} OrcQ4Job;

static void orc_q4_span(void *ctx, int begin, int end) {
    const OrcQ4Job *j = (const OrcQ4Job *)ctx;
    for (int i = begin; i < end; i++) {
        int b = i / j->R, r = i % j->R;
        j->ys[i] = orc_q4_row(j->vals, j->scales, j->biases, j->C,
                              j->xs + (size_t)b * j->C, (size_t)r);
    }
}

int orc_q4_matvec(const void *vals, const void *scales, const void *biases,
                  int R, int C, const float *x, float *y, int threads) {
    OrcQ4Job job = {vals, scales, biases, R, C, 1, x, y};
    if (!vals || !scales || !x || !y || R < 1 || C < 1) return -1;
    orc_parallel_for(R, threads, orc_q4_span, &job);
    return 0;
}

/* src/kernels.c:1355-1497 (salt_q4_matvec_batch): Y[b][r], bit-identical per
 * (row, token) to the single-vector form. */
int orc_q4_matvec_batch(const void *vals, const void *scales,
                        const void *biases, int R, int C, int B,
                        const float *xs, float *ys, int threads) {
    OrcQ4Job job = {vals, scales, biases, R, C, B, xs, ys};
    if (!vals || !scales || !xs || !ys || R < 1 || C < 1 || B < 1) return -1;
    orc_parallel_for(R * B, threads, orc_q4_span, &job);
    return 0;
}

/* ------------------------------------------------------------------ */
/* router (reference gemma4.c:46-186, src/kernels.c:98-106)            */
/* ------------------------------------------------------------------ */

/* models/gemma4-26b-a4b/src/gemma4.c:46-101 (salt_gemma4_rmsnorm):
 * serial sum of squares, inv = rsqrt(ss/n + eps) through the pow(-0.5)
 * shortcut (src/bitmath.c:95-100), y = (x*inv)*w. */
int orc_rmsnorm(float *out, const float *x, const float *weight, int n,
                float eps, int with_scale) {
    float ss = 0.0f, inv, mean;
    if (!out || !x || n < 1 || (with_scale && !weight)) return -1;
    for (int i = 0; i < n; i++) {
        float sq;
        if (!isfinite(x[i]) || (with_scale && !isfinite(weight[i]))) return -1;
        sq = x[i] * x[i];
        ss = ss + sq;
    }
    mean = ss / (float)n;
    mean = mean + eps;
    inv = orc_pow_neg_half(mean);
    if (!isfinite(inv)) return -1;
    for (int i = 0; i < n; i++) {
        float y = x[i] * inv;
        if (with_scale) y = y * weight[i];
        if (!isfinite(y)) return -1;
        out[i] = y;
    }
    return 0;
}

/* gemma4.c:103-130 (salt_gemma4_router_input):
 * out = ((x*inv)*scale)*(1/sqrt(H)). */
int orc_router_input(float *out, const float *x, const float *scale, int H,
                     float eps) {
    float ss = 0.0f, inv, mean, root;
    if (!out || !x || !scale || H < 1) return -1;
    for (int i = 0; i < H; i++) {
        float sq;
        if (!isfinite(x[i]) || !isfinite(scale[i])) return -1;
        sq = x[i] * x[i];
        ss = ss + sq;
    }
    mean = ss / (float)H;
    mean = mean + eps;
    inv = orc_pow_neg_half(mean);
    root = 1.0f / orc_sqrtf((float)H);
    if (!isfinite(inv) || !isfinite(root)) return -1;
    for (int i = 0; i < H; i++) {
        float y = x[i] * inv;
        y = y * scale[i];
        y = y * root;
        if (!isfinite(y)) return -1;
        out[i] = y;
    }
    return 0;
}

/* src/kernels.c:343-369 (salt_q8_matvec): affine 8-bit, one byte per element, bf16 scale and
 * bias per 64 consecutive elements of the flattened matrix (a row may straddle groups).
 * One serial chain per row: acc = fl(acc + fl(d * x[c])), d = fl(fl(q*s) + b), q = 0..255. */
void orc_q8_matvec(const void *vals, const void *scales, const void *biases, int R, int C,
                   const float *x, float *y) {
    const unsigned char *b8 = (const unsigned char *)vals;
    for (int r = 0; r < R; r++) {
        float acc = 0.0f;
        for (int c = 0; c < C; c++) {
            size_t k = (size_t)r * (size_t)C + (size_t)c;
            size_t g = k >> 6;
            float s = orc_bf16(scales, g);
            float b = biases ? orc_bf16(biases, g) : 0.0f;
            float d = (float)b8[k] * s;
            float p;
            d = d + b;
            p = d * x[c];
            acc = acc + p;
        }
        y[r] = acc;
    }
}

/* src/kernels.c:139-174 (salt_bf16_matvec): eight accumulators, a_j takes the columns c with c % 8 == j
 * (product rounded, then added); y = ((a0+a2)+(a4+a6)) + ((a1+a3)+(a5+a7)), then the columns past the
 * last multiple of 8 one by one, then the optional bias. */
void orc_bf16_matvec(const void *W, int R, int C, const float *x, const float *bias, float *y) {
    for (int r = 0; r < R; r++) {
        float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        size_t base = (size_t)r * (size_t)C;
        int c = 0;
        float s, e, o;
        for (; c + 7 < C; c += 8)
            for (int j = 0; j < 8; j++) {
                float t = orc_bf16(W, base + (size_t)(c + j)) * x[c + j];
                a[j] = a[j] + t;
            }
        e = (a[0] + a[2]) + (a[4] + a[6]);
        o = (a[1] + a[3]) + (a[5] + a[7]);
        s = e + o;
        for (; c < C; c++) {
            float t = orc_bf16(W, base + (size_t)c) * x[c];
            s = s + t;
        }
        y[r] = s + (bias ? bias[r] : 0.0f);
    }
}

/* models/gemma4-26b-a4b/src/gemma4_vision.c:700-717 (the portable loop behind salt_gpu_bf16_matvec_batch,
 * the same chain as salt_f32_matvec, src/kernels.c:98-116, on the widened weights): per (token, row)
 * sum = fl(sum + fl(w * x[c])), c ascending. */
void orc_bf16_matvec_serial(const void *W, int R, int C, int B, const float *xs, float *ys) {
    for (int t = 0; t < B; t++)
        for (int r = 0; r < R; r++) {
            float sum = 0.0f;
            size_t base = (size_t)r * (size_t)C;
            for (int c = 0; c < C; c++) {
                float p = orc_bf16(W, base + (size_t)c) * xs[(size_t)t * C + c];
                sum = sum + p;
            }
            ys[(size_t)t * R + r] = sum;
        }
}

/* gemma4.c:188-213 (salt_gemma4_residual_postnorm): the branch is RMS-normalised with its
 * post-norm weight, then added to the residual: out = residual + (branch*inv)*w.
 * Non-finite inputs or outputs reject the whole call. */
int orc_residual_postnorm(float *out, const float *residual, const float *branch,
                          const float *weight, int n, float eps) {
    float ss = 0.0f, inv, mean;
    if (!out || !residual || !branch || !weight || n < 1) return -1;
    for (int i = 0; i < n; i++)
        if (!isfinite(residual[i])) return -1;
    for (int i = 0; i < n; i++) {
        float sq;
        if (!isfinite(branch[i]) || !isfinite(weight[i])) return -1;
        sq = branch[i] * branch[i];
        ss = ss + sq;
    }
    mean = ss / (float)n;
    mean = mean + eps;
    inv = orc_pow_neg_half(mean);
    if (!isfinite(inv)) return -1;
    for (int i = 0; i < n; i++) {
        float y = branch[i] * inv;
        y = y * weight[i];
        if (!isfinite(y)) return -1;
        y = residual[i] + y;
        if (!isfinite(y)) return -1;
    }
    for (int i = 0; i < n; i++) {
        float y = branch[i] * inv;
        y = y * weight[i];
        out[i] = residual[i] + y;
    }
    return 0;
}

/* gemma4.c:215-276 (salt_gemma4_parallel_ffn_combine): the consumer of the routed-expert
 * output.  sum = RMSNorm(dense, wd) + RMSNorm(routed, wr); final = RMSNorm(sum, wf);
 * out = (residual + final) * layer_scalar.  scratch_2n receives sum | final as the reference
 * leaves them. */
int orc_parallel_ffn_combine(float *out, const float *residual, const float *dense,
                             const float *routed, const float *dense_w, const float *routed_w,
                             const float *final_w, float layer_scalar, int n, float eps,
                             float *scratch_2n) {
    float *sum, *fin;
    if (!out || !residual || !dense || !routed || !dense_w || !routed_w || !final_w ||
        !scratch_2n || n < 1 || !isfinite(layer_scalar))
        return -1;
    for (int i = 0; i < n; i++)
        if (!isfinite(residual[i])) return -1;
    sum = scratch_2n;
    fin = scratch_2n + n;
    if (orc_rmsnorm(sum, dense, dense_w, n, eps, 1) != 0 ||
        orc_rmsnorm(fin, routed, routed_w, n, eps, 1) != 0)
        return -1;
    for (int i = 0; i < n; i++) {
        float c = sum[i] + fin[i];
        if (!isfinite(c)) return -1;
        sum[i] = c;
    }
    if (orc_rmsnorm(fin, sum, final_w, n, eps, 1) != 0) return -1;
    for (int i = 0; i < n; i++) {
        float y = residual[i] + fin[i];
        y = y * layer_scalar;
        if (!isfinite(y)) return -1;
    }
    for (int i = 0; i < n; i++) {
        float y = residual[i] + fin[i];
        out[i] = y * layer_scalar;
    }
    return 0;
}

/* gemma4.c:278-286 (salt_gemma4_softcap): logits = cap * tanh(logits / cap), in place. */
int orc_softcap(float *logits, int n, float cap) {
    if (!logits || n < 1 || !(cap > 0.0f) || !isfinite(cap)) return -1;
    for (int i = 0; i < n; i++)
        if (!isfinite(logits[i])) return -1;
    for (int i = 0; i < n; i++) {
        float q = logits[i] / cap;
        logits[i] = cap * orc_tanhf(q);
    }
    return 0;
}

/* src/kernels.c:98-106 (salt_router_scores): one serial chain per expert,
 * acc = fl(acc + fl(W[e][c]*x[c])), then + bias[e] (0 when absent). */
void orc_router_scores(const float *W, const float *bias, int E, int H,
                       const float *x, float *scores) {
    for (int e = 0; e < E; e++) {
        const float *w = W + (size_t)e * H;
        float acc = 0.0f;
        for (int c = 0; c < H; c++) {
            float p = w[c] * x[c];
            acc = acc + p;
        }
        scores[e] = acc + (bias ? bias[e] : 0.0f);
    }
}

/* gemma4.c:132-186 (salt_gemma4_router_topk) followed by the adapter's
 * ascending-expert sort (gemma4_text.c:8541-8550; src/text_verify_cpu.c:
 * 1256-1265).  Insertion top-k with strict '>' (ties keep the lower expert
 * index ahead), softmax denominators over ALL experts in ascending order,
 * renormalisation over the selected ranks in rank order, then the per-expert
 * scale.  sort_by_expert != 0 applies the final (selected, weight) sort. */
int orc_router_topk(const float *logits, const float *per_expert_scale, int E,
                    int topk, int32_t *selected, float *weights,
                    int sort_by_expert) {
    float mx = -INFINITY, all = 0.0f, sel = 0.0f;
    if (!logits || !selected || !weights || E < 1 || topk < 1 || topk > E)
        return -1;
    for (int e = 0; e < E; e++) {
        if (!isfinite(logits[e]) ||
            (per_expert_scale && !isfinite(per_expert_scale[e])))
            return -1;
        if (logits[e] > mx) mx = logits[e];
    }
    for (int j = 0; j < topk; j++) { selected[j] = -1; weights[j] = -INFINITY; }
    for (int e = 0; e < E; e++) {
        float s = logits[e];
        int j = topk - 1;
        while (j >= 0 && (selected[j] < 0 || s > weights[j])) j--;
        if (j < topk - 1) {
            for (int q = topk - 2; q > j; q--) {
                selected[q + 1] = selected[q];
                weights[q + 1] = weights[q];
            }
            selected[j + 1] = e;
            weights[j + 1] = s;
        }
    }
    for (int e = 0; e < E; e++) all = all + orc_expf(logits[e] - mx);
    if (!(all > 0.0f) || !isfinite(all)) return -1;
    for (int j = 0; j < topk; j++) {
        weights[j] = orc_expf(weights[j] - mx) / all;
        sel = sel + weights[j];
    }
    if (!(sel > 0.0f) || !isfinite(sel)) return -1;
    for (int j = 0; j < topk; j++) {
        float n = weights[j] / sel;
        weights[j] = n * (per_expert_scale ? per_expert_scale[selected[j]] : 1.0f);
    }
    if (sort_by_expert)
        for (int a = 0; a < topk; a++)
            for (int b = a + 1; b < topk; b++)
                if (selected[b] < selected[a]) {
                    int32_t id = selected[a];
                    float w = weights[a];
                    selected[a] = selected[b]; weights[a] = weights[b];
                    selected[b] = id; weights[b] = w;
                }
    return 0;
}

/* ------------------------------------------------------------------ */
/* grouping and reduction (reference src/tensorops.c:239-325)          */
/* ------------------------------------------------------------------ */

/* src/tensorops.c:239-289 (salt_tensor_selected_route_group): stable counting
 * sort of the rows*topk selections by expert.  expert_offsets ends holding the
 * END of each expert's range (the reference advances it while scattering). */
int orc_route_group(const int32_t *selected, uint32_t rows, uint32_t topk,
                    uint32_t n_experts, const float *row_inputs,
                    uint32_t hidden, uint32_t *expert_offsets,
                    int32_t *grouped_to_canonical,
                    int32_t *canonical_to_grouped, float *routed_inputs) {
    uint32_t jobs = rows * topk, next = 0;
    if (!selected || !expert_offsets || !grouped_to_canonical ||
        !canonical_to_grouped || rows == 0 || topk == 0 || n_experts == 0 ||
        topk > n_experts)
        return -1;
    for (uint32_t i = 0; i < jobs; i++)
        if (selected[i] < 0 || (uint32_t)selected[i] >= n_experts) return -1;
    memset(expert_offsets, 0, (size_t)n_experts * sizeof *expert_offsets);
    for (uint32_t i = 0; i < jobs; i++) expert_offsets[selected[i]]++;
    for (uint32_t e = 0; e < n_experts; e++) {
        uint32_t pop = expert_offsets[e];
        expert_offsets[e] = next;
        next += pop;
    }
    for (uint32_t i = 0; i < jobs; i++) {
        uint32_t g = expert_offsets[selected[i]]++;
        grouped_to_canonical[g] = (int32_t)i;
    }
    for (uint32_t g = 0; g < jobs; g++) {
        uint32_t canonical = (uint32_t)grouped_to_canonical[g];
        canonical_to_grouped[canonical] = (int32_t)g;
        if (routed_inputs && row_inputs)
            memcpy(routed_inputs + (size_t)g * hidden,
                   row_inputs + (size_t)(canonical / topk) * hidden,
                   (size_t)hidden * sizeof(float));
    }
    return 0;
}

/* src/tensorops.c:291-325 (salt_tensor_selected_weighted_reduce), identical
 * in order to src/moe_group.c:211-224: out = 0; for rank ascending:
 * out = fl(out + fl(w * o)). */
int orc_weighted_reduce(const float *weights,
                        const int32_t *canonical_to_grouped,
                        const float *grouped_outputs, uint32_t rows,
                        uint32_t topk, uint32_t width, float *outputs) {
    if (!weights || !canonical_to_grouped || !grouped_outputs || !outputs)
        return -1;
    for (uint32_t i = 0; i < rows * topk; i++)
        if (canonical_to_grouped[i] < 0 ||
            (uint32_t)canonical_to_grouped[i] >= rows * topk ||
            !isfinite(weights[i]))
            return -1;
    for (uint32_t row = 0; row < rows; row++) {
        float *out = outputs + (size_t)row * width;
        for (uint32_t d = 0; d < width; d++) out[d] = 0.0f;
        for (uint32_t rank = 0; rank < topk; rank++) {
            uint32_t canonical = row * topk + rank;
            const float *o = grouped_outputs +
                (size_t)canonical_to_grouped[canonical] * width;
            float w = weights[canonical];
            for (uint32_t d = 0; d < width; d++) {
                float p = w * o[d];
                out[d] = out[d] + p;
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* one MoE feed-forward layer, affine Q4 (the chain of reference call   */
/* stack gemma4_text.c:8344-8363 / 7908-8064 and moe_group.c:9-235)    */
/* ------------------------------------------------------------------ */

/* Expert weights live in one pool: expert e starts at pool + e*expert_stride
 * and holds gate | up | down, each as values | scales | biases
 * (tools/gemma4-mlx4-source.py:180-199 slot order). */
typedef struct {
    int hidden, inter, n_experts, topk;
    float eps;
    const float *router_w;          /* [E][H] fp32 */
    const float *router_scale;      /* [H] */
    const float *per_expert_scale;  /* [E] */
    const uint8_t *pool;
    size_t expert_stride;
} OrcMoeLayer;

static void orc_expert_tensors(const OrcMoeLayer *L, int e, int which,
                               const uint8_t **v, const uint8_t **s,
                               const uint8_t **b) {
    size_t elems = (size_t)L->hidden * (size_t)L->inter;
    size_t vb = elems / 2, gb = elems / ORC_GROUP * 2;
    const uint8_t *base = L->pool + (size_t)e * L->expert_stride +
                          (size_t)which * (vb + 2 * gb);
    *v = base; *s = base + vb; *b = base + vb + gb;
}

/* x [B][H] -> y [B][H]; optional taps: selected [B][k], weights [B][k].
 * Per token: router input, logits, top-k (sorted by expert), then for each
 * selection in ascending-expert order: gate, up, GeGLU, down; y = ordered
 * weighted sum starting from 0.  Threads partition (selection, row) pairs. */
typedef struct {
    const OrcMoeLayer *L;
    const float *x;
    int B;
    int32_t *sel;
    float *w, *chain, *down, *y;
    int rc;
} OrcMoeRun;

static void orc_moe_route_span(void *ctx, int begin, int end) {
    OrcMoeRun *run = (OrcMoeRun *)ctx;
    const OrcMoeLayer *L = run->L;
    float *rin = (float *)malloc(sizeof(float) * (size_t)(L->hidden + L->n_experts));
    float *logits = rin + L->hidden;
    for (int t = begin; t < end; t++) {
        if (!rin || orc_router_input(rin, run->x + (size_t)t * L->hidden,
                                     L->router_scale, L->hidden, L->eps) != 0) {
            run->rc = -1;
            continue;
        }
        orc_router_scores(L->router_w, NULL, L->n_experts, L->hidden, rin, logits);
        if (orc_router_topk(logits, L->per_expert_scale, L->n_experts, L->topk,
                            run->sel + (size_t)t * L->topk,
                            run->w + (size_t)t * L->topk, 1) != 0)
            run->rc = -1;
    }
    free(rin);
}

static void orc_moe_gateup_span(void *ctx, int begin, int end) {
    OrcMoeRun *run = (OrcMoeRun *)ctx;
    const OrcMoeLayer *L = run->L;
    for (int i = begin; i < end; i++) {
        int job = i / L->inter, r = i % L->inter;
        const float *xt = run->x + (size_t)(job / L->topk) * L->hidden;
        const uint8_t *v, *s, *b;
        float g, u;
        orc_expert_tensors(L, run->sel[job], 0, &v, &s, &b);
        g = orc_q4_row(v, s, b, L->hidden, xt, (size_t)r);
        orc_expert_tensors(L, run->sel[job], 1, &v, &s, &b);
        u = orc_q4_row(v, s, b, L->hidden, xt, (size_t)r);
        run->chain[i] = orc_gelu_tanh(g) * u;
    }
}

static void orc_moe_down_span(void *ctx, int begin, int end) {
    OrcMoeRun *run = (OrcMoeRun *)ctx;
    const OrcMoeLayer *L = run->L;
    for (int i = begin; i < end; i++) {
        int job = i / L->hidden, r = i % L->hidden;
        const uint8_t *v, *s, *b;
        orc_expert_tensors(L, run->sel[job], 2, &v, &s, &b);
        run->down[i] = orc_q4_row(v, s, b, L->inter,
                                  run->chain + (size_t)job * L->inter, (size_t)r);
    }
}

static void orc_moe_reduce_span(void *ctx, int begin, int end) {
    OrcMoeRun *run = (OrcMoeRun *)ctx;
    const OrcMoeLayer *L = run->L;
    for (int t = begin; t < end; t++) {
        float *yt = run->y + (size_t)t * L->hidden;
        for (int d = 0; d < L->hidden; d++) yt[d] = 0.0f;
        for (int j = 0; j < L->topk; j++) {
            const float *o = run->down + ((size_t)t * L->topk + j) * L->hidden;
            float w = run->w[(size_t)t * L->topk + j];
            for (int d = 0; d < L->hidden; d++) {
                float p = o[d] * w;
                yt[d] = yt[d] + p;
            }
        }
    }
}

int orc_moe_layer_q4(const OrcMoeLayer *L, const float *x, int B, float *y,
                     int32_t *selected_out, float *weights_out, int threads) {
    OrcMoeRun run;
    size_t jobs;
    if (!L || !x || !y || B < 1 || L->topk < 1 || L->topk > L->n_experts)
        return -1;
    jobs = (size_t)B * (size_t)L->topk;
    run.L = L; run.x = x; run.B = B; run.y = y; run.rc = 0;
    run.sel = (int32_t *)malloc(jobs * sizeof(int32_t));
    run.w = (float *)malloc(jobs * sizeof(float));
    run.chain = (float *)malloc(jobs * (size_t)L->inter * sizeof(float));
    run.down = (float *)malloc(jobs * (size_t)L->hidden * sizeof(float));
    if (!run.sel || !run.w || !run.chain || !run.down) run.rc = -1;
    if (run.rc == 0) orc_parallel_for(B, threads, orc_moe_route_span, &run);
    if (run.rc == 0) {
        orc_parallel_for((int)(jobs * (size_t)L->inter), threads, orc_moe_gateup_span, &run);
        orc_parallel_for((int)(jobs * (size_t)L->hidden), threads, orc_moe_down_span, &run);
        orc_parallel_for(B, threads, orc_moe_reduce_span, &run);
        if (selected_out) memcpy(selected_out, run.sel, jobs * sizeof(int32_t));
        if (weights_out) memcpy(weights_out, run.w, jobs * sizeof(float));
    }
    free(run.sel); free(run.w); free(run.chain); free(run.down);
    return run.rc;
}

/* ------------------------------------------------------------------ */
/* NVFP4 (reference src/nvfp4.c)                                       */
/* ------------------------------------------------------------------ */

static const float orc_e2m1_pos[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* src/nvfp4.c:19-23: sign-magnitude codebook; both zero codes give +0. */
float orc_e2m1(uint8_t code) {
    float v = orc_e2m1_pos[code & 7u];
    if (v == 0.0f) return 0.0f;
    return (code & 8u) ? -v : v;
}

/* src/nvfp4.c:25-39: E4M3FN, subnormals m*2^-9, 0x7f/0xff NaN, max 448. */
float orc_e4m3fn(uint8_t code) {
    int sign = code >> 7, ex = (code >> 3) & 15, man = code & 7;
    float v;
    if (ex == 0) v = (float)man * 0.001953125f;
    else if (ex == 15 && man == 7) return NAN;
    else v = (1.0f + (float)man * 0.125f) * ldexpf(1.0f, ex - 7);
    return sign ? -v : v;
}

/* src/nvfp4.c:41-63: nearest of the 127 finite magnitudes, saturating at 448;
 * on an exact tie the even code wins (a later candidate replaces the current
 * best only if strictly closer, or equally close, even, and the best is odd). */
int orc_e4m3fn_encode(float value, uint8_t *code) {
    uint8_t best = 0;
    float best_d = 3.402823466e+38f, mag;
    if (!code || isnan(value)) return -1;
    mag = fabsf(value);
    if (mag > 448.0f) mag = 448.0f;
    for (unsigned cand = 0; cand <= 0x7eu; cand++) {
        float d = fabsf(mag - orc_e4m3fn((uint8_t)cand));
        if (d < best_d || (d == best_d && !(cand & 1u) && (best & 1u))) {
            best_d = d;
            best = (uint8_t)cand;
        }
    }
    *code = (uint8_t)(best | (signbit(value) ? 0x80u : 0u));
    return 0;
}

/* src/nvfp4.c:65-80 */
static uint8_t orc_e2m1_encode(float value) {
    float mag = fabsf(value), best_d = 3.402823466e+38f;
    uint8_t best = 0;
    for (unsigned cand = 0; cand < 8u; cand++) {
        float d = fabsf(mag - orc_e2m1_pos[cand]);
        if (d < best_d || (d == best_d && !(cand & 1u) && (best & 1u))) {
            best_d = d;
            best = (uint8_t)cand;
        }
    }
    if (signbit(value)) best |= 8u;
    return best;
}

/* src/nvfp4.c:82-130 (salt_nvfp4_quantize_input_reference): per 16 inputs,
 * amax -> fl(amax*(1/6)) -> fl(ig*that) clamp 448 -> e4m3 code; codes from
 * fl(x * fl(ig/scale)) clamped to +-6; dequant = e2m1 * fl(scale/ig).
 * Low nibble holds the even element. */
int orc_nvfp4_qdq(const float *input, int C, float input_global_scale,
                  uint8_t *packed, uint8_t *scales, float *dequant) {
    if (!input || !packed || !scales || !dequant || C < 16 || (C & 15) ||
        !isfinite(input_global_scale) || input_global_scale <= 0.0f)
        return -1;
    for (int blk = 0; blk < C / 16; blk++) {
        const float *in = input + blk * 16;
        float amax = 0.0f, raw, scale, out_scale, dq_scale;
        uint8_t sc;
        for (int i = 0; i < 16; i++) {
            float m = fabsf(in[i]);
            if (!isfinite(m)) return -1;
            if (m > amax) amax = m;
        }
        raw = amax * (1.0f / 6.0f);
        raw = input_global_scale * raw;
        if (raw > 448.0f) raw = 448.0f;
        if (orc_e4m3fn_encode(raw, &sc) != 0) return -1;
        scales[blk] = sc;
        scale = orc_e4m3fn(sc);
        out_scale = scale == 0.0f ? 0.0f : input_global_scale / scale;
        dq_scale = scale / input_global_scale;
        for (int i = 0; i < 16; i += 2) {
            float a = in[i] * out_scale, b = in[i + 1] * out_scale;
            uint8_t ca, cb;
            if (a > 6.0f) a = 6.0f;
            if (a < -6.0f) a = -6.0f;
            if (b > 6.0f) b = 6.0f;
            if (b < -6.0f) b = -6.0f;
            ca = orc_e2m1_encode(a);
            cb = orc_e2m1_encode(b);
            packed[(blk * 16 + i) / 2] = (uint8_t)(ca | (uint8_t)(cb << 4));
            dequant[blk * 16 + i] = orc_e2m1(ca) * dq_scale;
            dequant[blk * 16 + i + 1] = orc_e2m1(cb) * dq_scale;
        }
    }
    return 0;
}

/* src/nvfp4.c:132-155 */
int orc_nvfp4_dequant_weights(const uint8_t *packed, const uint8_t *scales,
                              float weight_divisor, int R, int C, float *out) {
    float wg;
    if (!packed || !scales || !out || R < 1 || C < 16 || (C & 15) ||
        !isfinite(weight_divisor) || weight_divisor == 0.0f)
        return -1;
    wg = 1.0f / weight_divisor;
    for (size_t k = 0; k < (size_t)R * (size_t)C; k++) {
        uint8_t byte = packed[k >> 1];
        uint8_t code = (k & 1u) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 15u);
        float sc = orc_e4m3fn(scales[k / 16]) * wg;
        out[k] = orc_e2m1(code) * sc;
    }
    return 0;
}

typedef struct {
    const uint8_t *packed, *scales;
    float wg;
    int C;
    const float *xdq;
    float *out;
} OrcFp4Job;

static void orc_nvfp4_span(void *ctx, int begin, int end) {
    const OrcFp4Job *job = (const OrcFp4Job *)ctx;
    int C = job->C;
    for (int r = begin; r < end; r++) {
        float acc[32], lane[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int j = 0; j < 32; j++) acc[j] = 0.0f;
        for (int c = 0; c < C; c++) {
            size_t k = (size_t)r * (size_t)C + (size_t)c;
            uint8_t byte = job->packed[k >> 1];
            uint8_t code = (k & 1u) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 15u);
            float sc = orc_e4m3fn(job->scales[(size_t)r * (size_t)(C / 16) + (size_t)(c / 16)]);
            float w, p;
            sc = sc * job->wg;
            w = orc_e2m1(code) * sc;
            p = w * job->xdq[c];
            acc[c & 31] = acc[c & 31] + p;
        }
        for (int a = 0; a < 8; a++)
            for (int j = 0; j < 4; j++) lane[j] = lane[j] + acc[4 * a + j];
        {
            float t0 = lane[0] + lane[2];
            float t1 = lane[1] + lane[3];
            job->out[r] = t0 + t1;
        }
    }
}

/* src/nvfp4.c:157-192 row + fold, :228-256 driver: W4A4 -- activations go
 * through the group-16 Q/DQ first; w = e2m1 * fl(e4m3(scale) * (1/divisor));
 * p = fl(w * xdq[c]); acc[c&31] += p; same fold as the Q4 row. */
int orc_nvfp4_matvec(const uint8_t *packed, const uint8_t *scales,
                     float weight_divisor, float input_global_scale, int R,
                     int C, const float *input, float *output,
                     uint8_t *x_packed, uint8_t *x_scales, float *x_dequant,
                     int threads) {
    float wg;
    if (!packed || !scales || !input || !output || !x_packed || !x_scales ||
        !x_dequant || R < 1 || C < 16 || (C & 15) ||
        !isfinite(weight_divisor) || weight_divisor == 0.0f)
        return -1;
    wg = 1.0f / weight_divisor;
    if (orc_nvfp4_qdq(input, C, input_global_scale, x_packed, x_scales, x_dequant))
        return -1;
    {
        OrcFp4Job job = {packed, scales, wg, C, x_dequant, output};
        orc_parallel_for(R, threads, orc_nvfp4_span, &job);
    }
    return 0;
}
