// Grouped affine-Q4 expert GEMMs on the 5th-generation tensor cores (tcgen05 +
// TMEM) for prefill-sized token groups.  TOLERANCE path: operands are fp16
// (weights dequantised in fp32 as q*s+b, then rounded to fp16; activations
// rounded to fp16), accumulation is fp32 in TMEM.  The bit-exact kernels in
// q4_kernels.cu remain the reference-conformant path.
//
// Two precisions (template SPLIT):
//   single  one MMA per k-step, operands rounded to fp16 once: measured
//           max |err| / max(|ref|, row rms) about 2e-3 (5e-4 of the row maximum)
//   split   every operand is carried as hi + lo fp16 halves (lo = fp16(v - hi)) and
//           each k-step issues Ah*Bh + Al*Bh + Ah*Bl: operand error ~2^-22, three
//           times the tensor work, which the HBM-bound prefill sizes can afford
//
// One block = one 128-row weight tile of one expert group.  Weight rows sit on
// the MMA M dimension (always full), the group's tokens on N (16..128 per pass),
// so small groups waste no tensor rows.  K advances in 64-column chunks = one
// quantisation group per row:
//   all 256 threads  : dequantise 2 x 128 row-chunks (gate, up) Q4 -> fp16 into the
//                      K-major, unswizzled core-matrix layout (8 rows x 16 bytes),
//                      copy the tokens' fp16 activations next to them
//   one thread       : four tcgen05.mma.kind::f16 (M128 x N x K16) per matrix,
//                      then tcgen05.commit on the stage's mbarrier
//   3 stages         : conversion of chunk k+1, k+2 overlaps the MMAs of chunk k
//   epilogue warps   : tcgen05.ld the accumulators, GeGLU (fused gate/up) or plain
//                      store (down)
// Every mbarrier wait is bounded: on expiry the block records an error in the
// status word, skips its remaining work, frees its TMEM and returns.
#include <cuda_fp16.h>

#include "internal.h"
#include "q4_core.cuh"

namespace sb {

constexpr int TC_STAGES = 3;
constexpr int TC_THREADS = 256;
constexpr int TC_KC = 64;                    // K columns per chunk
constexpr int TC_A_BYTES = 128 * TC_KC * 2;  // one matrix' 128 x 64 fp16 tile
constexpr int TC_MAX_NT = 128;
constexpr int TC_B_BYTES = TC_MAX_NT * TC_KC * 2;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Bounded wait for the phase with the given parity.  Returns false on expiry.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// K-major operand without swizzle: core matrices of 8 rows x 16 bytes; LBO = byte
// distance between the two K-adjacent core matrices of one MMA, SBO = distance
// between 8-row groups.  Descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// kind::f16 instruction descriptor: D = F32, A = B = F16, both K-major.
__device__ __forceinline__ uint32_t umma_idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_half2(f32x2 v) {
    float lo, hi;
    unpack2(v, lo, hi);
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ f32x2 half2_to_f32x2(uint32_t h2) {
    float lo, hi;
    asm("{\n\t.reg .f16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}\n"
        : "=f"(lo), "=f"(hi)
        : "r"(h2));
    return pack2(lo, hi);
}

// hi = fp16(v), lo = fp16(v - hi) for a pair
__device__ __forceinline__ void split_half2(f32x2 v, uint32_t& hi, uint32_t& lo) {
    hi = pack_half2(v);
    const f32x2 neg_one = pack2(-1.0f, -1.0f);
    lo = pack_half2(fma2(half2_to_f32x2(hi), neg_one, v));   // v - hi, exact in fp32
}

// 64 consecutive Q4 elements of one row (32 packed bytes) -> 64 fp16 written as
// eight 16-byte core-matrix rows at dst + kcore*128 (and their fp16 residuals at
// dst_lo when SPLIT).  Nibbles become floats by the mask-and-exponent trick.
template <bool SPLIT>
__device__ __forceinline__ void dequant_row_chunk(const NibbleMagic& mg, const uint4& p0, const uint4& p1, float s,
                                                  float b, uint8_t* dst, uint8_t* dst_lo) {
    const uint32_t w[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    const f32x2 ss = pack2(s, s), bb = pack2(b, b);
#pragma unroll
    for (int i = 0; i < 8; i++) {  // word i = columns 8i .. 8i+7 = K core matrix i
        f32x2 q[4];
        nibbles4(w[i] & 0xffffu, mg, q[0], q[1]);
        nibbles4(w[i] >> 16, mg, q[2], q[3]);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const f32x2 d = fma2(q[k], ss, bb);
            if (SPLIT) split_half2(d, hi[k], lo[k]);
            else hi[k] = pack_half2(d);
        }
        *(uint4*)(dst + i * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        if (SPLIT) *(uint4*)(dst_lo + i * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

struct TcArgs {
    const Q4Job* jobs;         // per expert group: weights (A = gate or the only matrix, B = up), R, C, ntok
    const int* njobs_dev;
    const __half* xh;          // [grouped rows][C] fp16 activations, grouped order
    const __half* xl;          // their fp16 residuals (split precision) or null
    const float* y_base;       // base the jobs' y pointers are relative to (to recover the group's first row)
    int y_cols;                // columns of that buffer (inter for gate/up, hidden for down)
    __half* out_h;             // fused: GeGLU output [grouped rows][R] fp16
    __half* out_l;             // its fp16 residual (split precision) or null
    float* out_f;              // plain: projection output [grouped rows][R] fp32
    int* status;
};

template <bool FUSED, bool SPLIT>
__global__ void __launch_bounds__(TC_THREADS, 1) q4_gemm_tc_kernel(TcArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar_free[TC_STAGES];
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ uint32_t s_tmem;

    const int job_id = blockIdx.y;
    if (a.njobs_dev != nullptr && job_id >= *a.njobs_dev) return;
    const Q4Job jb = a.jobs[job_id];
    const int r0 = blockIdx.x * 128;
    if (r0 >= jb.R || jb.ntok < 1) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int C = jb.C, nchunks = C / TC_KC;
    const int g0 = (int)((jb.y - a.y_base) / a.y_cols);     // first grouped row of this expert group
    constexpr int NMAT = FUSED ? 2 : 1;
    constexpr int NPART = SPLIT ? 2 : 1;                     // hi (+ lo) copies of every operand tile
    constexpr int STAGES = (FUSED && SPLIT) ? 2 : TC_STAGES;
    constexpr int A_ALL = NMAT * NPART * TC_A_BYTES;         // A tiles of a stage: [matrix][hi, lo]
    constexpr int STAGE_BYTES = A_ALL + NPART * TC_B_BYTES;
    uint8_t* stage_base = smem;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(&bar_free[s], 1);
        mbar_init(&bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(256u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    // converter role of this thread: (matrix, row) of the A tiles
    const int cm = FUSED ? (tid >> 7) : 0;
    const int crow = tid & 127;
    const bool conv_active = FUSED || tid < 128;
    const int grow = min(r0 + crow, jb.R - 1);
    const uint8_t* cvals = (cm == 0 ? jb.vals : jb.vals2) + (size_t)grow * (C >> 1);
    const uint16_t* csc = (const uint16_t*)(cm == 0 ? jb.scales : jb.scales2) + (size_t)grow * nchunks;
    const uint8_t* cbi_raw = (cm == 0 ? jb.biases : jb.biases2);
    const uint16_t* cbi = cbi_raw ? (const uint16_t*)cbi_raw + (size_t)grow * nchunks : nullptr;
    const uint32_t a_off = (uint32_t)cm * NPART * TC_A_BYTES + (uint32_t)(crow >> 3) * 1024 + (uint32_t)(crow & 7) * 16;

    const NibbleMagic mg = load_nibble_magic();
    uint32_t it = 0;          // running chunk counter across token passes (stage / parity bookkeeping)
    uint32_t done_phase = 0;
    bool failed = false;

    for (int tb = 0; tb < jb.ntok; tb += TC_MAX_NT) {
        const int nt_real = min(TC_MAX_NT, jb.ntok - tb);
        const int NT = (nt_real + 15) & ~15;
        const uint32_t idesc = umma_idesc_f16(128, NT);

        uint4 p0 = make_uint4(0, 0, 0, 0), p1 = p0;
        uint32_t hs = 0, hb = 0;
        if (conv_active) {
            p0 = __ldg((const uint4*)cvals);
            p1 = __ldg((const uint4*)cvals + 1);
            hs = csc[0];
            hb = cbi ? cbi[0] : 0;
        }
        for (int kc = 0; kc < nchunks; kc++, it++) {
            const int s = it % STAGES;
            uint8_t* st = stage_base + s * STAGE_BYTES;
            if (it >= STAGES && !failed) {
                // the MMAs that last read this stage must have completed
                if (!mbar_wait(&bar_free[s], ((it / STAGES) - 1) & 1)) failed = true;
            }
            // current chunk's packed data is in registers; fetch the next chunk's first
            const uint4 c0 = p0, c1 = p1;
            const uint32_t chs = hs, chb = hb;
            if (conv_active && kc + 1 < nchunks) {
                p0 = __ldg((const uint4*)(cvals + (kc + 1) * 32));
                p1 = __ldg((const uint4*)(cvals + (kc + 1) * 32) + 1);
                hs = csc[kc + 1];
                hb = cbi ? cbi[kc + 1] : 0;
            }
            // B tile: NT token rows x 64 fp16 of this chunk -> core-matrix layout
            {
                uint8_t* sb_ = st + A_ALL;
                for (int p = tid; p < NT * 8; p += TC_THREADS) {
                    const int n = p >> 3, kcore = p & 7;
                    const int tok = min(tb + n, jb.ntok - 1);
                    const size_t src = (size_t)(g0 + tok) * C + kc * TC_KC;
                    const uint32_t off = (n >> 3) * 1024 + kcore * 128 + (n & 7) * 16;
                    *(uint4*)(sb_ + off) = __ldg((const uint4*)(a.xh + src) + kcore);
                    if (SPLIT) *(uint4*)(sb_ + TC_B_BYTES + off) = __ldg((const uint4*)(a.xl + src) + kcore);
                }
            }
            if (conv_active)
                dequant_row_chunk<SPLIT>(mg, c0, c1, bf16_bits_to_f32(chs), bf16_bits_to_f32(chb), st + a_off,
                                         st + a_off + TC_A_BYTES);
            // make the generic-proxy writes visible to the tensor core (async proxy)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if (tid == 0 && !failed) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = smem_u32(st);
                const uint32_t sbh = sa + A_ALL, sbl = sbh + TC_B_BYTES;
#pragma unroll
                for (int j = 0; j < TC_KC / 16; j++) {
                    const uint64_t bh = umma_desc(sbh + j * 256, 128, 1024);
                    const uint64_t bl = umma_desc(sbl + j * 256, 128, 1024);
                    const uint32_t acc = (kc > 0 || j > 0) ? 1u : 0u;
#pragma unroll
                    for (int m = 0; m < NMAT; m++) {
                        const uint32_t ah = sa + m * NPART * TC_A_BYTES + j * 256;
                        const uint32_t d = tmem + m * 128;
                        umma_f16(d, umma_desc(ah, 128, 1024), bh, idesc, acc);
                        if (SPLIT) {
                            umma_f16(d, umma_desc(ah + TC_A_BYTES, 128, 1024), bh, idesc, 1u);   // A_lo * B_hi
                            umma_f16(d, umma_desc(ah, 128, 1024), bl, idesc, 1u);                // A_hi * B_lo
                        }
                    }
                }
                umma_commit(&bar_free[s]);
                if (kc == nchunks - 1) umma_commit(&bar_done);
            }
        }
        // ---- epilogue of this token pass ----
        if (!failed && !mbar_wait(&bar_done, done_phase & 1)) failed = true;
        done_phase++;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (warp < 4 && !failed) {
            const int m = r0 + warp * 32 + lane;
            const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
            for (int n0 = 0; n0 < NT; n0 += 32) {
                uint32_t g[32];
                tmem_ld32(trow + n0, g);
                if (FUSED) {
                    uint32_t u[32];
                    tmem_ld32(trow + 128 + n0, u);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int n = n0 + i;
                        if (n < nt_real && m < jb.R) {
                            const float gv = __uint_as_float(g[i]), uv = __uint_as_float(u[i]);
                            const float inner = 0.7978845608028654f * (gv + 0.044715f * gv * gv * gv);
                            const float act = 0.5f * gv * (1.0f + tanhf(inner));
                            const float o = act * uv;
                            const __half oh = __float2half_rn(o);
                            a.out_h[(size_t)(g0 + tb + n) * jb.R + m] = oh;
                            if (SPLIT) a.out_l[(size_t)(g0 + tb + n) * jb.R + m] = __float2half_rn(o - __half2float(oh));
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int n = n0 + i;
                        if (n < nt_real && m < jb.R) a.out_f[(size_t)(g0 + tb + n) * jb.R + m] = __uint_as_float(g[i]);
                    }
                }
            }
        }
        // all accumulator reads of this pass precede the next pass' first MMA
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    }
    if (failed && a.status) atomicOr(a.status, SB_ERR_TIMEOUT);
    // wait (bounded) for any MMAs still in flight before releasing TMEM and shared memory
    if (tid == 0 && it > 0) {
        const uint32_t last = it - 1;
        (void)mbar_wait(&bar_free[last % STAGES], (last / STAGES) & 1);
    }
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

// x (fp32, token rows) -> fp16 rows in grouped order: xh[g] = fp16(x[g2c[g] / topk]),
// and (when xl != null) the residuals xl[g] = fp16(x - xh).
__global__ void __launch_bounds__(256)
gather_convert_kernel(const float* __restrict__ x, const int32_t* __restrict__ g2c, __half* __restrict__ xh,
                      __half* __restrict__ xl, int topk, int hidden) {
    const int g = blockIdx.y;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (d >= hidden) return;
    const float4 v = *(const float4*)(x + (size_t)(g2c[g] / topk) * hidden + d);
    const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
    __half2* o = (__half2*)(xh + (size_t)g * hidden + d);
    o[0] = h0;
    o[1] = h1;
    if (xl) {
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        __half2* l = (__half2*)(xl + (size_t)g * hidden + d);
        l[0] = __floats2half2_rn(v.x - f0.x, v.y - f0.y);
        l[1] = __floats2half2_rn(v.z - f1.x, v.w - f1.y);
    }
}

cudaError_t launch_gather_convert(const float* x, const int32_t* g2c, void* xh, void* xl, int jobs, int topk,
                                  int hidden, cudaStream_t stream) {
    if (jobs < 1) return cudaSuccess;
    dim3 grid((hidden / 4 + 255) / 256, jobs);
    gather_convert_kernel<<<grid, 256, 0, stream>>>(x, g2c, (__half*)xh, (__half*)xl, topk, hidden);
    return cudaGetLastError();
}

template <bool FUSED, bool SPLIT>
static cudaError_t launch_tc(const TcArgs& a, dim3 grid, cudaStream_t stream) {
    constexpr int NMAT = FUSED ? 2 : 1, NPART = SPLIT ? 2 : 1;
    constexpr int STAGES = (FUSED && SPLIT) ? 2 : TC_STAGES;
    // at least 116 KB of dynamic shared memory keeps one block per SM, so a block's 256 TMEM
    // columns can always be allocated without waiting for a neighbour
    size_t smem = (size_t)STAGES * (NMAT * NPART * TC_A_BYTES + NPART * TC_B_BYTES) + 1024;
    if (smem < 120 * 1024) smem = 120 * 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(q4_gemm_tc_kernel<FUSED, SPLIT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    q4_gemm_tc_kernel<FUSED, SPLIT><<<grid, TC_THREADS, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_q4_gemm_tc(bool fused, bool split, const Q4Job* jobs, int njobs_max, const int* njobs_dev,
                              const void* xh, const void* xl, const float* y_base, int y_cols, void* out_h,
                              void* out_l, float* out_f, int R, int* status, cudaStream_t stream) {
    if (njobs_max < 1) return cudaSuccess;
    TcArgs a;
    a.jobs = jobs; a.njobs_dev = njobs_dev; a.xh = (const __half*)xh; a.xl = (const __half*)xl;
    a.y_base = y_base; a.y_cols = y_cols;
    a.out_h = (__half*)out_h; a.out_l = (__half*)out_l; a.out_f = out_f; a.status = status;
    dim3 grid((R + 127) / 128, njobs_max);
    if (fused) return split ? launch_tc<true, true>(a, grid, stream) : launch_tc<true, false>(a, grid, stream);
    return split ? launch_tc<false, true>(a, grid, stream) : launch_tc<false, false>(a, grid, stream);
}

}  // namespace sb
