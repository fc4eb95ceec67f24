// Decode-sized expert execution in ONE launch: gate | up -> GeGLU -> down for every selected
// expert of a layer, bit-exact against the reference row DAG (src/kernels.c:220-250, GeGLU
// models/gemma4-26b-a4b/src/gemma4.c:80-83).
//
// One persistent block per SM, SLOTS row slots of 16 lanes each.  The selected experts are
// processed in rounds of up to `jobs_per_round` jobs.  Inside a round the jobs' gate/up row
// pairs form one index space [0, J*M) and their down rows another [0, J*H); block i owns the
// contiguous share [i*P, (i+1)*P) of the first and [i*Q, (i+1)*Q) of the second, so every SM
// streams the same number of bytes whatever the number of experts.
//
//   * every packed weight row is one cp.async.bulk copy (global -> shared, tracked by an
//     mbarrier with a transaction count) into a padded row of shared memory; a warp issues
//     the copies of its own rows, and the copies of BOTH phases are issued before the first
//     product is formed: the down rows are in flight while gate/up computes;
//   * the bf16 scales and biases of a warp's rows are fetched with plain loads and interleaved
//     into one word per quantisation group;
//   * the GeGLU values go through global memory (a few KB that stay in L2): a block adds the
//     number of row pairs it finished to a per-job arrival counter (release), and a block
//     whose down rows need that job polls the counter (acquire, bounded), then reads the
//     values through L2;
//   * all blocks must be resident at the same time (grid <= number of SMs, one block per SM):
//     a block never waits before its own gate/up share is done, so residency is the only
//     condition for progress.  Every wait is bounded; on expiry the block records
//     SB_ERR_TIMEOUT in the status word and carries on, so the launch always ends.
#include "internal.h"
#include "mbar.cuh"
#include "pdl.cuh"
#include "q4_core.cuh"

namespace sb {

constexpr uint32_t FUSED_SPIN_LIMIT = 1u << 21;   // polls of a counter or of an mbarrier (a fraction of a second)

// Stride of a packed row in shared memory: the smallest multiple of 16 bytes for which the two
// rows a warp reads at the same byte index (`apart` rows from each other: adjacent slots hold
// adjacent gate or up rows, but every second down row) start at least four banks apart.
static __host__ __device__ __forceinline__ int fused_row_stride(int row_bytes, int apart) {
    int s = row_bytes;
    while (((s * apart) & 127) < 16 || ((s * apart) & 127) > 112) s += 16;
    return s;
}

struct FusedGeom {
    int gu_rb, gu_stride, gu_gpr;     // gate/up: row bytes, padded stride, groups per row
    int dn_rb, dn_stride, dn_gpr;
    int dn_cap;                       // down rows held per block
    size_t off_dn, off_tgu, off_tdn, off_x, off_chain, off_jobs, off_bars, total;
};

static __host__ __device__ __forceinline__ FusedGeom fused_geom(int H, int M, int tt, int slots) {
    FusedGeom g;
    g.gu_rb = H >> 1; g.gu_stride = fused_row_stride(g.gu_rb, 1); g.gu_gpr = H >> 6;
    g.dn_rb = M >> 1; g.dn_stride = fused_row_stride(g.dn_rb, 2); g.dn_gpr = M >> 6;
    g.dn_cap = 4 * slots;
    size_t o = (size_t)2 * slots * g.gu_stride;
    g.off_dn = o;    o += (size_t)g.dn_cap * g.dn_stride;
    g.off_tgu = o;   o += (size_t)2 * slots * g.gu_gpr * 4;
    g.off_tdn = o;   o += (size_t)g.dn_cap * g.dn_gpr * 4;
    o = (o + 15) & ~(size_t)15;
    g.off_x = o;     o += (size_t)tt * H * 4;
    g.off_chain = o; o += (size_t)2 * tt * M * 4;
    g.off_jobs = o;  o += (size_t)FUSED_MAX_JOBS * sizeof(FusedJob);
    g.off_bars = o;  o += (size_t)(slots + 2) * 8;       // slots/2 gate/up + slots/2 down barriers, one for x
    g.total = o;
    return g;
}

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Bounded wait for the phase with the given parity; false on expiry.
__device__ __forceinline__ bool fused_mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < FUSED_SPIN_LIMIT; i++) {
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

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// (scale bf16 << 16) | bias bf16 for the groups of `nrows` rows owned by one warp.
// row r of the warp: packed scales at srcs[r], biases at srcb[r] (null: bias 0), table row at dst[r].
// Returns (in every lane) whether any scale needs the literal two-rounding dequantisation.
template <int NROWS>
__device__ __forceinline__ bool fused_build_table(const uint8_t* const (&srcs)[NROWS], const uint8_t* const (&srcb)[NROWS],
                                                  uint32_t* const (&dst)[NROWS], int gpr, int lane) {
    int lit = 0;
#pragma unroll
    for (int r = 0; r < NROWS; r++) {
        if (srcs[r] == nullptr) continue;
        for (int g = lane; g < gpr; g += 32) {
            const uint32_t hs = __ldg((const uint16_t*)srcs[r] + g);
            const uint32_t hb = srcb[r] ? (uint32_t)__ldg((const uint16_t*)srcb[r] + g) : 0u;
            dst[r][g] = (hs << 16) | hb;
            lit |= scale_needs_literal(hs) ? 1 : 0;
        }
    }
    return __any_sync(0xffffffffu, lit) != 0;
}

// All 32-column steps of one lane's two rows against TT activation rows.
template <int TT, bool LIT>
__device__ __forceinline__ void fused_rows(const NibbleMagic& mg, int steps, const uint8_t* wA, const uint8_t* wB,
                                           const uint32_t* tA, const uint32_t* tB, const float* const (&xrow)[TT],
                                           f32x2 (&accA)[TT], f32x2 (&accB)[TT], f32x2 nz) {
    int st = 0;
    for (; st + 8 <= steps; st += 8) {
        const float* xs[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) xs[tt] = xrow[tt] + st * 32;
        tile16_steps<TT, LIT, 8>(mg, wA + st * 16, wB + st * 16, tA + (st >> 1), tB + (st >> 1), xs, accA, accB, nz);
    }
    for (; st + 2 <= steps; st += 2) {
        const float* xs[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) xs[tt] = xrow[tt] + st * 32;
        tile16_steps<TT, LIT, 2>(mg, wA + st * 16, wB + st * 16, tA + (st >> 1), tB + (st >> 1), xs, accA, accB, nz);
    }
}

// One lane's two rows for the NT tokens of its job (NT <= TT is the job's token count rounded
// up to 1, 2 or 4; surplus tokens repeat the last row and are not stored).
template <int NT>
__device__ __forceinline__ void fused_slot(const NibbleMagic& mg, bool lit, int steps, const uint8_t* wA,
                                           const uint8_t* wB, const uint32_t* tA, const uint32_t* tB,
                                           const float* const (&xrow)[NT], int v, float (&yA)[NT], float (&yB)[NT],
                                           f32x2 nz) {
    // the two row slots of a warp may belong to jobs with different token counts (or one of them
    // may be empty): the fold only involves the slot's own sixteen lanes
    const uint32_t half_mask = 0xffffu << (threadIdx.x & 16);
    f32x2 accA[NT], accB[NT];
#pragma unroll
    for (int tt = 0; tt < NT; tt++) { accA[tt] = pack2(0.0f, 0.0f); accB[tt] = pack2(0.0f, 0.0f); }
    if (lit) fused_rows<NT, true>(mg, steps, wA, wB, tA, tB, xrow, accA, accB, nz);
    else fused_rows<NT, false>(mg, steps, wA, wB, tA, tB, xrow, accA, accB, nz);
#pragma unroll
    for (int tt = 0; tt < NT; tt++) {
        yA[tt] = fold_row_hexadecants(accA[tt], v, half_mask);
        yB[tt] = fold_row_hexadecants(accB[tt], v, half_mask);
    }
}

template <int TT, int SLOTS>
__global__ void __launch_bounds__(16 * SLOTS, 1) q4_fused_expert_kernel(FusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NT = 16 * SLOTS, NW = SLOTS / 2;
    const int H = a.H, M = a.M;
    const FusedGeom G = fused_geom(H, M, TT, SLOTS);
    uint8_t* sGU = smem;                                   // gate rows [0, SLOTS), up rows [SLOTS, 2*SLOTS)
    uint8_t* sDN = smem + G.off_dn;                        // [dn_cap] down rows
    uint32_t* tGU = (uint32_t*)(smem + G.off_tgu);
    uint32_t* tDN = (uint32_t*)(smem + G.off_tdn);
    float* sX = (float*)(smem + G.off_x);                  // [TT][H] the call's activation rows
    float* sC = (float*)(smem + G.off_chain);              // [2 jobs][TT][M] GeGLU rows of the down phase
    FusedJob* sJ = (FusedJob*)(smem + G.off_jobs);
    uint64_t* bar_gu = (uint64_t*)(smem + G.off_bars);     // [NW]
    uint64_t* bar_dn = bar_gu + NW;                        // [NW]
    uint64_t* bar_x = bar_dn + NW;
    __shared__ int s_njobs;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int v = tid & 15, pr = tid >> 4;
    const int cta = blockIdx.x, ncta = gridDim.x;

    if (tid == 0) {
        for (int i = 0; i < 2 * NW + 1; i++) mbar_init(bar_gu + i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_wait();                    // the jobs, the counters and the activations come from the previous kernel
    pdl_launch_dependents();
    {
        // the live count and the whole job table in one round trip (read through L2: another
        // layer's table may still sit in this SM's L1)
        const int n_live = __ldcg(a.n_jobs_dev);
        static_assert(sizeof(FusedJob) % 16 == 0, "job descriptors are copied in 16-byte pieces");
        const int pieces = a.n_jobs_max * (int)(sizeof(FusedJob) / 16);
        for (int i = tid; i < pieces; i += NT) ((uint4*)sJ)[i] = __ldcg((const uint4*)a.jobs + i);
        if (tid == 0) s_njobs = min(max(n_live, 0), a.n_jobs_max);
    }
    __syncthreads();               // barriers initialised, jobs and count in shared memory
    const int n_jobs = s_njobs;
    if (n_jobs == 0) return;
    if (tid == 0) {
        mbar_expect_tx(bar_x, (uint32_t)(a.n_x * H * 4));
        for (int t = 0; t < a.n_x; t++) bulk_g2s(sX + (size_t)t * H, a.x + (size_t)t * a.x_stride, (uint32_t)(H * 4), bar_x);
    }
    const int jpr = a.jobs_per_round;
    const int rounds = (n_jobs + jpr - 1) / jpr;
    const NibbleMagic mg = load_nibble_magic();
    const f32x2 nz = pack2u(c_neg_zero, c_neg_zero);
    uint32_t ph_gu = 0, ph_dn = 0;     // phases of this warp's two barriers
    bool timeout = false;

    // ---- geometry of a round -------------------------------------------------------------
    struct Round { int j0, J, gu_lo, gu_hi, dn_lo, dn_hi; };
    auto round_of = [&](int r) {
        Round R;
        R.j0 = r * jpr;
        R.J = min(jpr, n_jobs - R.j0);
        const int P = (R.J * M + ncta - 1) / ncta;
        int Q = (R.J * H + ncta - 1) / ncta;
        Q += Q & 1;                                   // a lane's two down rows belong to one job
        R.gu_lo = min(cta * P, R.J * M); R.gu_hi = min(R.gu_lo + P, R.J * M);
        R.dn_lo = min(cta * Q, R.J * H); R.dn_hi = min(R.dn_lo + Q, R.J * H);
        return R;
    };
    // slots 2*warp and 2*warp + 1 belong to this warp; lanes 0..3 issue the four gate/up rows
    // (slot, matrix), the table is built by the whole warp
    bool lit_gu = false, lit_dn = false;
    int gu_rows_w = 0, dn_rows_w = 0;                 // rows of this warp in flight / landed
    auto issue_gu = [&](const Round& R) {
        const int s0 = 2 * warp;
        const int nsl = max(0, min(2, R.gu_hi - R.gu_lo - s0));      // valid slots of this warp
        gu_rows_w = 2 * nsl;
        if (nsl == 0) return;
        if (lane == 0) mbar_expect_tx(bar_gu + warp, (uint32_t)(2 * nsl * G.gu_rb));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier reads of these rows precede the copies
        __syncwarp();
        const uint8_t* srcs[4]; const uint8_t* srcb[4]; uint32_t* dst[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int sl = q & 1, mat = q >> 1;
            srcs[q] = nullptr; srcb[q] = nullptr; dst[q] = nullptr;
            if (sl >= nsl) continue;
            const int p = R.gu_lo + s0 + sl;
            const FusedJob& jb = sJ[R.j0 + p / M];
            const int row = p % M;
            const uint8_t* vals = mat ? jb.up_v : jb.gate_v;
            const uint8_t* sc = mat ? jb.up_s : jb.gate_s;
            const uint8_t* bi = mat ? jb.up_b : jb.gate_b;
            const int srow = mat * SLOTS + s0 + sl;
            if (lane == q) bulk_g2s(sGU + (size_t)srow * G.gu_stride, vals + (size_t)row * G.gu_rb, (uint32_t)G.gu_rb, bar_gu + warp);
            srcs[q] = sc + (size_t)row * G.gu_gpr * 2;
            srcb[q] = bi ? bi + (size_t)row * G.gu_gpr * 2 : nullptr;
            dst[q] = tGU + (size_t)srow * G.gu_gpr;
        }
        lit_gu = fused_build_table<4>(srcs, srcb, dst, G.gu_gpr, lane);
        __syncwarp();
    };
    // down: slot s owns rows 2s, 2s + 1 of pass 0 and 2*SLOTS + 2s, + 1 of pass 1 (local indices)
    auto issue_dn = [&](const Round& R) {
        const int n = R.dn_hi - R.dn_lo;
        int cnt = 0;
#pragma unroll
        for (int ps = 0; ps < 2; ps++) cnt += max(0, min(4, n - (ps * 2 * SLOTS + 4 * warp)));
        dn_rows_w = cnt;
        if (cnt == 0) return;
        if (lane == 0) mbar_expect_tx(bar_dn + warp, (uint32_t)(cnt * G.dn_rb));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        const uint8_t* srcs[8]; const uint8_t* srcb[8]; uint32_t* dst[8];
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const int li = (q >> 2) * 2 * SLOTS + 4 * warp + (q & 3);     // local row index
            srcs[q] = nullptr; srcb[q] = nullptr; dst[q] = nullptr;
            if (li >= n) continue;
            const int qg = R.dn_lo + li;
            const FusedJob& jb = sJ[R.j0 + qg / H];
            const int row = qg % H;
            if (lane == q) bulk_g2s(sDN + (size_t)li * G.dn_stride, jb.down_v + (size_t)row * G.dn_rb, (uint32_t)G.dn_rb, bar_dn + warp);
            srcs[q] = jb.down_s + (size_t)row * G.dn_gpr * 2;
            srcb[q] = jb.down_b ? jb.down_b + (size_t)row * G.dn_gpr * 2 : nullptr;
            dst[q] = tDN + (size_t)li * G.dn_gpr;
        }
        lit_dn = fused_build_table<8>(srcs, srcb, dst, G.dn_gpr, lane);
        __syncwarp();
    };

    Round R = round_of(0);
    issue_gu(R);
    issue_dn(R);
    if (!fused_mbar_wait(bar_x, 0)) timeout = true;

    for (int r = 0; r < rounds; r++) {
        // ================= gate | up + GeGLU =================
        if (gu_rows_w > 0) {
            if (!fused_mbar_wait(bar_gu + warp, ph_gu & 1)) timeout = true;
            ph_gu++;
        }
        const int p = R.gu_lo + pr;
        if (p < R.gu_hi) {
            const FusedJob& jb = sJ[R.j0 + p / M];
            const int row = p % M;
            const uint8_t* wA = sGU + (size_t)pr * G.gu_stride + v;
            const uint8_t* wB = sGU + (size_t)(SLOTS + pr) * G.gu_stride + v;
            const uint32_t* tA = tGU + (size_t)pr * G.gu_gpr;
            const uint32_t* tB = tGU + (size_t)(SLOTS + pr) * G.gu_gpr;
            const int ntok = jb.ntok;
            float* crow = a.chain + (size_t)jb.g0 * M + row;
            if (TT >= 4 && ntok >= 3) {
                constexpr int N = TT >= 4 ? 4 : 1;
                const float* xr[N];
                float yA[N], yB[N];
#pragma unroll
                for (int t = 0; t < N; t++) xr[t] = sX + (size_t)jb.x_row[min(t, ntok - 1)] * H + 2 * v;
                fused_slot<N>(mg, lit_gu, H >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz);
                if (v == 0)
#pragma unroll
                    for (int t = 0; t < N; t++)
                        if (t < ntok) crow[(size_t)t * M] = __fmul_rn(gelu_tanh_exact(yA[t]), yB[t]);
            } else if (TT >= 2 && ntok == 2) {
                constexpr int N = TT >= 2 ? 2 : 1;
                const float* xr[N];
                float yA[N], yB[N];
#pragma unroll
                for (int t = 0; t < N; t++) xr[t] = sX + (size_t)jb.x_row[min(t, ntok - 1)] * H + 2 * v;
                fused_slot<N>(mg, lit_gu, H >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz);
                if (v == 0)
#pragma unroll
                    for (int t = 0; t < N; t++) crow[(size_t)t * M] = __fmul_rn(gelu_tanh_exact(yA[t]), yB[t]);
            } else {
                const float* xr[1] = {sX + (size_t)jb.x_row[0] * H + 2 * v};
                float yA[1], yB[1];
                fused_slot<1>(mg, lit_gu, H >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz);
                if (v == 0) crow[0] = __fmul_rn(gelu_tanh_exact(yA[0]), yB[0]);
            }
        }
        __syncwarp();
        Round Rn = R;
        if (r + 1 < rounds) {          // this warp's gate/up rows are free again: next round's copies
            Rn = round_of(r + 1);
            issue_gu(Rn);
        }
        __syncthreads();               // every GeGLU value of this block has been written
        if (tid == 0 && R.gu_hi > R.gu_lo) {
            __threadfence();
            const int ja = R.gu_lo / M, jb2 = (R.gu_hi - 1) / M;
            for (int j = ja; j <= jb2; j++) {
                const int lo = max(R.gu_lo, j * M), hi = min(R.gu_hi, (j + 1) * M);
                atomicAdd(a.done + R.j0 + j, hi - lo);
            }
        }
        // ================= down =================
        const int dn_n = R.dn_hi - R.dn_lo;
        const int dja = dn_n > 0 ? R.dn_lo / H : 0;
        const int djb = dn_n > 0 ? (R.dn_hi - 1) / H : -1;
        if (tid < 2 && dja + tid <= djb) {
            const int* ctr = a.done + R.j0 + dja + tid;
            uint32_t i = 0;
            while (ld_acquire_gpu(ctr) < M && i < FUSED_SPIN_LIMIT) i++;
            if (i >= FUSED_SPIN_LIMIT) timeout = true;
        }
        __syncthreads();
        for (int j = dja; j <= djb; j++) {
            const FusedJob& jb = sJ[R.j0 + j];
            const int n = jb.ntok * M;                      // the job's GeGLU rows are contiguous
            const float* src = a.chain + (size_t)jb.g0 * M;
            float* dstc = sC + (size_t)(j - dja) * TT * M;
            for (int i = tid * 4; i < n; i += NT * 4) *(float4*)(dstc + i) = __ldcg((const float4*)(src + i));
        }
        __syncthreads();
        if (dn_rows_w > 0) {
            if (!fused_mbar_wait(bar_dn + warp, ph_dn & 1)) timeout = true;
            ph_dn++;
        }
#pragma unroll 1
        for (int ps = 0; ps < 2; ps++) {
            const int li = ps * 2 * SLOTS + 2 * pr;
            if (li >= dn_n) continue;
            const int qg = R.dn_lo + li;
            const int jl = qg / H, row = qg % H;
            const FusedJob& jb = sJ[R.j0 + jl];
            const uint8_t* wA = sDN + (size_t)li * G.dn_stride + v;
            const uint8_t* wB = wA + G.dn_stride;
            const uint32_t* tA = tDN + (size_t)li * G.dn_gpr;
            const uint32_t* tB = tA + G.dn_gpr;
            const float* cbase = sC + (size_t)(jl - dja) * TT * M + 2 * v;
            const int ntok = jb.ntok;
            float* orow = a.out + (size_t)jb.g0 * H + row;
            if (TT >= 4 && ntok >= 3) {
                constexpr int N = TT >= 4 ? 4 : 1;
                const float* xr[N];
                float yA[N], yB[N];
#pragma unroll
                for (int t = 0; t < N; t++) xr[t] = cbase + (size_t)min(t, ntok - 1) * M;
                fused_slot<N>(mg, lit_dn, M >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz);
                if (v == 0)
#pragma unroll
                    for (int t = 0; t < N; t++)
                        if (t < ntok) *(float2*)(orow + (size_t)t * H) = make_float2(yA[t], yB[t]);
            } else if (TT >= 2 && ntok == 2) {
                constexpr int N = TT >= 2 ? 2 : 1;
                const float* xr[N];
                float yA[N], yB[N];
#pragma unroll
                for (int t = 0; t < N; t++) xr[t] = cbase + (size_t)t * M;
                fused_slot<N>(mg, lit_dn, M >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz);
                if (v == 0)
#pragma unroll
                    for (int t = 0; t < N; t++) *(float2*)(orow + (size_t)t * H) = make_float2(yA[t], yB[t]);
            } else {
                const float* xr[1] = {cbase};
                float yA[1], yB[1];
                fused_slot<1>(mg, lit_dn, M >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz);
                if (v == 0) *(float2*)orow = make_float2(yA[0], yB[0]);
            }
        }
        __syncwarp();
        if (r + 1 < rounds) issue_dn(Rn);
        R = Rn;
    }
    if (timeout && a.status) atomicOr(a.status, SB_ERR_TIMEOUT);
}

// ---- host side ---------------------------------------------------------------------------
namespace {
struct DeviceInfo { int sms = 0; bool configured[3] = {false, false, false}; };
DeviceInfo g_dev[64];

DeviceInfo* device_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    DeviceInfo* d = &g_dev[dev];
    if (d->sms == 0 && cudaDeviceGetAttribute(&d->sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    return d;
}
constexpr size_t FUSED_SMEM_LIMIT = 227 * 1024;
int fused_tt(int n_x) { return n_x <= 1 ? 1 : (n_x == 2 ? 2 : 4); }
int fused_slots(int tt) { return tt == 1 ? 40 : 32; }
}  // namespace

bool q4_fused_plan(int H, int M, int n_x, int n_jobs_max, FusedLaunch* out) {
    DeviceInfo* d = device_info();
    if (!d || H < 64 || M < 64 || (H & 63) || (M & 63) || n_x < 1 || n_x > 4 || n_jobs_max < 1 ||
        n_jobs_max > FUSED_MAX_JOBS)
        return false;
    const int tt = fused_tt(n_x), slots = fused_slots(tt);
    const FusedGeom g = fused_geom(H, M, tt, slots);
    if (g.total + 64 > FUSED_SMEM_LIMIT) return false;
    const int grid = d->sms;
    // most jobs per round whose shares fit the block: ceil(J*M/grid) <= slots, even ceil(J*H/grid) <= dn_cap
    int jmax = 0;
    for (int J = 1; J <= grid && J <= FUSED_MAX_JOBS; J++) {
        const int P = (J * M + grid - 1) / grid;
        int Q = (J * H + grid - 1) / grid;
        Q += Q & 1;
        if (P > slots || Q > g.dn_cap || P > M || Q > H) break;
        jmax = J;
    }
    if (jmax < 1) return false;
    if (out) { out->grid = grid; out->jobs_per_round = jmax; out->tt = tt; out->smem = g.total; }
    return true;
}

template <int TT, int SLOTS>
static cudaError_t launch_fused_t(FusedArgs& a, const FusedLaunch& L, DeviceInfo* d, int cfg_slot, cudaStream_t stream) {
    if (!d->configured[cfg_slot]) {
        cudaError_t e = cudaFuncSetAttribute(q4_fused_expert_kernel<TT, SLOTS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)FUSED_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        d->configured[cfg_slot] = true;
    }
    return launch_pdl(q4_fused_expert_kernel<TT, SLOTS>, dim3(L.grid), dim3(16 * SLOTS), L.smem, stream, a);
}

cudaError_t launch_q4_fused(const FusedArgs& args, cudaStream_t stream) {
    FusedLaunch L;
    if (!q4_fused_plan(args.H, args.M, args.n_x, args.n_jobs_max, &L)) return cudaErrorInvalidValue;
    if ((((uintptr_t)args.x) & 15) || ((args.x_stride * 4) & 15)) return cudaErrorInvalidValue;
    DeviceInfo* d = device_info();
    FusedArgs a = args;
    a.jobs_per_round = L.jobs_per_round;
    if (L.tt == 1) return launch_fused_t<1, 40>(a, L, d, 0, stream);
    if (L.tt == 2) return launch_fused_t<2, 32>(a, L, d, 1, stream);
    return launch_fused_t<4, 32>(a, L, d, 2, stream);
}

}  // namespace sb
