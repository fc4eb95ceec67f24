// Decode-sized expert execution in ONE launch: gate | up -> GeGLU -> down for every selected
// expert of a layer, bit-exact against the reference row DAG (src/kernels.c:220-250, GeGLU
// models/gemma4-26b-a4b/src/gemma4.c:80-83).
//
// One persistent block per SM, SLOTS row slots of 16 lanes each (a slot = a gate row and its up
// row, or two adjacent down rows).  The selected experts are
// processed in rounds of up to `jobs_per_round` jobs.  Inside a round the jobs' gate/up row
// pairs form one index space [0, J*M) and their down rows another [0, J*H); block i owns the
// contiguous share [i*P, (i+1)*P) of the first and [i*Q, (i+1)*Q) of the second, so every SM
// streams the same number of bytes whatever the number of experts.
//
//   * every packed gate/up row is one cp.async.bulk copy (global -> shared, tracked by an
//     mbarrier with a transaction count) into a padded row of shared memory, issued by the warp
//     that owns the row; the block's down rows are contiguous and go in one copy; the copies of
//     BOTH phases are issued before the first product is formed, so the down rows are in flight
//     while gate/up computes;
//   * scales and biases are read from a derived copy made when the weights are uploaded: one word
//     (scale bf16 << 16) | bias bf16 per quantisation group, [rows][groups per row] per tensor.  The
//     words of a block's share are contiguous: one more bulk copy per tensor;
//   * the GeGLU values go through global memory (a few KB that stay in L2): a block adds the
//     number of row pairs it finished to a per-job arrival counter (release), and a block
//     whose down rows need that job polls the counter (acquire, bounded), then reads the
//     values through L2;
//   * all blocks must be resident at the same time (grid <= number of SMs, one block per SM):
//     a block never waits before its own gate/up share is done, so residency is the only
//     condition for progress.  Every wait is bounded; on expiry the block records
//     SB_ERR_TIMEOUT in the status word and carries on, so the launch always ends.
// The kernel runs once per layer between other kernels, so its instructions are fetched cold
// every time: set-up code is written as short per-lane code instead of unrolled per-row code,
// and the rarely needed two-rounding dequantisation lives in a function that is not inlined.
#include "internal.h"
#include "mbar.cuh"
#include "pdl.cuh"
#include "q4_core.cuh"
#include "router_core.cuh"

namespace sb {

constexpr int FUSED_GU_CHUNKS = 2;                // pieces in which a packed gate/up row is requested
constexpr uint32_t FUSED_SPIN_LIMIT = 1u << 21;   // polls of a counter or of an mbarrier (a fraction of a second)

// Stride of a packed gate/up row in shared memory: the smallest multiple of 16 bytes for which the
// rows of two adjacent slots, read by one warp at the same byte index, start at least four banks apart.
static __host__ __device__ __forceinline__ int fused_row_stride(int row_bytes) {
    int s = row_bytes;
    while ((s & 127) < 16 || (s & 127) > 112) s += 16;
    return s;
}

struct FusedGeom {
    int gu_rb, gu_stride, gu_gpr;     // gate/up: row bytes, padded stride, groups per row
    int dn_rb, dn_stride, dn_gpr;
    int dn_cap;                       // down rows held per block
    int gu_sc_cap, dn_sc_cap;         // bytes of one staged scale | bias table (gate, up; down)
    size_t off_dn, off_sgu, off_sdn, off_x, off_chain, off_jobs, off_bars, total;
};

static __host__ __device__ __forceinline__ FusedGeom fused_geom(int H, int M, int tt, int slots) {
    FusedGeom g;
    g.gu_rb = H >> 1; g.gu_stride = fused_row_stride(g.gu_rb); g.gu_gpr = H >> 6;
    g.dn_rb = M >> 1; g.dn_stride = g.dn_rb; g.dn_gpr = M >> 6;      // dense: the block's down rows arrive as one copy
    g.dn_cap = 4 * slots;
    // a block's share may touch two jobs: two ranges, each widened to 16-byte boundaries
    g.gu_sc_cap = ((slots * g.gu_gpr * 4 + 15) & ~15) + 64;
    g.dn_sc_cap = ((g.dn_cap * g.dn_gpr * 4 + 15) & ~15) + 64;
    size_t o = (size_t)2 * slots * g.gu_stride;
    g.off_dn = o;    o += (size_t)g.dn_cap * g.dn_stride;
    g.off_sgu = o;   o += (size_t)2 * g.gu_sc_cap;       // scale | bias words of the gate rows, of the up rows
    g.off_sdn = o;   o += (size_t)g.dn_sc_cap;           // scale | bias words of the down rows
    g.off_x = o;     o += (size_t)tt * H * 4;
    g.off_chain = o; o += (size_t)2 * tt * M * 4;
    g.off_jobs = o;  o += (size_t)FUSED_MAX_JOBS * sizeof(FusedJob);
    g.off_bars = o;  o += (size_t)(slots / 2 * FUSED_GU_CHUNKS + 4) * 8;   // gate/up barriers per warp and chunk, x, scales, down
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
#pragma unroll 1
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

// One lane's two rows for the NT tokens of its job: the dot products in the reference order
// (tile16_steps: sixteen lanes per row, lane v owns accumulators 2v and 2v + 1) and the canonical
// fold.  The rarely needed two-rounding form (a scale so large that q*s could overflow) is
// rolled up, so that it adds little to the code the SM has to fetch.
template <int NT>
__device__ __forceinline__ bool fused_slot(const NibbleMagic& mg, bool lit, int steps, const uint8_t* wA,
                                           const uint8_t* wB, const uint32_t* tA, const uint32_t* tB,
                                           const float* const (&xrow)[NT], int v, float (&yA)[NT], float (&yB)[NT],
                                           f32x2 nz, uint64_t* chunk_bars, uint32_t parity, int chunk_steps) {
    // the two row slots of a warp may belong to jobs with different token counts (or one of them
    // may be empty): the fold only involves the slot's own sixteen lanes
    const uint32_t half_mask = 0xffffu << (threadIdx.x & 16);
    bool timeout = false;
    f32x2 accA[NT], accB[NT];
#pragma unroll
    for (int tt = 0; tt < NT; tt++) { accA[tt] = pack2(0.0f, 0.0f); accB[tt] = pack2(0.0f, 0.0f); }
    // the rows arrive in chunks of chunk_steps steps (chunk_bars: one barrier per chunk; null: all here)
#pragma unroll 1
    for (int c0 = 0; c0 < steps; c0 += chunk_steps) {
        if (chunk_bars != nullptr && !fused_mbar_wait(chunk_bars + c0 / chunk_steps, parity)) timeout = true;
        const int c1 = min(c0 + chunk_steps, steps);
        int st = c0;
        if (lit) {
#pragma unroll 1
            for (; st + 2 <= c1; st += 2) {
                const float* xs[NT];
#pragma unroll
                for (int tt = 0; tt < NT; tt++) xs[tt] = xrow[tt] + st * 32;
                tile16_steps<NT, true, 2>(mg, wA + st * 16, wB + st * 16, tA + (st >> 1), tB + (st >> 1), xs, accA, accB, nz);
            }
        } else {
#pragma unroll 1
            for (; st + 8 <= c1; st += 8) {
                const float* xs[NT];
#pragma unroll
                for (int tt = 0; tt < NT; tt++) xs[tt] = xrow[tt] + st * 32;
                tile16_steps<NT, false, 8>(mg, wA + st * 16, wB + st * 16, tA + (st >> 1), tB + (st >> 1), xs, accA, accB, nz);
            }
#pragma unroll 1
            for (; st + 2 <= c1; st += 2) {
                const float* xs[NT];
#pragma unroll
                for (int tt = 0; tt < NT; tt++) xs[tt] = xrow[tt] + st * 32;
                tile16_steps<NT, false, 2>(mg, wA + st * 16, wB + st * 16, tA + (st >> 1), tB + (st >> 1), xs, accA, accB, nz);
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < NT; tt++) {
        yA[tt] = fold_row_hexadecants(accA[tt], v, half_mask);
        yB[tt] = fold_row_hexadecants(accB[tt], v, half_mask);
    }
    return timeout;
}

// A contiguous range of bf16 scales (or biases) staged in shared memory: rows [r0, r1) of one
// tensor, widened to 16-byte boundaries.  row_ptr(r) = stage + (r * row_bytes - byte0).
struct ScaleRange {
    int r0, r1;        // rows
    int byte0;         // first staged byte (multiple of 16) within the tensor's scale array
    int stage_off;     // offset of the staged range in its staging area
};

// Scale / bias words of up to NROWS rows of a warp held in registers between the read of the
// staged bf16 arrays and the write of the interleaved table that replaces them in place.
template <int NROWS, int IT>
struct TableRegs { uint32_t w[NROWS][IT]; };

// Shared-memory views of a block (see fused_geom).
template <int TT, int SLOTS>
struct FusedSmem {
    static constexpr int NT = 16 * SLOTS, NW = SLOTS / 2;
    uint8_t *sGU, *sDN, *sSG, *sSD;
    float *sX, *sC;
    FusedJob* sJ;
    uint64_t *bar_gu, *bar_x, *bar_sc, *bar_dn;
    __device__ __forceinline__ FusedSmem(uint8_t* smem, const FusedGeom& G) {
        sGU = smem;                                   // gate rows [0, SLOTS), up rows [SLOTS, 2*SLOTS), padded
        sDN = smem + G.off_dn;                        // [dn_cap] down rows, dense
        sSG = smem + G.off_sgu;                       // [2][gu_sc_cap] (scale << 16) | bias words of the gate / up rows
        sSD = smem + G.off_sdn;                       // [dn_sc_cap] the same for the down rows
        sX = (float*)(smem + G.off_x);                // [TT][H] the call's activation rows
        sC = (float*)(smem + G.off_chain);            // [2 jobs][TT][M] GeGLU rows of the down phase
        sJ = (FusedJob*)(smem + G.off_jobs);
        bar_gu = (uint64_t*)(smem + G.off_bars);      // [NW][FUSED_GU_CHUNKS] packed gate/up rows of a warp, by chunk
        bar_x = bar_gu + NW * FUSED_GU_CHUNKS;        // activations
        bar_sc = bar_x + 1;                           // scales and biases of the block (both phases)
        bar_dn = bar_x + 2;                           // packed down rows of the block
    }
    // by one thread, when no thread of the block can still be waiting on them: before they are initialised again
    __device__ __forceinline__ void inval_barriers() {
        for (int i = 0; i < NW * FUSED_GU_CHUNKS + 3; i++)
            asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar_gu + i)) : "memory");
    }
    // by one thread, before the block's first barrier
    __device__ __forceinline__ void init_barriers() {
        for (int i = 0; i < NW * FUSED_GU_CHUNKS + 3; i++) mbar_init(bar_gu + i, bar_gu + i == bar_sc ? 6 : 1);   // bar_sc: one arrival per table and job segment
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
};

// The expert phases of a block for the n_jobs descriptors in S.sJ (barriers initialised, the block
// synchronised).  x_resident: S.sX already holds the activation rows; otherwise they are copied from
// a.x.  Returns true when a bounded wait ran out.  Every thread of the block must call.
template <int TT, int SLOTS>
__device__ __forceinline__ bool fused_expert_rounds(const FusedArgs& a, const FusedGeom& G, const FusedSmem<TT, SLOTS>& S,
                                                    int n_jobs, bool x_resident, ScaleRange* s_rg, ScaleRange* s_rd) {
    constexpr int NT = 16 * SLOTS;
    const int H = a.H, M = a.M;
    uint8_t* const sGU = S.sGU; uint8_t* const sDN = S.sDN; uint8_t* const sSG = S.sSG; uint8_t* const sSD = S.sSD;
    float* const sX = S.sX; float* const sC = S.sC;
    FusedJob* const sJ = S.sJ;
    uint64_t* const bar_gu = S.bar_gu; uint64_t* const bar_x = S.bar_x; uint64_t* const bar_sc = S.bar_sc; uint64_t* const bar_dn = S.bar_dn;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int v = tid & 15, pr = tid >> 4;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int jpr = a.jobs_per_round;
    const int rounds = (n_jobs + jpr - 1) / jpr;
    const NibbleMagic mg = load_nibble_magic();
    const f32x2 nz = pack2u(c_neg_zero, c_neg_zero);
    uint32_t ph_gu = 0;            // phase of this warp's gate/up barrier
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
    // Packed gate/up rows: slots 2*warp and 2*warp + 1 belong to this warp.  A row is requested in
    // FUSED_GU_CHUNKS pieces (chunk-major: piece 0 of the warp's four rows first), each piece on its own
    // barrier, so that the dot products start on the first columns while the rest is still on its way.
    // Lane 4c + q issues piece c of (slot q & 1, matrix q >> 1) into a padded row.
    const int gu_chunk_steps = ((((H >> 5) + FUSED_GU_CHUNKS - 1) / FUSED_GU_CHUNKS) + 7) & ~7;
    int gu_rows_w = 0;                                // rows of this warp in flight / landed
    auto issue_gu = [&](const Round& R) {
        const int s0 = 2 * warp;
        const int nsl = max(0, min(2, R.gu_hi - R.gu_lo - s0));      // valid slots of this warp
        gu_rows_w = 2 * nsl;
        if (nsl == 0) return;
        const int c = lane >> 2, q = lane & 3;
        const int b0 = min(c * gu_chunk_steps * 16, G.gu_rb), b1 = min(b0 + gu_chunk_steps * 16, G.gu_rb);
        if (lane < 4 * FUSED_GU_CHUNKS && q == 0) mbar_expect_tx(bar_gu + warp * FUSED_GU_CHUNKS + c, (uint32_t)(2 * nsl * (b1 - b0)));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier reads of these rows precede the copies
        __syncwarp();
        const int sl = q & 1, mat = q >> 1;
        if (lane < 4 * FUSED_GU_CHUNKS && sl < nsl && b1 > b0) {
            const int p = R.gu_lo + s0 + sl;
            const FusedJob& jb = sJ[R.j0 + p / M];
            const uint8_t* vals = jb.v[mat];
            bulk_g2s(sGU + (size_t)(mat * SLOTS + s0 + sl) * G.gu_stride + b0, vals + (size_t)(p % M) * G.gu_rb + b0,
                     (uint32_t)(b1 - b0), bar_gu + warp * FUSED_GU_CHUNKS + c);
        }
    };
    // Ranges of the block's share [lo, hi) of an index space of `rows`-row jobs: up to two job segments.
    // The (scale << 16) | bias words of a segment's rows are contiguous: one copy per tensor and segment,
    // widened to 16-byte boundaries.  Lanes 0..5 of warp 0 each own one (tensor, segment) pair: lane =
    // 2 * tensor + segment, tensor 0 gate, 1 up, 2 down; bar_sc counts their six arrivals per round.
    auto issue_scales = [&](const Round& R) {
        if (lane >= 6) return;
        const int t = lane >> 1, seg = lane & 1;
        const bool dn = t == 2;
        const int lo = dn ? R.dn_lo : R.gu_lo, hi = dn ? R.dn_hi : R.gu_hi, rows = dn ? H : M;
        const int row_bytes = (dn ? G.dn_gpr : G.gu_gpr) * 4;
        const int j_first = lo / rows;
        ScaleRange sr;
        sr.r0 = 0; sr.r1 = 0; sr.byte0 = 0; sr.stage_off = 0;
        int nbytes = 0;
        for (int sg = 0; sg <= seg; sg++) {          // segment 1 starts where segment 0 ends in the staging area
            sr.stage_off += nbytes;
            const int slo = max(lo, (j_first + sg) * rows), shi = min(hi, (j_first + sg + 1) * rows);
            sr.r0 = 0; sr.r1 = 0; sr.byte0 = 0; nbytes = 0;
            if (hi > lo && shi > slo) {
                sr.r0 = slo - (j_first + sg) * rows; sr.r1 = shi - (j_first + sg) * rows;
                sr.byte0 = (sr.r0 * row_bytes) & ~15;
                nbytes = ((sr.r1 * row_bytes + 15) & ~15) - sr.byte0;        // the table's size is a multiple of 16
            }
        }
        if (t == 0) s_rg[seg] = sr;
        if (dn) s_rd[seg] = sr;
        mbar_expect_tx(bar_sc, (uint32_t)nbytes);
        if (nbytes > 0) {
            uint8_t* stage = dn ? sSD : sSG + (size_t)t * G.gu_sc_cap;
            bulk_g2s(stage + sr.stage_off, (const uint8_t*)sJ[R.j0 + j_first + seg].t[t] + sr.byte0, (uint32_t)nbytes, bar_sc);
        }
    };
    // The block's down rows are contiguous in memory and need no padding (the dense rows a warp reads
    // together already fall in different banks): one copy per job segment (s_rd).  One thread.
    auto issue_dn = [&](const Round& R) {
        uint32_t total = 0;
        for (int seg = 0; seg < 2; seg++) total += (uint32_t)((s_rd[seg].r1 - s_rd[seg].r0) * G.dn_rb);
        mbar_expect_tx(bar_dn, total);
        int row_off = 0;
        for (int seg = 0; seg < 2; seg++) {
            const int n = s_rd[seg].r1 - s_rd[seg].r0;
            if (n <= 0) continue;
            const FusedJob& jb = sJ[R.j0 + R.dn_lo / H + seg];
            bulk_g2s(sDN + (size_t)row_off * G.dn_rb, jb.v[2] + (size_t)s_rd[seg].r0 * G.dn_rb, (uint32_t)(n * G.dn_rb), bar_dn);
            row_off += n;
        }
    };
    // table row of row `row` (job-local, in segment seg) of staged tensor t
    auto table_row = [&](const ScaleRange* rg, const uint8_t* stage, int cap, int t, int seg, int row, int gpr) {
        return (const uint32_t*)(stage + (size_t)t * cap + rg[seg].stage_off + (row * gpr * 4 - rg[seg].byte0));
    };

    // order of the requests: the small ones first (scales, biases, activations: the tables are built
    // from them while the weights stream in), then every warp's gate/up rows, then the down rows
    Round R = round_of(0);
    if (warp == 0) issue_scales(R);
    if (tid == 0) {
        if (!x_resident) {
            mbar_expect_tx(bar_x, (uint32_t)(a.n_x * H * 4));
            for (int t = 0; t < a.n_x; t++) bulk_g2s(sX + (size_t)t * H, a.x + (size_t)t * a.x_stride, (uint32_t)(H * 4), bar_x);
        }
    }
    __syncthreads();               // s_rg / s_rd are published, the small requests are queued
    issue_gu(R);
    if (tid == 0) issue_dn(R);
    if (!x_resident && !fused_mbar_wait(bar_x, 0)) timeout = true;

    for (int r = 0; r < rounds; r++) {
        if (!fused_mbar_wait(bar_sc, r & 1)) timeout = true;
        // ================= gate | up + GeGLU =================
        const int p = R.gu_lo + pr;
        if (p < R.gu_hi) {
            const int jl = p / M, row = p - jl * M;
            const FusedJob& jb = sJ[R.j0 + jl];
            const uint8_t* wA = sGU + (size_t)pr * G.gu_stride + v;
            const uint8_t* wB = sGU + (size_t)(SLOTS + pr) * G.gu_stride + v;
            const uint32_t* tA = table_row(s_rg, sSG, G.gu_sc_cap, 0, jl - R.gu_lo / M, row, G.gu_gpr);
            const uint32_t* tB = table_row(s_rg, sSG, G.gu_sc_cap, 1, jl - R.gu_lo / M, row, G.gu_gpr);
            const bool lit_gu = (jb.lit & 3) != 0;
            const int ntok = jb.ntok;
            float* crow = a.chain + (size_t)jb.g0 * M + row;
            if (TT >= 4 && ntok >= 3) {
                constexpr int N = TT >= 4 ? 4 : 1;
                const float* xr[N];
                float yA[N], yB[N];
#pragma unroll
                for (int t = 0; t < N; t++) xr[t] = sX + (size_t)jb.x_row[min(t, ntok - 1)] * H + 2 * v;
                timeout |= fused_slot<N>(mg, lit_gu, H >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz, bar_gu + warp * FUSED_GU_CHUNKS, ph_gu & 1, gu_chunk_steps);
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
                timeout |= fused_slot<N>(mg, lit_gu, H >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz, bar_gu + warp * FUSED_GU_CHUNKS, ph_gu & 1, gu_chunk_steps);
                if (v == 0)
#pragma unroll
                    for (int t = 0; t < N; t++) crow[(size_t)t * M] = __fmul_rn(gelu_tanh_exact(yA[t]), yB[t]);
            } else {
                const float* xr[1] = {sX + (size_t)jb.x_row[0] * H + 2 * v};
                float yA[1], yB[1];
                timeout |= fused_slot<1>(mg, lit_gu, H >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz, bar_gu + warp * FUSED_GU_CHUNKS, ph_gu & 1, gu_chunk_steps);
                if (v == 0) crow[0] = __fmul_rn(gelu_tanh_exact(yA[0]), yB[0]);
            }
        }
        __syncwarp();
        if (gu_rows_w > 0) ph_gu++;    // this warp's chunk barriers have all completed a phase
        Round Rn = R;
        if (r + 1 < rounds) {          // this warp's gate/up rows are free again: next round's copies
            Rn = round_of(r + 1);
            issue_gu(Rn);
        }
        __syncthreads();               // every GeGLU value of this block has been written
        if (tid == 0) {
            if (R.gu_hi > R.gu_lo) {
                __threadfence();
                const int ja = R.gu_lo / M, jb2 = (R.gu_hi - 1) / M;
                for (int j = ja; j <= jb2; j++) {
                    const int lo = max(R.gu_lo, j * M), hi = min(R.gu_hi, (j + 1) * M);
                    atomicAdd(a.done + R.j0 + j, hi - lo);
                }
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
        if (!fused_mbar_wait(bar_dn, r & 1)) timeout = true;
        __syncthreads();
#pragma unroll 1
        for (int ps = 0; ps < 2; ps++) {
            const int li = ps * 2 * SLOTS + 2 * pr;
            if (li >= dn_n) continue;
            const int qg = R.dn_lo + li;
            const int jl = qg / H, row = qg - jl * H;
            const FusedJob& jb = sJ[R.j0 + jl];
            const uint8_t* wA = sDN + (size_t)li * G.dn_stride + v;
            const uint8_t* wB = wA + G.dn_stride;
            const uint32_t* tA = table_row(s_rd, sSD, G.dn_sc_cap, 0, jl - dja, row, G.dn_gpr);
            const uint32_t* tB = tA + G.dn_gpr;
            const bool lit_dn = (jb.lit & 4) != 0;
            const float* cbase = sC + (size_t)(jl - dja) * TT * M + 2 * v;
            const int ntok = jb.ntok;
            float* orow = a.out + (size_t)jb.g0 * H + row;
            if (TT >= 4 && ntok >= 3) {
                constexpr int N = TT >= 4 ? 4 : 1;
                const float* xr[N];
                float yA[N], yB[N];
#pragma unroll
                for (int t = 0; t < N; t++) xr[t] = cbase + (size_t)min(t, ntok - 1) * M;
                fused_slot<N>(mg, lit_dn, M >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz, nullptr, 0, M >> 5);
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
                fused_slot<N>(mg, lit_dn, M >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz, nullptr, 0, M >> 5);
                if (v == 0)
#pragma unroll
                    for (int t = 0; t < N; t++) *(float2*)(orow + (size_t)t * H) = make_float2(yA[t], yB[t]);
            } else {
                const float* xr[1] = {cbase};
                float yA[1], yB[1];
                fused_slot<1>(mg, lit_dn, M >> 5, wA, wB, tA, tB, xr, v, yA, yB, nz, nullptr, 0, M >> 5);
                if (v == 0) *(float2*)orow = make_float2(yA[0], yB[0]);
            }
        }
        __syncthreads();               // the block is done with this round's down rows and tables
        if (r + 1 < rounds && warp == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_scales(Rn);
            __syncwarp();              // s_rd is read by the thread that requests the down rows
            if (tid == 0) issue_dn(Rn);
        }
        __syncthreads();               // next round's s_rg / s_rd are published
        R = Rn;
    }
    return timeout;
}

template <int TT, int SLOTS>
__global__ void __launch_bounds__(16 * SLOTS, 1) q4_fused_expert_kernel(FusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NT = 16 * SLOTS;
    const FusedGeom G = fused_geom(a.H, a.M, TT, SLOTS);
    FusedSmem<TT, SLOTS> S(smem, G);
    __shared__ int s_njobs;
    __shared__ ScaleRange s_rg[2], s_rd[2];                // the (up to two) job segments of the block's shares
    const int tid = threadIdx.x;
    if (tid == 0) S.init_barriers();
    pdl_wait();                    // the jobs, the counters and the activations come from the previous kernel
    pdl_launch_dependents();
    {
        // the live count and the whole job table in one round trip (read through L2: another
        // layer's table may still sit in this SM's L1)
        const int n_live = __ldcg(a.n_jobs_dev);
        static_assert(sizeof(FusedJob) % 16 == 0, "job descriptors are copied in 16-byte pieces");
        const int pieces = a.n_jobs_max * (int)(sizeof(FusedJob) / 16);
        for (int i = tid; i < pieces; i += NT) ((uint4*)S.sJ)[i] = __ldcg((const uint4*)a.jobs + i);
        if (tid == 0) s_njobs = min(max(n_live, 0), a.n_jobs_max);
    }
    __syncthreads();               // barriers initialised, jobs and count in shared memory
    const int n_jobs = s_njobs;
    if (n_jobs == 0) return;
    const bool timeout = fused_expert_rounds<TT, SLOTS>(a, G, S, n_jobs, false, s_rg, s_rd);
    if (timeout && a.status) atomicOr(a.status, SB_ERR_TIMEOUT);
}

// ---- one launch per decode layer (one token) -------------------------------------------------
// [ordered reduce + RMSNorm of the previous layer] -> router input -> router logits -> softmax
// top-k -> job list -> the expert phases above, in ONE launch of one block per SM.
//   * the row-wise glue (reference src/tensorops.c:291-325, gemma4.c:85-130) is computed by EVERY
//     block for itself: its results (the experts' activation row, the router input) stay in the
//     block's shared memory and nothing is waited for;
//   * block e forms the logit of expert e (reference src/kernels.c:98-106: one dependent-add chain
//     over the hidden size, handed from lane to lane of one warp), stores it and bumps an arrival
//     counter; every block polls the counter (bounded), reads the logits and repeats the top-k
//     (gemma4.c:132-186) and the job list for itself;
//   * block 0 also leaves selections, weights and the (trivial, one token) grouping in global
//     memory for the next layer's reduce and for the caller.
// The scratch of these phases overlays the weight rows, which are not requested before the job
// list exists.  The previous layer's grouped outputs and weights are read from the buffers of the
// OTHER parity, so a block that is late in its glue never sees rows of this layer.
constexpr int LAYER_NV = 5;                 // columns per thread of the row-wise glue
constexpr int LAYER_SLOTS = 40;

struct LayerScratch {                        // offsets in floats from the start of shared memory
    int sq, rin, wrow, logits, pes, lit, topk, scan, end;
};
static __host__ __device__ __forceinline__ LayerScratch layer_scratch(int H, int E, int topk) {
    LayerScratch L;
    const int h4 = (H + 3) & ~3;
    L.sq = 0; L.rin = h4; L.wrow = 2 * h4; L.logits = 3 * h4;
    L.pes = L.logits + ((E + 3) & ~3);           // the layer's per-expert scales ...
    L.lit = L.pes + ((E + 3) & ~3);              // ... and literal-dequantisation flags, fetched before the grid dependency
    L.topk = L.lit + ((E + 3) & ~3);
    L.scan = L.topk + topk_scratch_floats(E, topk);
    L.end = L.scan + POSSUM_SCRATCH;
    return L;
}

// one copy of the in-order sum for both of its uses (less code for the SM to fetch)
static __device__ __noinline__ float layer_ordered_sum(const float* sq, int n, bool bad, uint32_t* scan) {
    return ordered_sum_of_squares<LAYER_NV>(sq, n, bad, scan);
}

// One layer by the whole grid.  STACKED = false: the body of q4_layer_decode_kernel (one launch per layer; the
// previous layer is the previous kernel).  STACKED = true: layer `li` of q4_stack_decode_kernel, whose blocks
// stay resident over all layers: the previous layer is complete when every block has bumped its counter
// (prev_done reaches the grid size; bounded wait), and the block's barriers are re-initialised.
template <bool STACKED>
__device__ __forceinline__ void layer_decode_body(const LayerDecodeArgs& a, uint8_t* smem, int li, const int* prev_done,
                                                  int* my_done) {
    constexpr int SLOTS = LAYER_SLOTS, NT = 16 * SLOTS, NV = LAYER_NV;
    const int H = a.f.H, M = a.f.M, E = a.E, K = a.topk;
    const FusedGeom G = fused_geom(H, M, 1, SLOTS);
    FusedSmem<1, SLOTS> S(smem, G);
    const LayerScratch L = layer_scratch(H, E, K);
    float* const fsm = (float*)smem;
    float* const sq = fsm + L.sq;                 // squares / products for the in-order chains
    float* const rin = fsm + L.rin;               // router input
    float* const wrow = fsm + L.wrow;             // router weights of this block's expert
    float* const s_logits = fsm + L.logits;
    float* const s_pes = fsm + L.pes;
    int* const s_lit = (int*)(fsm + L.lit);
    float* const tk = fsm + L.topk;
    uint32_t* const scan = (uint32_t*)(fsm + L.scan);
    __shared__ float s_inv, s_root, s_w[64], s_wts[64];
    __shared__ int s_sel[64], s_njobs;
    __shared__ ScaleRange s_rg[2], s_rd[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;
    bool bad = false, timeout = false;

    // ---- before the dependency: barriers, this block's router row, the norm weights ----
    if (tid == 0) {
        if (STACKED && li > 0) S.inval_barriers();    // every wait of the previous layer is over (block barrier at its end)
        S.init_barriers();
        if (cta < E) {
            mbar_expect_tx(S.bar_x, (uint32_t)(H * 4));
            bulk_g2s(wrow, a.router_w + (size_t)cta * H, (uint32_t)(H * 4), S.bar_x);
        }
    }
    float v[NV], nw[NV], rs[NV];
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const int d = tid + j * NT;
        nw[j] = (a.norm_w != nullptr && d < H) ? __ldg(a.norm_w + d) : 1.0f;
        rs[j] = d < H ? __ldg(a.router_scale + d) : 1.0f;
        v[j] = 0.0f;
    }
    // layer constants the top-k and the job list need: in shared memory long before they are used
    for (int e = tid; e < E; e += NT) {
        s_pes[e] = a.per_expert_scale != nullptr ? __ldg(a.per_expert_scale + e) : 1.0f;
        s_lit[e] = (e >= a.expert_begin && e < a.expert_end) ? __ldg(a.lit_flags + (e - a.expert_begin)) : 0;
    }
    if (!STACKED) {
        pdl_wait();                // the previous layer's outputs
        pdl_launch_dependents();
    } else if (li > 0) {
        // the previous layer's outputs: every block of the grid has finished it
        if (tid == 0) {
            uint32_t i = 0;
            while (ld_acquire_gpu(prev_done) < ncta && i < FUSED_SPIN_LIMIT) i++;
            if (i >= FUSED_SPIN_LIMIT) timeout = true;
        }
        __syncthreads();
    } else {
        pdl_wait();
    }

    // ---- the layer's input row: ordered weighted reduce of the previous layer, or the stack input ----
    if (a.prev_grouped != nullptr) {
        if (tid < K) {
            const float w = __ldcg(a.prev_weights + tid);
            if (!finite_f(w)) flag(a.f.status, SB_ERR_NONFINITE);
            s_w[tid] = w;
        }
        __syncthreads();
        for (int r0 = 0; r0 < K; r0 += 8) {
            float o[NV][8];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < NV; j++) {
                    const int d = tid + j * NT;
                    o[j][i] = (r0 + i < K && d < H) ? __ldcg(a.prev_grouped + (size_t)(r0 + i) * H + d) : 0.0f;
                }
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (r0 + i < K && finite_f(s_w[r0 + i])) {
                    const float w = s_w[r0 + i];
#pragma unroll
                    for (int j = 0; j < NV; j++) v[j] = __fadd_rn(v[j], __fmul_rn(w, o[j][i]));
                }
        }
    } else {
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int d = tid + j * NT;
            if (d < H) v[j] = __ldcg(a.x_in + d);
        }
    }
    if (a.norm_w != nullptr) {      // RMSNorm of the previous layer (gemma4.c:85-101)
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int d = tid + j * NT;
            if (d < H) {
                sq[d] = __fmul_rn(v[j], v[j]);
                bad |= !finite_f(v[j]) || !finite_f(nw[j]);
            }
        }
        const float ss = layer_ordered_sum(sq, H, bad, scan);
        if (tid == 0) {
            s_inv = pow_neg_half(__fadd_rn(__fdiv_rn(ss, (float)H), a.eps_norm));
            if (!finite_f(s_inv)) flag(a.f.status, SB_ERR_NONFINITE);
        }
        __syncthreads();
        const float inv = s_inv;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            v[j] = __fmul_rn(__fmul_rn(v[j], inv), nw[j]);
            if (tid + j * NT < H) bad |= !finite_f(v[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const int d = tid + j * NT;
        if (d < H) {
            S.sX[d] = v[j];           // the experts' activation row
            if (cta == 0 && a.y_out != nullptr) a.y_out[d] = v[j];
        }
    }
    // ---- router input (gemma4.c:103-130) ----
    __syncthreads();                // the previous in-order sum has been read by everyone
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const int d = tid + j * NT;
        if (d < H) {
            sq[d] = __fmul_rn(v[j], v[j]);
            bad |= !finite_f(v[j]) || !finite_f(rs[j]);
        }
    }
    {
        const float ss = layer_ordered_sum(sq, H, bad, scan);
        if (tid == 0) {
            s_inv = pow_neg_half(__fadd_rn(__fdiv_rn(ss, (float)H), a.eps_router));
            s_root = __fdiv_rn(1.0f, sqrtf_exact((float)H));
            if (!finite_f(s_inv) || !finite_f(s_root)) flag(a.f.status, SB_ERR_NONFINITE);
        }
        __syncthreads();
        const float inv = s_inv, root = s_root;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int d = tid + j * NT;
            if (d < H) {
                const float t = __fmul_rn(__fmul_rn(__fmul_rn(v[j], inv), rs[j]), root);
                bad |= !finite_f(t);
                rin[d] = t;
            }
        }
    }
    if (bad) flag(a.f.status, SB_ERR_NONFINITE);
    __syncthreads();                // the router input is complete
    // ---- router logits: expert e = cta, cta + grid, ... ----
    uint32_t ph_w = 0;
    for (int e = cta; e < E; e += ncta) {
        if (e != cta && tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(S.bar_x, (uint32_t)(H * 4));
            bulk_g2s(wrow, a.router_w + (size_t)e * H, (uint32_t)(H * 4), S.bar_x);
        }
        if (warp == 0) {
            if (!fused_mbar_wait(S.bar_x, ph_w & 1)) timeout = true;
            // acc = fl(acc + fl(W[c] * rin[c])), c ascending (reference src/kernels.c:98-106), handed from
            // lane to lane.  The row is cut into passes of 32 * CHP columns; in a pass lane l holds the
            // products of columns [l*CHP, (l+1)*CHP) in registers, so a step of the chain costs one
            // dependent-add latency and nothing else.  Every lane runs the adds of every turn on its own
            // products (no divergence); only the lane whose turn it is keeps the result.
            constexpr int CHP = 44;
            float acc = 0.0f;
            float cur[CHP];
            const int npass = (H + 32 * CHP - 1) / (32 * CHP);
#pragma unroll 1
            for (int ps = 0; ps < npass; ps++) {
                const int c0 = ps * 32 * CHP + lane * CHP;
#pragma unroll
                for (int i = 0; i < CHP; i += 4) {
                    // columns past H read scratch that is never added
                    const float4 wv = *(const float4*)(wrow + c0 + i), xv = *(const float4*)(rin + c0 + i);
                    cur[i] = __fmul_rn(wv.x, xv.x); cur[i + 1] = __fmul_rn(wv.y, xv.y);
                    cur[i + 2] = __fmul_rn(wv.z, xv.z); cur[i + 3] = __fmul_rn(wv.w, xv.w);
                }
                const bool full = (ps + 1) * 32 * CHP <= H;                 // every lane has CHP valid columns
                const int mine = min(CHP, max(0, H - c0));
#pragma unroll 1
                for (int l = 0; l < 32; l++) {
                    float s = __shfl_sync(0xffffffffu, acc, (l + 31) & 31);
                    if (l == 0 && ps == 0) s = 0.0f;
                    if (full) {
#pragma unroll
                        for (int i = 0; i < CHP; i++) s = __fadd_rn(s, cur[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < CHP; i++) {
                            const float t = __fadd_rn(s, cur[i]);
                            s = i < mine ? t : s;
                        }
                    }
                    acc = lane == l ? s : acc;
                }
            }
            if (lane == 31) {
                a.logits[e] = acc;
                asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(a.logits_count) : "memory");
            }
        }
        ph_w++;
        if (e + ncta < E) __syncthreads();     // the router row is free for the next expert's copy
    }
    // ---- all logits, then top-k and the job list, by every block for itself ----
    if (tid == 0) {
        uint32_t i = 0;
        while (ld_acquire_gpu(a.logits_count) < E && i < FUSED_SPIN_LIMIT) i++;
        if (i >= FUSED_SPIN_LIMIT) timeout = true;
    }
    __syncthreads();
    for (int e = tid; e < E; e += NT) s_logits[e] = __ldcg(a.logits + e);
    __syncthreads();
    topk_group(tid < 128, s_logits, s_pes, s_sel, s_wts, E, K, 1, cta == 0 ? a.f.status : nullptr, tk,
               tk + topk_scratch_floats(E, K) - 4, tid & 127, 128);
    __syncthreads();
    // job list: thread j takes selection j (its slot = the local selections before it; the list keeps rank order)
    if (tid < K) {
        const int j = tid, e = s_sel[j];
        int slot = 0, total = 0;
        for (int i = 0; i < K; i++) {
            const int ei = s_sel[i];
            const int local = (ei >= a.expert_begin && ei < a.expert_end) ? 1 : 0;
            total += local;
            if (i < j) slot += local;
        }
        if (e >= a.expert_begin && e < a.expert_end && slot < FUSED_MAX_JOBS) {
            const uint8_t* base = a.pool + (size_t)(e - a.expert_begin) * a.expert_stride;
            FusedJob fj;
            const uint8_t* tb = a.tables + (size_t)(e - a.expert_begin) * 6 * a.group_bytes;
            for (int k = 0; k < 3; k++) {
                fj.v[k] = base + (size_t)k * a.tensor_bytes;
                fj.t[k] = (const uint32_t*)(tb + (size_t)k * 2 * a.group_bytes);
            }
            fj.lit = s_lit[e]; fj.pad = 0;
            for (int t = 0; t < FUSED_MAX_TOKENS; t++) fj.x_row[t] = 0;
            fj.g0 = j; fj.ntok = 1;              // one token: grouped order = rank order (experts ascending)
            S.sJ[slot] = fj;
        }
        if (j == 0) s_njobs = min(total, FUSED_MAX_JOBS);
    }
    if (cta == 0) {                 // what the next layer's reduce and the caller read
        if (tid < K) {
            a.selected[tid] = s_sel[tid];
            a.weights_out[tid] = s_wts[tid];
            a.c2g[tid] = tid;
            a.g2c[tid] = tid;
        }
        for (int e = tid; e <= E; e += NT) {
            int lt = 0;
            for (int j = 0; j < K; j++) lt += s_sel[j] < e ? 1 : 0;
            a.group_offsets[e] = lt;
        }
    }
    __syncthreads();                // jobs published; the scratch is dead: the weight rows may land on it
    const int n_jobs = s_njobs;
    if (n_jobs > 0) timeout |= fused_expert_rounds<1, SLOTS>(a.f, G, S, n_jobs, true, s_rg, s_rd);
    if (timeout && a.f.status) atomicOr(a.f.status, SB_ERR_TIMEOUT);
    if (STACKED) {
        __syncthreads();            // all of this block's rows of the layer are written, its shared memory is free
        if (tid == 0) {
            __threadfence();
            asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(my_done) : "memory");
        }
    }
}

__global__ void __launch_bounds__(16 * LAYER_SLOTS, 1) q4_layer_decode_kernel(LayerDecodeArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    layer_decode_body<false>(a, smem, 0, nullptr, nullptr);
}

// All layers of a decode step in ONE launch: the blocks (one per SM) stay resident, so the code of a layer is
// fetched once per step instead of once per layer, and a layer ends with one arrival counter instead of a kernel
// boundary.  layers[li] are the per-layer arguments (device memory), done[li] the arrival counters (zero at launch).
__global__ void __launch_bounds__(16 * LAYER_SLOTS, 1)
q4_stack_decode_kernel(const LayerDecodeArgs* __restrict__ layers, int n_layers, int* done) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(16) LayerDecodeArgs s_args;
    static_assert(sizeof(LayerDecodeArgs) % 16 == 0, "layer arguments are copied in 16-byte pieces");
#pragma unroll 1
    for (int li = 0; li < n_layers; li++) {
        __syncthreads();            // the previous layer's arguments are no longer read
        for (int i = threadIdx.x; i < (int)(sizeof(LayerDecodeArgs) / 16); i += blockDim.x)
            ((uint4*)&s_args)[i] = __ldg((const uint4*)(layers + li) + i);
        __syncthreads();
        layer_decode_body<true>(s_args, smem, li, li > 0 ? done + li - 1 : nullptr, done + li);
    }
    pdl_launch_dependents();
}

// ---- derived scale | bias tables ------------------------------------------------------------
// words[e][k][i] = (scale bf16 << 16) | bias bf16 of group i of tensor k (0 gate, 1 up, 2 down) of local
// expert e; flags[e] bit k = some scale of that tensor needs the two-rounding dequantisation.
__global__ void __launch_bounds__(256)
q4_interleave_tables_kernel(const uint8_t* __restrict__ pool, size_t expert_stride, size_t tensor_bytes, size_t value_bytes,
                            size_t groups, uint32_t* __restrict__ words, int* __restrict__ flags) {
    const int e = blockIdx.y, k = blockIdx.z;
    const uint8_t* t = pool + (size_t)e * expert_stride + (size_t)k * tensor_bytes;
    const uint16_t* sc = (const uint16_t*)(t + value_bytes);
    const uint16_t* bi = sc + groups;
    uint32_t* out = words + ((size_t)e * 3 + k) * groups;
    int lit = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t hs = sc[i];
        out[i] = (hs << 16) | (uint32_t)bi[i];
        lit |= scale_needs_literal(hs) ? 1 : 0;
    }
    if (lit) atomicOr(flags + e, 1 << k);
}

cudaError_t launch_q4_interleave_tables(const uint8_t* pool, size_t expert_stride, size_t tensor_bytes, size_t value_bytes,
                                        size_t groups, int n_experts, uint32_t* words, int* flags, cudaStream_t stream) {
    if (n_experts < 1) return cudaSuccess;
    cudaError_t e = cudaMemsetAsync(flags, 0, (size_t)n_experts * sizeof(int), stream);
    if (e != cudaSuccess) return e;
    q4_interleave_tables_kernel<<<dim3(32, n_experts, 3), 256, 0, stream>>>(pool, expert_stride, tensor_bytes, value_bytes, groups,
                                                                          words, flags);
    return cudaGetLastError();
}

// ---- host side ---------------------------------------------------------------------------
namespace {
struct DeviceInfo { int sms = 0; };
DeviceInfo g_dev[64];

DeviceInfo* device_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    DeviceInfo* d = &g_dev[dev];
    if (d->sms == 0 && cudaDeviceGetAttribute(&d->sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    return d;
}
constexpr size_t FUSED_SMEM_LIMIT = 227 * 1024 - 3072;   // dynamic part: the opt-in maximum less the kernel's static variables
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
    if (g.total > FUSED_SMEM_LIMIT) return false;
    const int grid = d->sms;
    // most jobs per round whose shares fit the block: ceil(J*M/grid) <= slots, ceil(J*H/grid) <= dn_cap
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
static cudaError_t launch_fused_t(FusedArgs& a, const FusedLaunch& L, cudaStream_t stream) {
    cudaError_t e = ensure_dynamic_smem((const void*)q4_fused_expert_kernel<TT, SLOTS>, FUSED_SMEM_LIMIT);
    if (e != cudaSuccess) return e;
    return launch_pdl(q4_fused_expert_kernel<TT, SLOTS>, dim3(L.grid), dim3(16 * SLOTS), L.smem, stream, a);
}

cudaError_t launch_q4_fused(const FusedArgs& args, cudaStream_t stream) {
    FusedLaunch L;
    if (!q4_fused_plan(args.H, args.M, args.n_x, args.n_jobs_max, &L)) return cudaErrorInvalidValue;
    if ((((uintptr_t)args.x) & 15) || ((args.x_stride * 4) & 15)) return cudaErrorInvalidValue;
    FusedArgs a = args;
    a.jobs_per_round = L.jobs_per_round;
    if (L.tt == 1) return launch_fused_t<1, 40>(a, L, stream);
    if (L.tt == 2) return launch_fused_t<2, 32>(a, L, stream);
    return launch_fused_t<4, 32>(a, L, stream);
}

bool q4_layer_decode_plan(int H, int M, int E, int topk, int n_jobs_max, FusedLaunch* out) {
    FusedLaunch L;
    if (!q4_fused_plan(H, M, 1, n_jobs_max, &L) || L.tt != 1 || H > 16 * LAYER_SLOTS * LAYER_NV || (H & 3) || E < 1 ||
        E > 1024 || topk < 1 || topk > 64 || topk > E)
        return false;
    const FusedGeom g = fused_geom(H, M, 1, LAYER_SLOTS);
    if ((size_t)layer_scratch(H, E, topk).end * 4 > g.off_sgu) return false;    // the scratch overlays the weight rows only
    if (out) *out = L;
    return true;
}

cudaError_t launch_q4_stack_decode(const LayerDecodeArgs* d_layers, int n_layers, int* d_done, int H, int M, int E, int topk,
                                   int n_jobs_max, cudaStream_t stream) {
    FusedLaunch L;
    if (n_layers < 1 || !q4_layer_decode_plan(H, M, E, topk, n_jobs_max, &L)) return cudaErrorInvalidValue;
    cudaError_t e = ensure_dynamic_smem((const void*)q4_stack_decode_kernel, FUSED_SMEM_LIMIT);
    if (e != cudaSuccess) return e;
    return launch_pdl(q4_stack_decode_kernel, dim3(L.grid), dim3(16 * LAYER_SLOTS), L.smem, stream, d_layers, n_layers, d_done);
}

// jobs_per_round of a layer's arguments (what launch_q4_layer_decode fills in for a single launch)
int q4_layer_decode_jobs_per_round(int H, int M, int E, int topk, int n_jobs_max) {
    FusedLaunch L;
    return q4_layer_decode_plan(H, M, E, topk, n_jobs_max, &L) ? L.jobs_per_round : 0;
}

cudaError_t launch_q4_layer_decode(const LayerDecodeArgs& args, int n_jobs_max, cudaStream_t stream) {
    FusedLaunch L;
    if (!q4_layer_decode_plan(args.f.H, args.f.M, args.E, args.topk, n_jobs_max, &L)) return cudaErrorInvalidValue;
    cudaError_t e = ensure_dynamic_smem((const void*)q4_layer_decode_kernel, FUSED_SMEM_LIMIT);
    if (e != cudaSuccess) return e;
    LayerDecodeArgs a = args;
    a.f.jobs_per_round = L.jobs_per_round;
    a.f.n_x = 1;
    return launch_pdl(q4_layer_decode_kernel, dim3(L.grid), dim3(16 * LAYER_SLOTS), L.smem, stream, a);
}

}  // namespace sb
