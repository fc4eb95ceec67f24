// Grouped NVFP4 (W4A4) expert GEMMs on the 5th-generation tensor cores: block-scaled
// tcgen05.mma.kind::mxf4nvf4 (E2M1 codes in both operands, one unsigned E4M3 scale per 16 K elements of
// each operand, fp32 accumulation in TMEM) for batches where the bit-exact CUDA-core kernels of
// nvfp4_kernels.cu are compute bound.  TOLERANCE path: the tensor core forms
//     sum over 16-blocks of (sum of code products) * weight scale * activation scale
// in its own order and the epilogue applies the two per-tensor scalars (1 / weight divisor, 1 / input global
// scale), where the reference (src/nvfp4.c:173-192, 228-256) rounds scale * scalar first and adds in its
// 32-accumulator order: same real number, different fp32 roundings (measured against the CPU path in the
// tests; the bound is 1e-3 of max(|ref|, row rms)).  Activation codes and scales come from the bit-exact
// quantiser (nvfp4_qdq_kernel), so the only difference is the order of the additions.
//
// One tile = 128 rows of one weight matrix of one expert; the weight rows sit on the MMA M dimension, the
// expert's tokens on N (16, 32 or 64 per pass), K advances in chunks of 256 columns = one 128-byte row of
// packed codes = four MMAs of K = 64.  Blocks are persistent, one per SM: each walks its share of the
// launch's tiles with the copy pipeline running across tile boundaries.  Warp roles:
//   warp 9      producer: TMA (cp.async.bulk.tensor, no multicast) of the weight tile (3-D map: byte column,
//               row, expert; 128-byte swizzle), of the tokens' packed activations (2-D map), and of the chunk's
//               16 scale bytes of every weight row (row-major [R][C/16], reference layout
//               src/nvfp4.c:147-149) and token row (the quantiser's output), eight stages ahead
//   warps 0-3   scale warps: move the stage's scale bytes from shared memory into TMEM with tcgen05.st in the
//               layout the MMA reads - row r of a 128-row operand in lane r % 32 of every 32-lane quarter,
//               32-bit column r / 32, byte j = K block j of the MMA - so the scales need no rearranged copy
//   warp 8      issuer: waits for the stage's data and scales, issues the four MMAs, tcgen05.commit
//   warps 4-7   epilogue: tcgen05.ld of a finished accumulator buffer (two alternate), scalars, store
// Every mbarrier wait is bounded; on expiry the block raises its failure flag, sets SB_ERR_TIMEOUT, waits
// (bounded) for copies and MMAs in flight, frees its TMEM and returns.
#include <algorithm>

#include "internal.h"
#include "umma.cuh"

namespace sb {

constexpr int FT_STAGES = 8;
constexpr int FT_THREADS = 320;                   // warps 0-3 scales, 4-7 epilogue, 8 issuer, 9 producer
constexpr int FT_KC_BYTES = 128;                  // packed bytes of a K chunk (256 columns)
constexpr int FT_A_BYTES = 128 * FT_KC_BYTES;     // 128 weight rows
constexpr int FT_MAX_NT = 64;                     // tokens per pass
constexpr int FT_B_BYTES = FT_MAX_NT * FT_KC_BYTES;
constexpr int FT_SFA_BYTES = 128 * 16, FT_SFB_BYTES = FT_MAX_NT * 16;   // 16 scale bytes per row and chunk
constexpr int FT_STAGE_BYTES = FT_A_BYTES + FT_B_BYTES + FT_SFA_BYTES + FT_SFB_BYTES;
constexpr int FT_SMEM_BYTES = FT_STAGES * FT_STAGE_BYTES + 1024;
constexpr int FT_MAX_TILES = 48;                  // tiles of one block's list
constexpr uint32_t FT_TMEM_COLS = 512;            // accumulators at 0..63 and 64..127, scale stages from 128
constexpr uint32_t FT_SF_BASE = 128, FT_SF_STAGE = 32, FT_SFB_OFF = 16;

// kind::mxf4nvf4 instruction descriptor: A = B = E2M1 (format 1), both K-major, scales unsigned E4M3
// (format 0), scale ids 0 (a K = 64 MMA with 16-element blocks uses all four bytes of a scale column), K = 64.
__device__ __forceinline__ uint32_t umma_idesc_fp4(int M, int N) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_fp4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}\n" ::
            "r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
}

struct Fp4TcArgs {
    const Fp4TcJob* jobs;
    int njobs, tiles_per_job;
    int C;                // K of the launch (columns of the weight matrices), a multiple of 256
    int* status;
};

// One tile of a block's list: the job's fields every role needs, and the tile's first weight row.
struct Fp4Tile {
    float* y;
    float wg, ig;
    int w_row, ws_row, w_slice, x_row0, ntok, R, y_stride, r0;
};

__global__ void __launch_bounds__(FT_THREADS, 1)
nvfp4_gemm_tc_kernel(const Fp4TcArgs a, const __grid_constant__ Fp4TcMaps maps) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ Fp4Tile s_tiles[FT_MAX_TILES];
    __shared__ __align__(8) uint64_t bar_free[FT_STAGES];   // the stage's MMAs are complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_full[FT_STAGES];   // the stage's TMA copies have landed
    __shared__ __align__(8) uint64_t bar_sf[FT_STAGES];     // the stage's scales are in TMEM (4 warp arrivals)
    __shared__ __align__(8) uint64_t bar_done[2];           // an accumulator buffer is final
    __shared__ __align__(8) uint64_t bar_accfree[2];        // ... and has been read out (4 warp arrivals)
    __shared__ __align__(8) uint64_t bar_drain;             // failure path only: everything issued has completed
    __shared__ uint32_t s_tmem;
    __shared__ int s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nchunks = a.C >> 8;
    // this block's tiles: t = blockIdx.x, + gridDim.x, ... over (job, row tile); consecutive blocks take the
    // row tiles of one job, so its activations stay in L2.  The launch keeps the list within FT_MAX_TILES.
    const int total_tiles = a.njobs * a.tiles_per_job;
    const int my_tiles = ((int)blockIdx.x < total_tiles) ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    for (int i = tid; i < my_tiles && i < FT_MAX_TILES; i += FT_THREADS) {
        const int t = (int)blockIdx.x + i * (int)gridDim.x;
        const int j = t / a.tiles_per_job, rt = t - j * a.tiles_per_job;
        const Fp4TcJob jb = a.jobs[j];
        Fp4Tile ti;
        ti.y = jb.y; ti.wg = jb.wg; ti.ig = jb.ig;
        ti.r0 = rt * 128; ti.w_row = jb.w_row0 + ti.r0; ti.ws_row = jb.ws_row0 + ti.r0; ti.w_slice = jb.w_slice;
        ti.x_row0 = jb.x_row0;
        ti.ntok = ti.r0 < jb.R ? jb.ntok : 0; ti.R = jb.R; ti.y_stride = jb.y_stride;
        s_tiles[i] = ti;
    }
    const int ntiles = min(my_tiles, FT_MAX_TILES);
    uint8_t* stage_base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    volatile int* fail = &s_fail;

    if (tid == 0) {
        for (int s = 0; s < FT_STAGES; s++) {
            mbar_init(&bar_free[s], 1);
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_sf[s], 4);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&bar_done[b], 1);
            mbar_init(&bar_accfree[b], 4);
        }
        mbar_init(&bar_drain, 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(FT_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    // Every role walks the same sequence: tiles of the list that have tokens, their token passes ("units":
    // one accumulator buffer each, alternating), the K chunks of a pass (one pipeline stage each).
    uint32_t produced = 0;                                   // producer: chunks requested so far
    uint32_t issued_units = 0;                               // issuer: passes whose MMAs have been issued
    if (warp == 9) {
        // ================= producer =================
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < ntiles && ok; i++) {
                const Fp4Tile& ti = s_tiles[i];
                if (ti.ntok < 1) continue;
                const int ntok_cap = min(ti.ntok, FT_MAX_NT);
                const int variant = ntok_cap <= 16 ? 0 : ntok_cap <= 32 ? 1 : 2;
                const uint32_t stage_tx = FT_A_BYTES + FT_SFA_BYTES + (16u << variant) * (FT_KC_BYTES + 16u);
                for (int tb = 0; tb < ti.ntok && ok; tb += FT_MAX_NT)
                    for (int kc = 0; kc < nchunks; kc++, produced++) {
                        const uint32_t s = produced % FT_STAGES;
                        if (produced >= (uint32_t)FT_STAGES &&
                            !mbar_wait(&bar_free[s], ((produced / FT_STAGES) - 1) & 1, fail)) {
                            ok = false;
                            break;
                        }
                        const uint32_t dst = smem_u32(stage_base + s * FT_STAGE_BYTES);
                        mbar_expect_tx(&bar_full[s], stage_tx);
                        tma_load_3d(dst, &maps.w, kc * FT_KC_BYTES, ti.w_row, ti.w_slice, &bar_full[s]);
                        tma_load_2d(dst + FT_A_BYTES, &maps.x[variant], kc * FT_KC_BYTES, ti.x_row0 + tb, &bar_full[s]);
                        tma_load_3d(dst + FT_A_BYTES + FT_B_BYTES, &maps.ws, kc * 16, ti.ws_row, ti.w_slice, &bar_full[s]);
                        tma_load_2d(dst + FT_A_BYTES + FT_B_BYTES + FT_SFA_BYTES, &maps.xs[variant], kc * 16,
                                    ti.x_row0 + tb, &bar_full[s]);
                    }
            }
        }
        __syncwarp();
    } else if (warp == 8) {
        // ================= issuer =================
        const uint32_t lo0 = DESC_B_LO | ((smem_u32(stage_base) & 0x3ffffu) >> 4);
        uint32_t my = 0;
        bool ok = true;
        for (int i = 0; i < ntiles && ok; i++) {
            const Fp4Tile& ti = s_tiles[i];
            if (ti.ntok < 1) continue;
            for (int tb = 0; tb < ti.ntok && ok; tb += FT_MAX_NT, issued_units++) {
                const int NT = (min(FT_MAX_NT, ti.ntok - tb) + 15) & ~15;
                const uint32_t idesc = umma_idesc_fp4(128, NT);
                const uint32_t buf = issued_units & 1u;
                // the epilogue has read this buffer's previous contents
                if (issued_units >= 2u) ok = mbar_wait(&bar_accfree[buf], ((issued_units >> 1) - 1) & 1, fail);
                for (int kc = 0; kc < nchunks && ok; kc++, my++) {
                    const uint32_t s = my % FT_STAGES, ph = (my / FT_STAGES) & 1;
                    ok = mbar_wait(&bar_full[s], ph, fail);
                    if (ok) ok = mbar_wait(&bar_sf[s], ph, fail);
                    if (ok && lane == 0) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t alo = lo0 + s * (FT_STAGE_BYTES >> 4);
                        const uint32_t blo = alo + (FT_A_BYTES >> 4);
                        const uint32_t sf = tmem + FT_SF_BASE + s * FT_SF_STAGE;
#pragma unroll
                        for (int j = 0; j < 4; j++)      // K = 64 per MMA: 32 bytes further along the swizzled row
                            umma_fp4(tmem + buf * FT_MAX_NT, make_desc(alo + j * 2, DESC_B_HI),
                                     make_desc(blo + j * 2, DESC_B_HI), idesc, sf + 4 * j, sf + FT_SFB_OFF + 4 * j,
                                     (kc > 0 || j > 0) ? 1u : 0u);
                        umma_commit(&bar_free[s]);
                        if (kc == nchunks - 1) umma_commit(&bar_done[buf]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp < 4) {
        // ================= scale warps =================
        // The producer's copies leave the chunk's 16 scale bytes of every row in the stage (weights: 128 rows,
        // activations: the pass' token rows).  Lane l of every warp takes, per operand, the words of rows l,
        // l + 32, l + 64, l + 96 and stores them to its TMEM lane as 16 columns: column 4 j + c = K block j
        // (the MMA's K = 64) of row l + 32 c.
        const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
        uint32_t my = 0;
        bool ok = true;
        for (int i = 0; i < ntiles && ok; i++) {
            const Fp4Tile& ti = s_tiles[i];
            if (ti.ntok < 1) continue;
            for (int tb = 0; tb < ti.ntok && ok; tb += FT_MAX_NT)
                for (int kc = 0; kc < nchunks && ok; kc++, my++) {
                    const uint32_t s = my % FT_STAGES;
                    // landed copies also mean that the MMAs which last read this stage's scale columns are
                    // complete: the producer refilled the stage only after their commit
                    ok = mbar_wait(&bar_full[s], (my / FT_STAGES) & 1, fail);
                    if (ok) {
                        const uint4* sfa = (const uint4*)(stage_base + s * FT_STAGE_BYTES + FT_A_BYTES + FT_B_BYTES);
                        const uint4* sfb = sfa + FT_SFA_BYTES / 16;
                        uint32_t wa[16], wb[16];
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const uint4 v = sfa[lane + 32 * c];
                            wa[c] = v.x; wa[4 + c] = v.y; wa[8 + c] = v.z; wa[12 + c] = v.w;
                        }
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const uint4 v = c < FT_MAX_NT / 32 ? sfb[lane + 32 * c] : make_uint4(0u, 0u, 0u, 0u);
                            wb[c] = v.x; wb[4 + c] = v.y; wb[8 + c] = v.z; wb[12 + c] = v.w;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t sf = tlane + FT_SF_BASE + s * FT_SF_STAGE;
                        tmem_st16(sf, wa);
                        tmem_st16(sf + FT_SFB_OFF, wb);
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_sf[s]);   // always: the issuer never waits for a warp that gave up
                }
        }
    } else {
        // ================= epilogue warps (4-7: TMEM lane quarter warp - 4) =================
        const int q = warp - 4;
        const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16);
        uint32_t unit = 0;
        bool ok = true;
        for (int i = 0; i < ntiles && ok; i++) {
            const Fp4Tile& ti = s_tiles[i];
            if (ti.ntok < 1) continue;
            const int m = ti.r0 + q * 32 + lane;
            for (int tb = 0; tb < ti.ntok && ok; tb += FT_MAX_NT, unit++) {
                const int nt_real = min(FT_MAX_NT, ti.ntok - tb);
                const int NT = (nt_real + 15) & ~15;
                const uint32_t buf = unit & 1u;
                ok = mbar_wait(&bar_done[buf], (unit >> 1) & 1, fail);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int n0 = 0; n0 < NT; n0 += 32) {
                    uint32_t acc[32];
                    tmem_ld32(trow + buf * FT_MAX_NT + n0, acc);
#pragma unroll
                    for (int k = 0; k < 32; k++) {
                        const int n = n0 + k;
                        if (n < nt_real && m < ti.R)
                            ti.y[(size_t)(tb + n) * ti.y_stride + m] =
                                __fdiv_rn(__fmul_rn(__uint_as_float(acc[k]), ti.wg), ti.ig);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_accfree[buf]);
            }
        }
    }

    __syncthreads();
    if (*fail) {
        if (tid == 0 && a.status) atomicOr(a.status, SB_ERR_TIMEOUT);
        // wait (bounded, no early exit) for the copies requested and the MMAs issued before TMEM and shared
        // memory are released: every requested stage completes its copy (bar_full) ...
        if (warp == 9 && lane == 0) {
            int none = 0;
            for (uint32_t t = (produced > (uint32_t)FT_STAGES ? produced - FT_STAGES : 0); t < produced; t++)
                (void)mbar_wait(&bar_full[t % FT_STAGES], (t / FT_STAGES) & 1, &none);
        }
        __syncthreads();
        // ... and the tensor core has drained: one more commit tracks everything issued so far
        if (warp == 8 && lane == 0) {
            int none = 0;
            umma_commit(&bar_drain);
            (void)mbar_wait(&bar_drain, 0, &none);
        }
        __syncthreads();
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(FT_TMEM_COLS) : "memory");
    }
}

// Weight map of a layer's matrices: bytes [C/2] x rows x local experts (expert stride = the pool's), boxes of
// 128 bytes x 128 rows, 128-byte swizzle, zero fill past the last row.  Activation maps: [rows][C/2] packed
// codes, boxes of 128 bytes x 16 / 32 / 64 rows.
cudaError_t make_fp4_weight_map(CUtensorMap* out, const void* base, int C, int rows, int slices, size_t slice_stride) {
    TensorMapEncodeFn encode = nullptr;
    cudaError_t e = tensor_map_encoder(&encode);
    if (e != cudaSuccess) return e;
    if ((C % 256) != 0 || rows < 1 || slices < 1 || (slice_stride % 16) != 0 || ((uintptr_t)base % 16) != 0)
        return cudaErrorInvalidValue;
    cuuint64_t dims[3] = {(cuuint64_t)(C / 2), (cuuint64_t)rows, (cuuint64_t)slices};
    cuuint64_t strides[2] = {(cuuint64_t)(C / 2), (cuuint64_t)slice_stride};
    cuuint32_t box[3] = {(cuuint32_t)FT_KC_BYTES, 128u, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Scale maps: the same shapes with 16 bytes (one chunk's block scales) per row, unswizzled.
cudaError_t make_fp4_weight_scale_map(CUtensorMap* out, const void* base, int C, int rows, int slices, size_t slice_stride) {
    TensorMapEncodeFn encode = nullptr;
    cudaError_t e = tensor_map_encoder(&encode);
    if (e != cudaSuccess) return e;
    if ((C % 256) != 0 || rows < 1 || slices < 1 || (slice_stride % 16) != 0 || ((uintptr_t)base % 16) != 0)
        return cudaErrorInvalidValue;
    cuuint64_t dims[3] = {(cuuint64_t)(C / 16), (cuuint64_t)rows, (cuuint64_t)slices};
    cuuint64_t strides[2] = {(cuuint64_t)(C / 16), (cuuint64_t)slice_stride};
    cuuint32_t box[3] = {16u, 128u, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t make_fp4_act_scale_maps(CUtensorMap* out3, const void* base, int C, int rows) {
    TensorMapEncodeFn encode = nullptr;
    cudaError_t e = tensor_map_encoder(&encode);
    if (e != cudaSuccess) return e;
    if ((C % 256) != 0 || rows < 1 || ((uintptr_t)base % 16) != 0) return cudaErrorInvalidValue;
    for (int v = 0; v < 3; v++) {
        cuuint64_t dims[2] = {(cuuint64_t)(C / 16), (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)(C / 16)};
        cuuint32_t box[2] = {16u, (cuuint32_t)(16 << v)};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(&out3[v], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

cudaError_t make_fp4_act_maps(CUtensorMap* out3, const void* base, int C, int rows) {
    TensorMapEncodeFn encode = nullptr;
    cudaError_t e = tensor_map_encoder(&encode);
    if (e != cudaSuccess) return e;
    if ((C % 256) != 0 || rows < 1 || ((uintptr_t)base % 16) != 0) return cudaErrorInvalidValue;
    for (int v = 0; v < 3; v++) {
        cuuint64_t dims[2] = {(cuuint64_t)(C / 2), (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)(C / 2)};
        cuuint32_t box[2] = {(cuuint32_t)FT_KC_BYTES, (cuuint32_t)(16 << v)};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(&out3[v], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

cudaError_t launch_nvfp4_gemm_tc(const Fp4TcJob* jobs, int njobs, int R, int C, const Fp4TcMaps& maps, int* status,
                                 cudaStream_t stream) {
    if (njobs < 1 || R < 1) return cudaSuccess;
    if ((C % 256) != 0) return cudaErrorInvalidValue;
    cudaError_t e = ensure_dynamic_smem((const void*)nvfp4_gemm_tc_kernel, (size_t)FT_SMEM_BYTES);
    if (e != cudaSuccess) return e;
    int dev = 0, sms = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
        return e;
    Fp4TcArgs a;
    a.jobs = jobs; a.njobs = njobs; a.tiles_per_job = (R + 127) / 128; a.C = C; a.status = status;
    // persistent blocks, one per SM (the whole shared memory and all of TMEM each); more only when a block's
    // tile list would not hold its share
    const int total = njobs * a.tiles_per_job;
    const int grid = std::max(std::min(sms, total), (total + FT_MAX_TILES - 1) / FT_MAX_TILES);
    nvfp4_gemm_tc_kernel<<<grid, FT_THREADS, FT_SMEM_BYTES, stream>>>(a, maps);
    return cudaGetLastError();
}

}  // namespace sb
