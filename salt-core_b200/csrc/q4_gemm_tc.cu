// Grouped affine-Q4 expert GEMMs on the 5th-generation tensor cores (tcgen05 +
// TMEM) for prefill-sized token groups.  TOLERANCE path: operands are fp16
// (weights dequantised as q*s+b and rounded to fp16; activations rounded to
// fp16), accumulation is fp32 in TMEM.  The bit-exact kernels in q4_kernels.cu
// remain the reference-conformant path.
//
// Two precisions (template SPLIT):
//   single  one MMA per k-step, operands rounded to fp16 once: measured
//           max |err| / max(|ref|, row rms) about 2e-3 (5e-4 of the row maximum)
//   split   every operand is carried as hi + lo fp16 halves (lo = fp16(v - hi)) and
//           each k-step issues Xh*Wh + Xh*Wl + Xl*Wh: operand error ~2^-22, three
//           times the tensor work
//
// A unit of work = one 128-token pass of one tile of weight rows of one expert group.  A small kernel writes
// the layer's units into a work list from the grouped jobs (pass and tile counts are only known on the device);
// one resident block per SM draws units from it with an atomic counter until it is empty, its pipeline (input
// ring, converted stages, double-buffered accumulators) running on from one unit into the next.  Grids of one
// block per tile paid for every block's launch with 225 KB of shared memory, for the empty blocks of experts
// with fewer passes than the grid allowed, and for experts with several hundred tokens finishing last.
// The tokens of a pass (up to 128, stale rows above them) are the MMA's M side, read from shared
// memory as they arrive by TMA; 256 weight rows are the N side, dequantised into a K-major
// 128-byte-swizzled shared-memory stage.  The 256 rows are one tile of the down matrix, or - fused -
// 128 rows of gate followed by the same 128 rows of up: gate and up of a chunk are ONE instruction
// (M128 x N256 x K16), and the GeGLU pairs accumulator column c with 128 + c.  Accumulators: lane =
// token, column = weight row.  K advances in 64-column chunks = one quantisation group per row.
//   producer thread   draws the unit and passes it to the other roles through a shared-memory ring; packed
//                     nibbles (tiled TMA over the expert pool: bytes x rows x experts),
//                     the (scale << 16) | bias words of the rows (tiled TMA in blocks of four
//                     chunks where a table row is a multiple of 16 bytes, otherwise one bulk copy
//                     of the tile's whole table) and the tokens' fp16 activations (128-byte swizzle)
//                     into a ring of input slots, several chunks ahead
//   converter warps   two groups of eight warps on alternate chunks (thread = stage row): shared
//                     memory -> registers -> Q4 -> fp16 -> the stage; one mbarrier arrival per warp
//   issuer thread     tcgen05.mma.kind::f16 of every converted chunk, tcgen05.commit on the
//                     chunk's "done" barrier (frees the input slot and, some chunks later, the stage);
//                     polls the next chunk's barriers before issuing, so the answer arrives behind
//                     the MMAs
//   epilogue          all converter warps tcgen05.ld the accumulators after a unit (warp w: lane
//                     quarter w % 4, a quarter of the columns): GeGLU (fused gate/up) or plain store (down);
//                     the issuer is already filling the other accumulator buffer
// What was measured on the way here (B200, 1965 MHz): a register ring of global loads does not prefetch -
// waiting for the oldest load also waits for the younger ones that share its scoreboard, so every chunk paid
// a full memory latency (hence TMA); one mbarrier operation costs the issuing thread 100-190 cycles, so the
// one-thread issuer carries as few of them as possible; a tcgen05.mma costs the issuing thread about 100
// cycles for any N <= 128 (weights on M, in shared memory or dequantised straight into tensor memory with
// tcgen05.st, 128 rows per instruction: both forms ran 8 such instructions per fused chunk), so the weights sit
// on N, 256 rows per instruction.  What bounds this form is shared-memory traffic: about 110 KB per fused chunk
// (stage written once and read once, token tile read by every instruction) against 128 bytes per cycle.
// Column order inside every group of 8 K columns is permuted to [0,4,1,5,2,6,3,7] in
// BOTH operands (a contraction does not care): it is the order in which two masks
// and one shift peel half2 pairs out of a packed 32-bit word.
// Every mbarrier wait is bounded: on expiry the block raises a shared flag, records
// an error in the status word, every role leaves its loop, outstanding copies and
// MMAs are waited for (bounded), TMEM is freed and the block returns.
#include <cuda_fp16.h>

#include <stdlib.h>
#include <algorithm>
#include "internal.h"
#include "mbar.cuh"
#include "umma.cuh"
#include "q4_core.cuh"

namespace sb {

constexpr int TC_GROUP = 256;                // converter threads of one chunk (two groups take alternate chunks)
constexpr int TC_CONVERTERS = 2 * TC_GROUP;
constexpr int TC_THREADS = TC_CONVERTERS + 64;   // + issuer warp + producer warp
constexpr int TC_ISSUER_WARP = TC_CONVERTERS / 32, TC_PRODUCER_WARP = TC_ISSUER_WARP + 1;
constexpr int TC_KC = 64;                    // K columns per chunk
constexpr uint32_t TC_TMEM_COLS = 512;
constexpr int TC_PK_BYTES = 128 * TC_KC / 2; // packed chunk of 128 rows (one matrix' share of a fused stage)
constexpr int TC_TAB_BYTES = 128 * 16;       // scale | bias words of 128 rows x 4 chunks
constexpr int TC_MAX_NT = 128;
constexpr int TC_MAX_SLOTS = 8;
// Entries of the ring through which the producing thread passes work items to the other roles.  The producer is
// at most TC_MAX_SLOTS chunks, i.e. at most TC_MAX_SLOTS units, ahead of the last completed MMA, and no role is more
// than two units behind that, so 16 entries are never overrun and need no "free" barrier.
constexpr int TC_ITEM_RING = 16;
constexpr int TC_SMEM_BYTES = 225 * 1024;    // dynamic shared memory of every launch (one block per SM)

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

// half2 {lo, hi} from two floats (round to nearest even)
__device__ __forceinline__ uint32_t f16x2_from(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float f16_lo_to_f32(uint32_t h2) {
    float f;
    asm("{\n\t.reg .f16 l, h;\n\tmov.b32 {l, h}, %1;\n\tcvt.f32.f16 %0, l;\n\t}\n" : "=f"(f) : "r"(h2));
    return f;
}
__device__ __forceinline__ float f16_hi_to_f32(uint32_t h2) {
    float f;
    asm("{\n\t.reg .f16 l, h;\n\tmov.b32 {l, h}, %1;\n\tcvt.f32.f16 %0, h;\n\t}\n" : "=f"(f) : "r"(h2));
    return f;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Position of original column o (0..7) inside its group of 8 in the operands' K order
// [0,4,1,5,2,6,3,7].
__host__ __device__ __forceinline__ int tc_kpos(int o) { return ((o & 3) << 1) | (o >> 2); }

// Can q*s+b of this group be formed in fp16 arithmetic without loss?  s/16 and b must be
// exact fp16 values (bf16 has 8 significant bits) and 15*s+b must stay finite.
// bf16 exponent fields: s in [2^-13, 2^10), b zero or in [2^-17, 2^14).
__device__ __forceinline__ bool fp16_path_ok(uint32_t s_bits, uint32_t b_bits) {
    const uint32_t es = (s_bits >> 7) & 0xffu, eb = (b_bits >> 7) & 0xffu;
    const bool s_ok = es >= 114u && es <= 136u;
    const bool b_ok = (b_bits & 0x7fffu) == 0u || (eb >= 110u && eb <= 140u);
    return s_ok && b_ok;
}

// 32 consecutive Q4 elements of one row (16 packed bytes) -> 16 half2 words in the operands' K order
// (word 4 i + k holds columns (k, k + 4) of the i-th group of 8), fp16 arithmetic: a nibble masked in place
// under the exponent of 2^10 reads as 1024 + q (low nibble of a byte) or 1024 + 16 q (high nibble);
// subtracting 1024 is exact and one half2 fma with s (or s/16) forms q*s + b with a single rounding.
__device__ __forceinline__ void dequant_half_chunk_f16(const uint4& p, uint32_t s_bits, uint32_t b_bits,
                                                       uint32_t (&o)[16]) {
    const float s = bf16_bits_to_f32(s_bits), b = bf16_bits_to_f32(b_bits);
    const uint32_t s2 = f16x2_from(s, s), s2_16 = f16x2_from(s * 0.0625f, s * 0.0625f), b2 = f16x2_from(b, b);
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
    const uint32_t k1024 = 0x64006400u;
#pragma unroll
    for (int i = 0; i < 4; i++) {  // word i = 8 columns
        const uint32_t w0 = w[i], w1 = w[i] >> 8;
        uint32_t a0, a1, a2, a3;
        asm("lop3.b32 %0, %1, 0x000f000f, %2, 0xEA;" : "=r"(a0) : "r"(w0), "r"(k1024));   // cols (0,4)
        asm("lop3.b32 %0, %1, 0x00f000f0, %2, 0xEA;" : "=r"(a1) : "r"(w0), "r"(k1024));   // cols (1,5) * 16
        asm("lop3.b32 %0, %1, 0x000f000f, %2, 0xEA;" : "=r"(a2) : "r"(w1), "r"(k1024));   // cols (2,6)
        asm("lop3.b32 %0, %1, 0x00f000f0, %2, 0xEA;" : "=r"(a3) : "r"(w1), "r"(k1024));   // cols (3,7) * 16
        o[4 * i + 0] = hfma2(hsub2(a0, k1024), s2, b2);
        o[4 * i + 1] = hfma2(hsub2(a1, k1024), s2_16, b2);
        o[4 * i + 2] = hfma2(hsub2(a2, k1024), s2, b2);
        o[4 * i + 3] = hfma2(hsub2(a3, k1024), s2_16, b2);
    }
}

// The same 32 elements through fp32 (any scale), optionally with the fp16 residuals lo = fp16(v - hi).
template <bool SPLIT>
__device__ __forceinline__ void dequant_half_chunk_f32(const NibbleMagic& mg, const uint4& p, uint32_t s_bits,
                                                       uint32_t b_bits, uint32_t (&hi)[16], uint32_t (&lo)[16]) {
    const float s = bf16_bits_to_f32(s_bits), b = bf16_bits_to_f32(b_bits);
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
    const f32x2 ss = pack2(s, s), bb = pack2(b, b);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f32x2 q[4];
        nibbles4(w[i] & 0xffffu, mg, q[0], q[1]);
        nibbles4(w[i] >> 16, mg, q[2], q[3]);
        float v[8];
#pragma unroll
        for (int k = 0; k < 4; k++) unpack2(fma2(q[k], ss, bb), v[2 * k], v[2 * k + 1]);
#pragma unroll
        for (int k = 0; k < 4; k++) {   // half2 k holds columns (k, k + 4)
            const uint32_t h = f16x2_from(v[k], v[k + 4]);
            hi[4 * i + k] = h;
            if (SPLIT) lo[4 * i + k] = f16x2_from(v[k] - f16_lo_to_f32(h), v[k + 4] - f16_hi_to_f32(h));
        }
    }
}

// One unit of work: one token pass (up to 128 tokens) of one row tile of one expert group.
struct TcItem {
    int expert;   // local expert = slice of the weight maps
    int r0;       // first weight row of the tile (in each matrix)
    int grow;     // first grouped row of the pass
    int nt;       // tokens of the pass (1..128); 0 in a block's ring marks the end of the work
};

struct TcArgs {
    const TcItem* items;       // the launch's work list (written on the device)
    int* work;                 // [0] number of items, [1] next item to hand out, [2] most tokens of any item
    int R, C;                  // rows and columns of the weight matrices of this launch
    __half* out_h;             // fused: GeGLU output [grouped rows][R] fp16, columns in operand K order
    __half* out_l;             // its fp16 residual (split precision) or null
    float* out_f;              // plain: projection output [grouped rows][R] fp32
    int* status;
    const uint32_t* tables;    // (scale << 16) | bias words, [local expert][3 tensors][R * C/64]
    int tensor0;               // first tensor of the slot this launch reads (0: gate, then up; 2: down)
    int tab_tma;               // table rows are a multiple of 16 bytes: blocks of 4 groups come by tiled TMA
    int tab_bufs;              // untiled form: buffers for a tile's whole table (2, or 1 where shared memory is short)
};

// Bounded wait for two barriers at once: both polls are in flight together, so the pair costs one
// barrier round trip instead of two.
__device__ __forceinline__ bool mbar_wait2(uint64_t* bar_a, uint32_t par_a, uint64_t* bar_b, uint32_t par_b,
                                           volatile int* fail) {
    const uint32_t aa = smem_u32(bar_a), ab = smem_u32(bar_b);
    uint32_t done_a = 0, done_b = 0;
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
        uint32_t ra = 1, rb = 1;
        if (!done_a)
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}\n"
                : "=r"(ra)
                : "r"(aa), "r"(par_a)
                : "memory");
        if (!done_b)
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}\n"
                : "=r"(rb)
                : "r"(ab), "r"(par_b)
                : "memory");
        done_a |= ra;
        done_b |= rb;
        if (done_a && done_b) return true;
        if ((i & 255u) == 255u && *fail) return false;
    }
    *fail = 1;
    return false;
}

__device__ __forceinline__ uint4 lds_v4(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}

constexpr int TW_ROWS = 256;                        // rows of a converted stage
constexpr int TW_PK_BYTES = TW_ROWS * TC_KC / 2;    // packed chunk
constexpr int TW_TAB_BYTES = TW_ROWS * 16;          // table block (4 chunks)
constexpr int TW_B_BYTES = TW_ROWS * TC_KC * 2;     // converted chunk
constexpr int TW_TOK_BYTES = TC_MAX_NT * TC_KC * 2; // token tile
constexpr int TW_STAGES = 3;

template <bool FUSED, bool SPLIT>
__global__ void __launch_bounds__(TC_THREADS, 1)
q4_gemm_tc_kernel(const TcArgs a, const __grid_constant__ TcMaps maps, const __grid_constant__ TcWeightMaps wm) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_in[TC_MAX_SLOTS];    // input slot landed (TMA transaction bytes)
    __shared__ __align__(8) uint64_t bar_done[TC_MAX_SLOTS];  // the chunk's MMAs are complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t bar_full[TW_STAGES];     // stage converted (8 warp arrivals)
    // A unit = one token pass of one row tile.  Accumulators are double-buffered by unit parity (256 columns each).
    __shared__ __align__(8) uint64_t bar_acc[2];              // a unit's accumulators are final
    __shared__ __align__(8) uint64_t bar_epi[2];              // ... and have been read (16 warp arrivals)
    __shared__ __align__(8) uint64_t bar_tab[2];              // a tile's whole scale table landed (untiled form)
    __shared__ __align__(8) uint64_t bar_tabfree[2];          // ... and its last conversion is over (16 warp arrivals)
    // The block draws units from the launch's work list (one atomic per unit, by the producing thread, which
    // passes the item to the other roles through a small ring).
    __shared__ __align__(16) TcItem s_items[TC_ITEM_RING];
    __shared__ __align__(8) uint64_t bar_item[TC_ITEM_RING];  // ring entry published
    __shared__ uint32_t s_tmem;
    __shared__ int s_fail;

    constexpr int NMAT = FUSED ? 2 : 1;
    constexpr int RT = TW_ROWS / NMAT;                        // weight rows of a tile, per matrix
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int C = a.C, nchunks = C / TC_KC;
    constexpr int NPART = SPLIT ? 2 : 1;                     // hi (+ lo) copies of every operand tile
    constexpr int STAGES = SPLIT ? 2 : TW_STAGES;
    constexpr int STAGE_BYTES = NPART * TW_B_BYTES;          // [hi][lo] converted chunks
    const bool tab_tma = a.tab_tma != 0;
    // carve-up: converted stages | whole-tile table (untiled form) | input slots, each
    // [packed weights, 8 KB][table block, 4 KB (tiled form)][token tile(s): hi, lo]
    uint8_t* stage_base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // untiled tables: two buffers, so the next unit's table lands while this one is in use - or one where two do
    // not fit (the host decides): the producer then waits for the unit's last conversion
    const uint32_t TABBUF = (uint32_t)a.tab_bufs;
    const uint32_t tabw_bytes = tab_tma ? 0u : (((uint32_t)(TW_ROWS * nchunks * 4) + 1023u) & ~1023u);
    uint8_t* tabw = stage_base + STAGES * STAGE_BYTES;
    uint8_t* in_base = tabw + TABBUF * tabw_bytes;
    const uint32_t tok_off = TW_PK_BYTES + (tab_tma ? TW_TAB_BYTES : 0);
    // The MMA always reads 128 token rows: rows above the copied box (16, 32, 64 or 128 rows, by the pass' size)
    // are stale bytes of the slot's other part, of the next slot or of the pad behind the last one, and only reach
    // accumulator lanes nobody reads.
    // room of a token tile: the TMA box (16, 32, 64 or 128 rows) that holds the launch's largest pass
    const int nt_max = *(volatile const int*)&a.work[2];
    const uint32_t tok_room = nt_max <= 16 ? 2048u : nt_max <= 32 ? 4096u : nt_max <= 64 ? 8192u : (uint32_t)TW_TOK_BYTES;
    const uint32_t slot_bytes = tok_off + NPART * tok_room;
    const int avail = TC_SMEM_BYTES - 1024 - STAGES * STAGE_BYTES - (int)(TABBUF * tabw_bytes) - (TW_TOK_BYTES - (int)tok_room);
    const uint32_t NQ = (uint32_t)min(TC_MAX_SLOTS, avail / (int)slot_bytes);
    if ((int)NQ < STAGES) {                                   // the host checks the geometry; never expected
        if (tid == 0 && a.status) atomicOr(a.status, SB_ERR_INDEX);
        return;
    }
    volatile int* fail = &s_fail;

    if (tid == 0) {
        for (int s = 0; s < TC_MAX_SLOTS; s++) {
            mbar_init(&bar_in[s], 1);
            mbar_init(&bar_done[s], 1);
        }
        for (int s = 0; s < TW_STAGES; s++) mbar_init(&bar_full[s], TC_GROUP / 32);
        for (int s = 0; s < TC_ITEM_RING; s++) mbar_init(&bar_item[s], 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&bar_acc[s], 1);
            mbar_init(&bar_epi[s], TC_CONVERTERS / 32);
            mbar_init(&bar_tab[s], 1);
            mbar_init(&bar_tabfree[s], TC_CONVERTERS / 32);
        }
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    uint32_t it = 0;          // running chunk counter across token passes (every role counts the same chunks)
    uint32_t p_issued = 0;    // producer: chunks requested
    uint32_t i_committed = 0; // issuer: chunks committed
    uint32_t p_tabs = 0;      // producer: whole-tile table copies requested

    if (warp < TC_ISSUER_WARP) {
        // ================= converters, then the epilogue of every pass =================
        const uint32_t grp = (uint32_t)warp >> 3;
        const int crow = (warp & 7) * 32 + lane;                 // stage row
        const uint32_t b_off = (uint32_t)crow * 128;             // the row's 128-byte line in the 256 x 64 fp16 tile
        const uint32_t b_sw = (uint32_t)crow & 7;
        const NibbleMagic mg = load_nibble_magic();
        uint32_t cs = 0, cq = 0, cq_ph = 0, dq = 0, dq_ph = 0;
        bool alive = true;
        for (uint32_t unit = 0; alive && !*fail; unit++) {
            alive = __all_sync(0xffffffffu, mbar_wait(&bar_item[unit % TC_ITEM_RING], (unit / TC_ITEM_RING) & 1u, fail));
            if (!alive) break;
            const TcItem item = s_items[unit % TC_ITEM_RING];
            if (item.nt < 1) break;                                      // end of the work
            const int r0 = item.r0, rows_here = min(RT, a.R - r0);      // rows_here: a multiple of 64
            const int nt_real = item.nt;
            const uint32_t tbuf = unit % TABBUF;
            const uint8_t* tabt = tabw + tbuf * tabw_bytes;
            if (!tab_tma) alive = __all_sync(0xffffffffu, mbar_wait(&bar_tab[tbuf], (unit / TABBUF) & 1u, fail));
            if (!alive) break;
            for (int kc0 = 0; kc0 < nchunks; kc0 += 4) {
                uint32_t tw[4];             // table words of this thread's row for four chunks
#pragma unroll
                for (int d = 0; d < 4; d++) {
                    const int kc = kc0 + d;
                    if (kc >= nchunks) break;
                    uint8_t* st = stage_base + cs * STAGE_BYTES + b_off;
                    const uint8_t* slot = in_base + cq * slot_bytes;
                    const bool mine = (it & 1u) == grp;
                    if (!tab_tma && d == 0) {
#pragma unroll
                        for (int dd = 0; dd < 4; dd++)
                            tw[dd] = kc0 + dd < nchunks ? *(const uint32_t*)(tabt + (size_t)(crow * nchunks + kc0 + dd) * 4) : 0u;
                    }
                    if (mine) {
                        // the chunk's packed weights have landed, and the MMAs that last read this stage are complete
                        bool ok = it < (uint32_t)STAGES ? mbar_wait(&bar_in[cq], cq_ph, fail)
                                                        : mbar_wait2(&bar_in[cq], cq_ph, &bar_done[dq], dq_ph, fail);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) { alive = false; kc0 = nchunks; break; }
                        // tiled form: the table block of these four chunks rides in the slots of the block's first two
                        // chunks, one copy for each group (chunk and column parities agree: C is a multiple of 256)
                        if (tab_tma && d < 2) {
                            const uint4 t = lds_v4(slot + TW_PK_BYTES + crow * 16);
                            tw[0] = t.x; tw[1] = t.y; tw[2] = t.z; tw[3] = t.w;
                        }
                        const uint32_t s_bits = tw[d] >> 16, b_bits = tw[d] & 0xffffu;
                        const bool half_math = !SPLIT && fp16_path_ok(s_bits, b_bits);
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const uint4 pk = lds_v4(slot + crow * 32 + h * 16);
                            uint32_t o[16], lo[16];
                            if (half_math) dequant_half_chunk_f16(pk, s_bits, b_bits, o);
                            else dequant_half_chunk_f32<SPLIT>(mg, pk, s_bits, b_bits, o, lo);
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const uint32_t off = (((uint32_t)(h * 4 + i)) ^ b_sw) << 4;
                                *(uint4*)(st + off) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                                if (SPLIT)
                                    *(uint4*)(st + TW_B_BYTES + off) = make_uint4(lo[4 * i], lo[4 * i + 1], lo[4 * i + 2], lo[4 * i + 3]);
                            }
                        }
                        // generic-proxy writes -> visible to the tensor core (async proxy), then one arrival per warp
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bar_full[cs]);
                    }
                    if (it >= (uint32_t)STAGES && ++dq == NQ) { dq = 0; dq_ph ^= 1u; }
                    if (++cs == (uint32_t)STAGES) cs = 0;
                    if (++cq == NQ) { cq = 0; cq_ph ^= 1u; }
                    it++;
                }
            }
            // ---- epilogue of this pass: warp w reads lane quarter w % 4 (tokens) and a quarter of the columns
            if (!tab_tma && alive) {                                  // this unit's table is no longer read
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_tabfree[tbuf]);
            }
            if (alive && __all_sync(0xffffffffu, mbar_wait(&bar_acc[unit & 1u], (unit >> 1) & 1u, fail))) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int q = warp & 3;
                const int n = q * 32 + lane;                        // token of the pass
                const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16) + (unit & 1u) * TW_ROWS;
                if (q * 32 < nt_real) {                             // warp-uniform: the quarter holds tokens
                    if (FUSED) {
                        const int col = (warp >> 2) * 32;           // output columns col ... col + 31 of the tile
                        if (col < rows_here) {
                            uint32_t g[32], u[32];
                            tmem_ld32(trow + col, g);
                            tmem_ld32(trow + RT + col, u);
                            if (n < nt_real) {
                                const size_t o_off = (size_t)(item.grow + n) * a.R + r0 + col;
                                __half* dst = a.out_h + o_off;
#pragma unroll
                                for (int i8 = 0; i8 < 32; i8 += 8) {
                                    float o[8];
#pragma unroll
                                    for (int i = 0; i < 8; i++) {
                                        const float gv = __uint_as_float(g[i8 + i]), uv = __uint_as_float(u[i8 + i]);
                                        const float inner = 0.7978845608028654f * (gv + 0.044715f * gv * gv * gv);
                                        o[i] = 0.5f * gv * (1.0f + tanhf(inner)) * uv;
                                    }
                                    // the next GEMM's K order inside a group of 8: [0,4,1,5,2,6,3,7]
                                    const uint4 hv = make_uint4(f16x2_from(o[0], o[4]), f16x2_from(o[1], o[5]),
                                                                f16x2_from(o[2], o[6]), f16x2_from(o[3], o[7]));
                                    *(uint4*)(dst + i8) = hv;
                                    if (SPLIT) {
                                        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
                                        uint32_t lw[4];
#pragma unroll
                                        for (int kk = 0; kk < 4; kk++)
                                            lw[kk] = f16x2_from(o[kk] - f16_lo_to_f32(hw[kk]), o[kk + 4] - f16_hi_to_f32(hw[kk]));
                                        *(uint4*)(a.out_l + o_off + i8) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                                    }
                                }
                            }
                        }
                    } else {
#pragma unroll
                        for (int c0 = 0; c0 < 64; c0 += 32) {
                            const int col = (warp >> 2) * 64 + c0;
                            if (col >= rows_here) break;
                            uint32_t g[32];
                            tmem_ld32(trow + col, g);
                            if (n < nt_real) {
                                float* dst = a.out_f + (size_t)(item.grow + n) * a.R + r0 + col;
#pragma unroll
                                for (int i = 0; i < 32; i += 4)
                                    *(float4*)(dst + i) = make_float4(__uint_as_float(g[i]), __uint_as_float(g[i + 1]),
                                                                      __uint_as_float(g[i + 2]), __uint_as_float(g[i + 3]));
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_epi[unit & 1u]);
            }
        }
    } else if (warp == TC_ISSUER_WARP) {
        // ================= issuer (one thread) =================
        if (lane == 0) {
            const uint32_t w_lo0 = DESC_B_LO | ((smem_u32(stage_base) & 0x3ffffu) >> 4);
            const uint32_t t_lo0 = DESC_B_LO | ((smem_u32(in_base + tok_off) & 0x3ffffu) >> 4);
            uint32_t is = 0, is_ph = 0, iq = 0, iq_ph = 0;
            uint32_t ready = 0;
            bool ok = true;
            for (uint32_t unit = 0; ok && !*fail; unit++) {
                if (!mbar_wait(&bar_item[unit % TC_ITEM_RING], (unit / TC_ITEM_RING) & 1u, fail)) break;
                const TcItem item = s_items[unit % TC_ITEM_RING];
                if (item.nt < 1) break;                                  // end of the work
                const uint32_t idesc = umma_idesc_f16(128, FUSED ? TW_ROWS : min(RT, a.R - item.r0));
                // this unit's accumulator buffer was last used two units ago: those accumulators have been read
                if (unit >= 2 && !mbar_wait(&bar_epi[unit & 1u], ((unit >> 1) - 1) & 1u, fail)) { ok = false; break; }
                const uint32_t acc_base = tmem + (unit & 1u) * TW_ROWS;
                for (int kc = 0; kc < nchunks; kc++) {
                    // the converted weights of the stage, and the chunk's token tile: the tensor core reads it
                    // through the async proxy, so the issuing thread observes that barrier itself
                    if (!ready) ok = mbar_wait2(&bar_full[is], is_ph, &bar_in[iq], iq_ph, fail);
                    if (!ok) break;
                    // poll the next chunk's barriers now; the answer arrives behind this chunk's MMAs
                    uint32_t ns = is + 1, ns_ph = is_ph, nq = iq + 1, nq_ph = iq_ph;
                    if (ns == (uint32_t)STAGES) { ns = 0; ns_ph ^= 1u; }
                    if (nq == NQ) { nq = 0; nq_ph ^= 1u; }
                    uint32_t r_full, r_in;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                        "selp.u32 %0, 1, 0, p;\n\t}\n"
                        : "=r"(r_full)
                        : "r"(smem_u32(&bar_full[ns])), "r"(ns_ph)
                        : "memory");
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                        "selp.u32 %0, 1, 0, p;\n\t}\n"
                        : "=r"(r_in)
                        : "r"(smem_u32(&bar_in[nq])), "r"(nq_ph)
                        : "memory");
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t wlo = w_lo0 + is * (STAGE_BYTES >> 4);
                    const uint32_t tlo = t_lo0 + iq * (slot_bytes >> 4);
#pragma unroll
                    for (int j = 0; j < TC_KC / 16; j++) {
                        const uint64_t th = make_desc(tlo + j * 2, DESC_B_HI), wh = make_desc(wlo + j * 2, DESC_B_HI);
                        umma_f16(acc_base, th, wh, idesc, (kc > 0 || j > 0) ? 1u : 0u);
                        if (SPLIT) {
                            // x_hi * w_lo, then x_lo * w_hi
                            umma_f16(acc_base, th, make_desc(wlo + (TW_B_BYTES >> 4) + j * 2, DESC_B_HI), idesc, 1u);
                            umma_f16(acc_base, make_desc(tlo + (tok_room >> 4) + j * 2, DESC_B_HI), wh, idesc, 1u);
                        }
                    }
                    umma_commit(&bar_done[iq]);
                    if (kc == nchunks - 1) umma_commit(&bar_acc[unit & 1u]);
                    i_committed++;
                    ready = r_full & r_in;
                    is = ns; is_ph = ns_ph; iq = nq; iq_ph = nq_ph;
                }
            }
        }
    } else if (lane == 0) {
        // ================= producer (one thread) =================
        uint32_t pq = 0, pq_ph = 0;
        bool pok = true;
        const int n_items = *(volatile const int*)&a.work[0];
        for (uint32_t unit = 0; pok && !*fail; unit++) {
            const int idx = atomicAdd(&a.work[1], 1);
            TcItem item;
            if (idx < n_items) {
                const int4 v = *(const int4*)&a.items[idx];
                item.expert = v.x; item.r0 = v.y; item.grow = v.z; item.nt = v.w;
            } else {
                item.expert = 0; item.r0 = 0; item.grow = 0; item.nt = 0;
            }
            s_items[unit % TC_ITEM_RING] = item;
            mbar_arrive(&bar_item[unit % TC_ITEM_RING]);       // release: the entry is visible to who sees the phase
            if (item.nt < 1) break;
            const int r0 = item.r0, expert = item.expert;
            const int variant = item.nt <= 16 ? 0 : item.nt <= 32 ? 1 : item.nt <= 64 ? 2 : 3;
            const uint32_t tok_bytes = (16u << variant) * 128u;
            if (!tab_tma) {
                // the tile's whole table, into the buffer whose previous unit has been converted to the end
                const uint32_t tbuf = unit % TABBUF, round = unit / TABBUF;
                if (round > 0 && !mbar_wait(&bar_tabfree[tbuf], (round - 1) & 1u, fail)) break;
                const uint32_t bytes = (uint32_t)(min(RT, a.R - r0) * nchunks * 4);
                mbar_expect_tx(&bar_tab[tbuf], NMAT * bytes);
                p_tabs++;
#pragma unroll
                for (int m = 0; m < NMAT; m++) {
                    const uint32_t* src = a.tables + ((size_t)(expert * 3 + a.tensor0 + m) * a.R + r0) * nchunks;
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     smem_u32(tabw + tbuf * tabw_bytes + (size_t)m * RT * nchunks * 4)),
                                 "l"(src), "r"(bytes), "r"(smem_u32(&bar_tab[tbuf]))
                                 : "memory");
                }
            }
            for (int kc = 0; kc < nchunks; kc++) {
                // the slot's previous chunk has been consumed: its MMAs (which followed its conversion) are complete
                if (p_issued >= NQ && !mbar_wait(&bar_done[pq], pq_ph ^ 1u, fail)) { pok = false; break; }
                const uint32_t dst = smem_u32(in_base + pq * slot_bytes);
                const bool with_tab = tab_tma && (kc & 3) < 2;     // one copy for each converter group
                mbar_expect_tx(&bar_in[pq], TW_PK_BYTES + (with_tab ? TW_TAB_BYTES : 0) + NPART * tok_bytes);
                if (FUSED) {
                    // 128 rows of gate, then the same 128 rows of up
#pragma unroll
                    for (int m = 0; m < 2; m++) {
                        tma_load_3d(dst + m * TC_PK_BYTES, &wm.w[m], kc * 32, r0, expert, &bar_in[pq]);
                        if (with_tab)
                            tma_load_3d(dst + TW_PK_BYTES + m * TC_TAB_BYTES, &wm.t[m], (kc & ~3) * 4, r0, expert, &bar_in[pq]);
                    }
                } else {
                    tma_load_3d(dst, &wm.w256[2], kc * 32, r0, expert, &bar_in[pq]);
                    if (with_tab) tma_load_3d(dst + TW_PK_BYTES, &wm.t256[2], (kc & ~3) * 4, r0, expert, &bar_in[pq]);
                }
                tma_load_2d(dst + tok_off, &maps.hi[variant], kc * TC_KC, item.grow, &bar_in[pq]);
                if (SPLIT) tma_load_2d(dst + tok_off + tok_room, &maps.lo[variant], kc * TC_KC, item.grow, &bar_in[pq]);
                p_issued++;
                if (++pq == NQ) { pq = 0; pq_ph ^= 1u; }
            }
        }
    }
    if (*fail) {
        // wait (bounded, no early exit) for the copies and MMAs still in flight before shared memory and
        // TMEM are released
        int none = 0;
        if (warp == TC_PRODUCER_WARP && lane == 0) {
            if (p_tabs > 0) {       // the last table copy requested
                const uint32_t t = p_tabs - 1;
                (void)mbar_wait(&bar_tab[t % TABBUF], (t / TABBUF) & 1u, &none);
            }
            for (uint32_t t = (p_issued > NQ ? p_issued - NQ : 0); t < p_issued; t++)
                (void)mbar_wait(&bar_in[t % NQ], (t / NQ) & 1, &none);
        }
        if (warp == TC_ISSUER_WARP && lane == 0 && i_committed > 0)
            (void)mbar_wait(&bar_done[(i_committed - 1) % NQ], ((i_committed - 1) / NQ) & 1, &none);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && *fail && a.status) atomicOr(a.status, SB_ERR_TIMEOUT);
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

// x (fp32, token rows) -> fp16 rows in grouped order: xh[g] = fp16(x[g2c[g] / topk]),
// and (when xl != null) the residuals xl[g] = fp16(x - xh).  Columns inside every group
// of 8 are written in the operands' K order.
__global__ void __launch_bounds__(256)
gather_convert_kernel(const float* __restrict__ x, const int32_t* __restrict__ g2c, __half* __restrict__ xh,
                      __half* __restrict__ xl, int topk, int hidden) {
    const int g = blockIdx.y;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (d >= hidden) return;
    const float* src = x + (size_t)(g2c[g] / topk) * hidden + d;
    const float4 v0 = *(const float4*)src, v1 = *(const float4*)(src + 4);
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {   // half2 k holds columns (k, k + 4)
        hi[k] = f16x2_from(v[k], v[k + 4]);
        lo[k] = f16x2_from(v[k] - f16_lo_to_f32(hi[k]), v[k + 4] - f16_hi_to_f32(hi[k]));
    }
    *(uint4*)(xh + (size_t)g * hidden + d) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    if (xl) *(uint4*)(xl + (size_t)g * hidden + d) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

cudaError_t launch_gather_convert(const float* x, const int32_t* g2c, void* xh, void* xl, int jobs, int topk,
                                  int hidden, cudaStream_t stream) {
    if (jobs < 1) return cudaSuccess;
    if (hidden % 8) return cudaErrorInvalidValue;
    dim3 grid((hidden / 8 + 255) / 256, jobs);
    gather_convert_kernel<<<grid, 256, 0, stream>>>(x, g2c, (__half*)xh, (__half*)xl, topk, hidden);
    return cudaGetLastError();
}

cudaError_t tensor_map_encoder(TensorMapEncodeFn* out) {
    static TensorMapEncodeFn encode = nullptr;     // the entry point is process-wide, not per device
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (!fn || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        encode = (TensorMapEncodeFn)fn;
    }
    *out = encode;
    return cudaSuccess;
}

// Tensor maps over a [rows][cols] fp16 buffer (and its residual buffer): boxes of 64
// columns x 16 / 32 / 64 / 128 rows, 128-byte swizzle, zero fill past the last row.
cudaError_t make_tc_maps(TcMaps* out, const void* hi, const void* lo, int rows, int cols) {
    TensorMapEncodeFn encode = nullptr;
    {
        cudaError_t e = tensor_map_encoder(&encode);
        if (e != cudaSuccess) return e;
    }
    if ((cols % TC_KC) != 0 || rows < 1) return cudaErrorInvalidValue;
    for (int v = 0; v < 4; v++)
        for (int part = 0; part < 2; part++) {
            const void* base = part ? lo : hi;
            if (!base) return cudaErrorInvalidValue;
            cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
            cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
            cuuint32_t box[2] = {(cuuint32_t)TC_KC, (cuuint32_t)(16 << v)};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = encode(part ? &out->lo[v] : &out->hi[v], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                                const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        }
    return cudaSuccess;
}

// Tiled maps over a layer's expert pool, one per tensor of a slot (gate, up, down): packed nibbles as
// [C/2 bytes][R rows][experts] in boxes of one chunk (32 bytes) x 128 rows, and - where a table row is a multiple
// of 16 bytes (C a multiple of 256) - the (scale << 16) | bias words as [C/16 bytes][R rows][experts] in boxes of
// four chunks (16 bytes) x 128 rows.  Rows past R read as zero.
cudaError_t make_q4_tc_weight_maps(TcWeightMaps* out, const uint8_t* pool, size_t expert_stride, const uint32_t* tables,
                                   int hidden, int inter, int experts) {
    TensorMapEncodeFn encode = nullptr;
    {
        cudaError_t e = tensor_map_encoder(&encode);
        if (e != cudaSuccess) return e;
    }
    if ((hidden % TC_KC) != 0 || (inter % TC_KC) != 0 || experts < 1 || (expert_stride % 16) != 0 ||
        ((uintptr_t)pool % 16) != 0 || ((uintptr_t)tables % 16) != 0)
        return cudaErrorInvalidValue;
    const size_t elems = (size_t)hidden * inter;
    const size_t tensor_bytes = elems / 2 + 2 * (elems / 64 * 2);
    if ((tensor_bytes % 16) != 0) return cudaErrorInvalidValue;
    for (int k = 0; k < 3; k++) {
        const int R = k < 2 ? inter : hidden, C = k < 2 ? hidden : inter;
        {
            cuuint64_t dims[3] = {(cuuint64_t)(C / 2), (cuuint64_t)R, (cuuint64_t)experts};
            cuuint64_t strides[2] = {(cuuint64_t)(C / 2), (cuuint64_t)expert_stride};
            cuuint32_t box[3] = {(cuuint32_t)(TC_KC / 2), 128u, 1u};
            cuuint32_t estr[3] = {1, 1, 1};
            if ((C / 2) % 16) return cudaErrorInvalidValue;
            CUresult r = encode(&out->w[k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                                const_cast<uint8_t*>(pool + (size_t)k * tensor_bytes), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        }
        {
            cuuint64_t dims[3] = {(cuuint64_t)(C / 2), (cuuint64_t)R, (cuuint64_t)experts};
            cuuint64_t strides[2] = {(cuuint64_t)(C / 2), (cuuint64_t)expert_stride};
            cuuint32_t box[3] = {(cuuint32_t)(TC_KC / 2), (cuuint32_t)TW_ROWS, 1u};
            cuuint32_t estr[3] = {1, 1, 1};
            CUresult r = encode(&out->w256[k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                                const_cast<uint8_t*>(pool + (size_t)k * tensor_bytes), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        }
        out->tab_tma[k] = (C % 256) == 0 ? 1 : 0;
        if (out->tab_tma[k]) {
            cuuint64_t dims[3] = {(cuuint64_t)(C / 16), (cuuint64_t)R, (cuuint64_t)experts};
            cuuint64_t strides[2] = {(cuuint64_t)(C / 16), (cuuint64_t)(3 * (elems / 64) * 4)};
            cuuint32_t box[3] = {16u, 128u, 1u};
            cuuint32_t estr[3] = {1, 1, 1};
            CUresult r = encode(&out->t[k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                                const_cast<uint32_t*>(tables + (size_t)k * (elems / 64)), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
            box[1] = (cuuint32_t)TW_ROWS;
            r = encode(&out->t256[k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                       const_cast<uint32_t*>(tables + (size_t)k * (elems / 64)), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        } else {
            out->t[k] = out->w[k];   // never read
            out->t256[k] = out->w256[k];
        }
    }
    out->pool = pool;
    out->expert_stride = expert_stride;
    out->tables = tables;
    return cudaSuccess;
}

// Does the kernel's shared-memory carve-up hold at least as many input slots as stages for a tensor with C
// columns, in the widest token tile?  (The untiled table form keeps 256 rows x C/64 words resident.)
static bool tc_geometry_ok(int C, bool split, int tab_bufs) {
    const int npart = split ? 2 : 1, stages = split ? 2 : TW_STAGES;
    const bool tab_tma = (C % 256) == 0;
    const int tabw = tab_tma ? 0 : tab_bufs * ((TW_ROWS * (C / TC_KC) * 4 + 1023) & ~1023);
    const int slot = TW_PK_BYTES + (tab_tma ? TW_TAB_BYTES : 0) + npart * TW_TOK_BYTES;
    const int avail = TC_SMEM_BYTES - 1024 - stages * npart * TW_B_BYTES - tabw;
    return avail / slot >= stages;
}
// Buffers for the untiled tables of a tensor with C columns: 2 where they fit, else 1, 0 if the plan does not hold at all.
static int tc_table_buffers(int C, bool split) {
    return tc_geometry_ok(C, split, 2) ? 2 : (tc_geometry_ok(C, split, 1) ? 1 : 0);
}

bool q4_tc_supported(int hidden, int inter, bool split) {
    if (hidden < TC_KC || inter < TC_KC || (hidden % TC_KC) || (inter % TC_KC)) return false;
    return tc_table_buffers(hidden, split) > 0 && tc_table_buffers(inter, split) > 0;
}

template <bool FUSED, bool SPLIT>
static cudaError_t launch_tc(const TcArgs& a, const TcMaps& maps, const TcWeightMaps& wm, dim3 grid,
                                  cudaStream_t stream) {
    {
        cudaError_t e = ensure_dynamic_smem((const void*)q4_gemm_tc_kernel<FUSED, SPLIT>, (size_t)TC_SMEM_BYTES);
        if (e != cudaSuccess) return e;
    }
    q4_gemm_tc_kernel<FUSED, SPLIT><<<grid, TC_THREADS, TC_SMEM_BYTES, stream>>>(a, maps, wm);
    return cudaGetLastError();
}

// Work lists of a layer's two launches: for every expert group with tokens, every 128-token pass, every row
// tile one item (tiles of a pass adjacent, so neighbouring blocks share the pass' token rows in L2).  One block.
__global__ void __launch_bounds__(256)
q4_tc_work_list_kernel(const Q4Job* __restrict__ jobs, const int* __restrict__ njobs_dev, int njobs_max,
                       const float* y_base, int y_cols, const uint8_t* pool, size_t expert_stride, int nx_fused,
                       int nx_plain, TcItem* __restrict__ items_fused, TcItem* __restrict__ items_plain,
                       int* __restrict__ work) {
    extern __shared__ int s_list[];           // [njobs_max + 1] first pass of every job, then expert, first row, tokens
    int* s_base = s_list;
    int* s_expert = s_list + njobs_max + 1;
    int* s_g0 = s_expert + njobs_max;
    int* s_ntok = s_g0 + njobs_max;
    __shared__ int s_nt_max;
    const int njobs = njobs_dev ? min(*njobs_dev, njobs_max) : njobs_max;
    if (threadIdx.x == 0) s_nt_max = 0;
    __syncthreads();
    for (int j = threadIdx.x; j < njobs_max; j += blockDim.x) {
        int ntok = 0;
        if (j < njobs) {
            const Q4Job jb = jobs[j];
            ntok = max(jb.ntok, 0);
            s_expert[j] = (int)((size_t)(jb.vals - pool) / expert_stride);
            s_g0[j] = (int)((jb.y - y_base) / y_cols);
        }
        s_ntok[j] = ntok;
        s_base[j + 1] = (ntok + TC_MAX_NT - 1) / TC_MAX_NT;
        if (ntok > 0) atomicMax(&s_nt_max, min(ntok, TC_MAX_NT));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        s_base[0] = 0;
        for (int j = 0; j < njobs_max; j++) s_base[j + 1] += s_base[j];
        const int passes = s_base[njobs_max];
        work[0] = passes * nx_fused; work[1] = 0; work[2] = s_nt_max;
        work[4] = passes * nx_plain; work[5] = 0; work[6] = s_nt_max;
    }
    __syncthreads();
    const int nxt = nx_fused + nx_plain;
    for (int j = 0; j < njobs; j++) {
        const int base = s_base[j], np = s_base[j + 1] - base;
        for (int i = threadIdx.x; i < np * nxt; i += blockDim.x) {
            const int p = i / nxt, x = i - p * nxt;
            TcItem it;
            it.expert = s_expert[j]; it.grow = s_g0[j] + p * TC_MAX_NT; it.nt = min(TC_MAX_NT, s_ntok[j] - p * TC_MAX_NT);
            if (x < nx_fused) {
                it.r0 = x * (TW_ROWS / 2);
                items_fused[(size_t)(base + p) * nx_fused + x] = it;
            } else {
                it.r0 = (x - nx_fused) * TW_ROWS;
                items_plain[(size_t)(base + p) * nx_plain + (x - nx_fused)] = it;
            }
        }
    }
}

size_t q4_tc_work_items_max(int n_experts, int rows_total, int hidden, int inter) {
    const size_t passes = (size_t)n_experts + (size_t)rows_total / TC_MAX_NT + 1;
    return passes * (size_t)std::max((inter + 127) / 128, (hidden + TW_ROWS - 1) / TW_ROWS);
}

cudaError_t launch_q4_tc_work_list(const Q4Job* gateup_jobs, const int* njobs_dev, int njobs_max, const float* y_base,
                                   int y_cols, const TcWeightMaps& wm, int hidden, int inter, void* items_fused,
                                   void* items_plain, int* work, cudaStream_t stream) {
    if (njobs_max < 1) return cudaSuccess;
    q4_tc_work_list_kernel<<<1, 256, (size_t)(4 * njobs_max + 1) * sizeof(int), stream>>>(
        gateup_jobs, njobs_dev, njobs_max, y_base, y_cols, wm.pool, wm.expert_stride, (inter + 127) / 128,
        (hidden + TW_ROWS - 1) / TW_ROWS, (TcItem*)items_fused, (TcItem*)items_plain, work);
    return cudaGetLastError();
}

cudaError_t launch_q4_gemm_tc(bool fused, bool split, const void* items, int* work, const TcMaps& bmaps,
                              const TcWeightMaps& wm, void* out_h, void* out_l, float* out_f, int R, int C, int* status,
                              cudaStream_t stream) {
    TcArgs a;
    a.items = (const TcItem*)items; a.work = work;
    a.R = R; a.C = C;
    a.out_h = (__half*)out_h; a.out_l = (__half*)out_l; a.out_f = out_f; a.status = status;
    a.tables = wm.tables;
    a.tensor0 = fused ? 0 : 2;
    a.tab_tma = wm.tab_tma[fused ? 0 : 2];
    a.tab_bufs = tc_table_buffers(C, split);
    if (a.tab_bufs < 1) return cudaErrorInvalidValue;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    // one resident block per SM; each draws units (one token pass of one row tile) from the work list until it is empty
    dim3 grid((unsigned)sms, 1, 1);
    if (fused)
        return split ? launch_tc<true, true>(a, bmaps, wm, grid, stream) : launch_tc<true, false>(a, bmaps, wm, grid, stream);
    return split ? launch_tc<false, true>(a, bmaps, wm, grid, stream) : launch_tc<false, false>(a, bmaps, wm, grid, stream);
}

}  // namespace sb
