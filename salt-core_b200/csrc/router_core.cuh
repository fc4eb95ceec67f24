// Device functions shared by the router, grouping and glue kernels: the in-order sums of the
// reference (serial by definition) and the softmax top-k of one row.
#pragma once
#include "bitmath.cuh"
#include "internal.h"

namespace sb {

static __device__ __forceinline__ void flag(int* status, int bit) {
    if (status) atomicOr(status, bit);
}

// Serial sum of squares of one row, in element order, as the reference does
// (gemma4.c:46-62, src/text_verify_cpu.c:642-655).  The squares are formed in
// parallel beforehand; one thread then runs the add chain over them, reading
// shared memory 16 bytes at a time so the loads run ahead of the 4-cycle adds.
static __device__ __forceinline__ float serial_sum(const float* sq, int n) {
    float ss = 0.0f;
    int i = 0;
    if ((((uintptr_t)sq) & 15) == 0) {
#pragma unroll 4
        for (; i + 8 <= n; i += 8) {
            const float4 a = *(const float4*)(sq + i);
            const float4 b = *(const float4*)(sq + i + 4);
            ss = __fadd_rn(ss, a.x); ss = __fadd_rn(ss, a.y); ss = __fadd_rn(ss, a.z); ss = __fadd_rn(ss, a.w);
            ss = __fadd_rn(ss, b.x); ss = __fadd_rn(ss, b.y); ss = __fadd_rn(ss, b.z); ss = __fadd_rn(ss, b.w);
        }
    }
    for (; i < n; i++) ss = __fadd_rn(ss, sq[i]);
    return ss;
}

// The same sum - S = 0; S = fl(S + sq[i]) for i = 0..n-1, bit for bit - by the whole
// block, for terms that are all finite and >= +0 (squares).
//
// While the running sum stays inside one binade, every partial sum is a multiple of that
// binade's ulp u, and fl(S + p) = S + (p rounded to a multiple of u): the roundings no
// longer depend on S, so the increments are integers that can be added in any order.
// Only two kinds of element need the real running sum: one whose addition may leave the
// binade, and a term exactly half-way between two multiples of u (its rounding goes to
// the even neighbour of the running sum).
//
//   1. an approximate prefix sum A (parallel float scan) PREDICTS the binade of the running
//      sum before and after every element;
//   2. an element is "certain" when A stays inside one binade across it, away from the
//      binade's ends, and the term is not a half-way case; all other elements are "serial
//      points".  Consecutive certain elements share one binade, so their integer increments
//      add up exactly (64-bit scan);
//   3. one thread walks the serial points in order: for the run of certain elements before
//      each point it CHECKS that the exact running sum really is in the predicted binade
//      and stays there (else it adds that run element by element), adds the run's integer
//      total, then performs the serial point's addition in floating point.
// The prediction only decides how much work is parallel; every step of the exact sum is
// either an integer identity that was checked or a real floating-point addition.  A typical
// row of a few thousand squares has ~20 serial points.  The first 64 terms (where the sum
// doubles every few steps) are added serially, and so is everything when the serial
// points exceed the list (half-way cases everywhere, subnormal sums).
//
// Needs blockDim.x * V >= n (V = elements per thread) and blockDim.x a multiple of 32.  scratch: POSSUM_SCRATCH words
// of shared memory.  Every thread of the block must call; all return the sum.
constexpr int POSSUM_V = 4, POSSUM_HEAD = 64, POSSUM_NS = 192;
constexpr int POSSUM_SCRATCH = 8 + 32 + 32 + 64 + 32 + POSSUM_NS * 4;

template <int V = POSSUM_V>
static __device__ float block_sum_nonneg(const float* sq, int n, uint32_t* scratch) {
    constexpr uint32_t ONE24 = 1u << 24, MARGIN = 1u << 13;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    float* fs = (float*)(scratch + 8);                 // [32] warp totals of the float scan
    float* flast = (float*)(scratch + 40);             // [32] last inclusive value of each warp
    unsigned long long* ws = (unsigned long long*)(scratch + 72);   // [32] warp totals of the integer scan
    uint32_t* wc = scratch + 136;                      // [32] warp counts of serial points
    uint32_t* sp_k = scratch + 168;                    // [NS] index of serial point
    uint32_t* sp_e = sp_k + POSSUM_NS;                 // [NS] predicted exponent field after it
    unsigned long long* sp_i = (unsigned long long*)(sp_e + POSSUM_NS);   // [NS] integer prefix at it
    const int base = tid * V;

    // ---- 1. approximate inclusive prefix sums
    float p[V], loc[V];
    float run = 0.0f;
#pragma unroll
    for (int j = 0; j < V; j++) {
        p[j] = base + j < n ? sq[base + j] : 0.0f;
        run += p[j];
        loc[j] = run;
    }
    float inc_s = run;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, inc_s, off);
        if (lane >= off) inc_s += t;
    }
    if (lane == 31) fs[warp] = inc_s;
    __syncthreads();
    float wt = lane < nw ? fs[lane] : 0.0f;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, wt, off);
        if (lane >= off) wt += t;
    }
    const float woff = warp ? __shfl_sync(0xffffffffu, wt, warp - 1) : 0.0f;
    const float incl_t = woff + inc_s;                 // this thread's last inclusive value
    if (lane == 31) flast[warp] = incl_t;
    __syncthreads();
    // value before this thread's first element = the previous thread's last inclusive value, bit for bit
    float before = __shfl_up_sync(0xffffffffu, incl_t, 1);
    if (lane == 0) before = warp ? flast[warp - 1] : 0.0f;

    // ---- 2. classify, integer increments
    unsigned long long isum = 0;        // increments of this thread's certain elements so far
    uint32_t nser = 0, ser_mask = 0;
    unsigned long long ser_i[V];
    uint32_t ser_e[V];
    float a_before = before;
#pragma unroll
    for (int j = 0; j < V; j++) {
        const int k = base + j;
        const float a_after = j == V - 1 ? incl_t : before + loc[j];
        const uint32_t bb = __float_as_uint(a_before), ab = __float_as_uint(a_after);
        ser_i[j] = 0; ser_e[j] = 0;
        if (k >= POSSUM_HEAD && k < n) {
            const uint32_t Eb = bb >> 23, Ea = ab >> 23;
            const uint32_t pb = __float_as_uint(p[j]);
            const uint32_t Ep = max(pb >> 23, 1u);
            const uint32_t m = (pb & 0x7fffffu) | ((pb >> 23) ? 0x800000u : 0u);
            bool certain = Eb == Ea && Eb >= 1u && Eb < 255u && (bb & 0x7fffffu) >= MARGIN &&
                           (ab & 0x7fffffu) <= 0x7fffffu - MARGIN && Ep <= Eb;
            uint32_t inc = 0;
            if (certain) {
                const uint32_t sh = Eb - Ep;
                if (sh == 0) {
                    inc = m;
                } else if (sh <= 24) {
                    const uint32_t rem = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
                    inc = (m >> sh) + (rem > half ? 1u : 0u);
                    certain = rem != half;
                }                                    // sh > 24: below half an ulp, adds nothing
            }
            if (certain) {
                isum += inc;
            } else {
                ser_mask |= 1u << j;
                ser_i[j] = isum;
                ser_e[j] = Ea;
                nser++;
            }
        }
        if (k == POSSUM_HEAD - 1) scratch[2] = ab >> 23;   // predicted exponent field after the serial head
        a_before = a_after;
    }

    // ---- 3. scan of (integer increments, serial point count)
    unsigned long long si = isum;
    uint32_t sc = nser;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const unsigned long long ti = __shfl_up_sync(0xffffffffu, si, off);
        const uint32_t tc = __shfl_up_sync(0xffffffffu, sc, off);
        if (lane >= off) { si += ti; sc += tc; }
    }
    if (lane == 31) { ws[warp] = si; wc[warp] = sc; }
    __syncthreads();
    unsigned long long wi = lane < nw ? ws[lane] : 0ull;
    uint32_t wcn = lane < nw ? wc[lane] : 0u;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const unsigned long long ti = __shfl_up_sync(0xffffffffu, wi, off);
        const uint32_t tc = __shfl_up_sync(0xffffffffu, wcn, off);
        if (lane >= off) { wi += ti; wcn += tc; }
    }
    const unsigned long long ioff = (warp ? __shfl_sync(0xffffffffu, wi, warp - 1) : 0ull) + (si - isum);
    uint32_t slot = (warp ? __shfl_sync(0xffffffffu, wcn, warp - 1) : 0u) + (sc - nser);
    const uint32_t ns = __shfl_sync(0xffffffffu, wcn, nw - 1);
    const unsigned long long itotal = __shfl_sync(0xffffffffu, wi, nw - 1);
#pragma unroll
    for (int j = 0; j < V; j++)
        if (ser_mask & (1u << j)) {
            if (slot < (uint32_t)POSSUM_NS) {
                sp_k[slot] = (uint32_t)(base + j);
                sp_e[slot] = ser_e[j];
                sp_i[slot] = ioff + ser_i[j];
            }
            slot++;
        }
    __syncthreads();

    // ---- 4. the exact walk, by warp 0: lane j fetches serial point j of a chunk of 32 (its index, integer
    // prefix, predicted exponent and the term itself), so that the chain below only waits for shuffles and
    // its own arithmetic; every lane runs the same chain on the same values
    if (warp == 0) {
        float S;
        if (ns > (uint32_t)POSSUM_NS || n <= POSSUM_HEAD) {
            S = lane == 0 ? serial_sum(sq, n) : 0.0f;
        } else {
            S = lane == 0 ? serial_sum(sq, POSSUM_HEAD) : 0.0f;
            S = __shfl_sync(0xffffffffu, S, 0);
            int prev = POSSUM_HEAD - 1;
            unsigned long long iprev = 0;
            uint32_t E = scratch[2];
            for (uint32_t base0 = 0; base0 <= ns; base0 += 32) {
                const uint32_t mine = base0 + (uint32_t)lane;
                const int my_idx = mine < ns ? (int)sp_k[mine] : n;
                const unsigned long long my_i = mine < ns ? sp_i[mine] : itotal;
                const uint32_t my_e = mine < ns ? sp_e[mine] : 0u;
                const float my_v = mine < ns ? sq[my_idx] : 0.0f;
                const int cnt = (int)min(32u, ns + 1u - base0);
                for (int j = 0; j < cnt; j++) {
                    const uint32_t jx = base0 + (uint32_t)j;
                    const int idx = __shfl_sync(0xffffffffu, my_idx, j);
                    const unsigned long long inow = __shfl_sync(0xffffffffu, my_i, j);
                    const uint32_t e_after = __shfl_sync(0xffffffffu, my_e, j);
                    const float term = __shfl_sync(0xffffffffu, my_v, j);
                    if (idx - 1 > prev) {
                        const unsigned long long tot = inow - iprev;
                        const uint32_t sb = __float_as_uint(S);
                        const uint32_t M = (sb & 0x7fffffu) | 0x800000u;
                        if ((sb >> 23) == E && tot < (unsigned long long)(ONE24 - M)) {
                            const uint32_t M2 = M + (uint32_t)tot;
                            S = __uint_as_float((E << 23) | (M2 & 0x7fffffu));
                        } else {
                            for (int i = prev + 1; i < idx; i++) S = __fadd_rn(S, sq[i]);   // prediction missed
                        }
                    }
                    if (jx < ns) {
                        S = __fadd_rn(S, term);
                        prev = idx;
                        iprev = inow;
                        E = e_after;
                    }
                }
            }
        }
        if (lane == 0) scratch[0] = __float_as_uint(S);
    }
    __syncthreads();
    return __uint_as_float(scratch[0]);
}

// Sum of the squares in sq[0..n) in element order.  `bad` = this thread saw a non-finite
// input; then (for any thread) the serial chain runs so that NaN / Inf propagate as in
// the reference.  Every thread of the block must call; all return the sum.
template <int V = POSSUM_V>
static __device__ __forceinline__ float ordered_sum_of_squares(const float* sq, int n, bool bad, uint32_t* scratch) {
    const bool serial = (int)blockDim.x * V < n || (blockDim.x & 31u);
    if (__syncthreads_or(bad) || serial) {   // the barrier also orders the writes of sq before the reads below
        if (threadIdx.x == 0) scratch[0] = __float_as_uint(serial_sum(sq, n));
        __syncthreads();
        return __uint_as_float(scratch[0]);
    }
    return block_sum_nonneg<V>(sq, n, scratch);
}

// Softmax top-k (gemma4.c:132-186) + ascending-expert ordering of the selected
// pairs (gemma4_text.c:8541-8550).  The insertion top-k with strict '>' equals
// ranking by (logit descending, expert ascending); the softmax denominator and
// the renormalisation sum are serial chains in expert / rank order.
//
// Executed by a group of `gsize` consecutive threads (ltid = index in group) on
// one row; every thread of the block must call it (block-wide barriers inside),
// groups without a row pass active = false.  sm = this group's scratch of
// 2E + 2*topk floats (16-byte aligned), sc = 4 floats of per-group scalars.
static __device__ __forceinline__ void topk_group(bool active, const float* lr, const float* per_expert_scale,
                                                  int32_t* sel_out, float* w_out, int E, int topk,
                                                  int sort_by_expert, int* status, float* sm, float* sc,
                                                  int ltid, int gsize) {
    float* sl = sm;                  // [E] logits
    float* se = sm + E;              // [E] exp(l - max)
    int* ssel = (int*)(sm + 2 * E);  // [topk]
    float* sw = sm + 2 * E + topk;   // [topk]
    int* s_bad = (int*)(sc + 3);
    if (ltid == 0) *s_bad = 0;
    __syncthreads();
    if (active)
        for (int e = ltid; e < E; e += gsize) {
            const float v = lr[e];
            sl[e] = v;
            if (!finite_f(v) || (per_expert_scale && !finite_f(per_expert_scale[e]))) *s_bad = 1;
        }
    __syncthreads();
    // the reference rejects non-finite logits before ranking (gemma4.c:149-152)
    const bool go = active && !*s_bad;
    if (go && ltid < 32) {
        float m = __int_as_float(0xff800000);
        for (int e = ltid; e < E; e += 32) m = fmaxf(m, sl[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (ltid == 0) sc[0] = m;
    }
    __syncthreads();
    if (go) {
        const float mx = sc[0];
        for (int e = ltid; e < E; e += gsize) {
            const float v = sl[e];
            se[e] = expf_exact(__fsub_rn(v, mx));
            int rank = 0;
            for (int o = 0; o < E; o++) {
                const float u = sl[o];
                rank += (u > v || (u == v && o < e)) ? 1 : 0;
            }
            if (rank < topk) ssel[rank] = e;
        }
    }
    __syncthreads();
    if (go && ltid == 0) {
        const float all = serial_sum(se, E);
        int bad = (!(all > 0.0f) || !finite_f(all)) ? 1 : 0;
        float selsum = 0.0f;
        for (int j = 0; j < topk; j++) {
            const float w = __fdiv_rn(se[ssel[j]], all);
            sw[j] = w;
            selsum = __fadd_rn(selsum, w);
        }
        sc[1] = selsum;
        if (!(selsum > 0.0f) || !finite_f(selsum)) bad = 1;
        if (bad) *s_bad = 1;
    }
    __syncthreads();
    if (go)
        for (int j = ltid; j < topk; j += gsize) {
            const int e = ssel[j];
            const float nrm = __fdiv_rn(sw[j], sc[1]);
            const float w = __fmul_rn(nrm, per_expert_scale ? per_expert_scale[e] : 1.0f);
            int pos = j;
            if (sort_by_expert) {
                pos = 0;
                for (int i = 0; i < topk; i++) pos += (ssel[i] < e) ? 1 : 0;
            }
            sel_out[pos] = e;
            w_out[pos] = w;
        }
    if (active && ltid == 0 && *s_bad) flag(status, SB_ERR_NONFINITE);
}

static __host__ __device__ __forceinline__ int topk_scratch_floats(int E, int topk) {
    return ((2 * E + 2 * topk + 3) & ~3) + 4;
}

}  // namespace sb
