// Expert-parallel exchange of the grouped expert outputs over peer memory (NVLink), one
// launch per layer, no host round trip and no library collective.
//
// Every rank owns a contiguous expert range and therefore a contiguous range of rows of the
// grouped output (the grouping is computed from a replicated router, so all ranks agree on
// it).  The kernel PUSHES its own rows into a landing buffer in every peer's memory, then
// PULLS the rows it does not own out of its own landing buffer into its grouped buffer.  Each
// row is produced by exactly one rank and copied unchanged, so the result does not depend on
// the number of ranks.  Remote data is only ever written into the consumer's memory and read
// locally.
//
// Data and arrival flag travel together: a 16-byte slot holds two floats, each followed by
// the 32-bit sequence number of the exchange {d0, seq, d1, seq}, written with one store.  The
// reader polls the slot until both sequence numbers match; each {float, seq} pair is one naturally
// aligned 64-bit element of the store, so a matching number vouches for the float next to it.  No fence and no
// separate flag round trip sit between the producer's store and the consumer's load.
//
// Landing buffers alternate with the parity of an epoch counter that lives on the device and
// advances once per exchange (seq = epoch + 1), so a replayed CUDA graph needs no host-side
// state.  A peer may be one epoch ahead (it pushes epoch e + 1 into the other buffer while this
// rank still reads epoch e); it cannot be two ahead, because completing epoch e + 1 needs this
// rank's push of e + 1, which this rank issues after it has finished reading epoch e.
//
// Every wait is bounded (spin_limit polls of about half a microsecond): when a slot does not arrive
// the block gives up, the kernel sets SB_ERR_TIMEOUT in the status word and still advances the epoch.
// After a timeout the ranks' epochs may differ; ep_region_reset on every rank (all idle) starts over.
#include "internal.h"
#include "pdl.cuh"

namespace sb {

struct EpHeader {
    int epoch;
    int done;
};
static_assert(sizeof(EpHeader) <= EP_HEADER_BYTES, "header area too small");

size_t ep_region_bytes(int rows_cap, int width) {
    return (size_t)EP_HEADER_BYTES + 2 * (size_t)rows_cap * (width / 2) * 16;
}

// A slot is two 64-bit elements {float, seq}: the vector access is made of 64-bit element accesses, and
// a naturally aligned 64-bit element is written and read as a whole, which is all the protocol needs.
__device__ __forceinline__ uint4 ld_slot(const uint4* p) {
    unsigned long long a, b;
    asm volatile("ld.volatile.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
}
__device__ __forceinline__ void st_slot(uint4* p, uint4 v) {
    const unsigned long long a = (unsigned long long)v.x | ((unsigned long long)v.y << 32);
    const unsigned long long b = (unsigned long long)v.z | ((unsigned long long)v.w << 32);
    asm volatile("st.volatile.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

__global__ void __launch_bounds__(EP_THREADS) ep_exchange_kernel(EpExchangeArgs a) {
    __shared__ int s_timed_out;
    pdl_wait();
    pdl_launch_dependents();
    EpHeader* own = (EpHeader*)a.region[a.rank];
    const int e = *(volatile const int*)&own->epoch;
    const uint32_t seq = (uint32_t)e + 1u;
    int lo = a.group_offsets[a.expert_begin], hi = a.group_offsets[a.expert_end];
    int total = a.group_offsets[a.n_experts];
    if (lo < 0 || lo > hi || hi > total || total > a.rows_cap) {
        if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(a.status, SB_ERR_CAPACITY);
        lo = hi = total = 0;
    }
    const int slots = a.width >> 1;              // 16-byte slots per row
    const size_t buf_off = (size_t)EP_HEADER_BYTES + (size_t)(e & 1) * a.rows_cap * slots * 16;
    const int stride = gridDim.x * blockDim.x;
    const int first = blockIdx.x * blockDim.x + threadIdx.x;

    if (a.phase & EP_PHASE_PUSH) {
        const int n = (hi - lo) * slots;
        for (int i = first; i < n; i += stride) {
            const int rr = i / slots, c = i - rr * slots;
            const int r = lo + rr;
            const float2 v = *(const float2*)(a.grouped + (size_t)r * a.width + 2 * c);
            const uint4 w = make_uint4(__float_as_uint(v.x), seq, __float_as_uint(v.y), seq);
            const size_t at = buf_off + ((size_t)r * slots + c) * 16;
            for (int p = 0; p < a.world; p++)
                if (p != a.rank) st_slot((uint4*)(a.region[p] + at), w);
        }
    }

    if (a.phase & EP_PHASE_PULL) {
        if (threadIdx.x == 0) s_timed_out = 0;
        __syncthreads();
        const int nown = hi - lo;
        const int n = (total - nown) * slots;
        for (int i = first; i < n; i += stride) {
            const int q = i / slots, c = i - q * slots;
            const int r = q < lo ? q : q + nown;
            const uint4* src = (const uint4*)(a.region[a.rank] + buf_off) + (size_t)r * slots + c;
            uint4 w = ld_slot(src);
            int spins = 0;
            while (w.y != seq || w.w != seq) {
                if (++spins > a.spin_limit || *(volatile int*)&s_timed_out) {
                    s_timed_out = 1;
                    break;
                }
                if (spins > 8) __nanosleep(100);
                w = ld_slot(src);
            }
            if (w.y == seq && w.w == seq)
                *(float2*)(a.grouped + (size_t)r * a.width + 2 * c) = make_float2(__uint_as_float(w.x), __uint_as_float(w.z));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            if (s_timed_out) atomicOr(a.status, SB_ERR_TIMEOUT);
            // the last block to get here has seen every block read the epoch: advance it
            __threadfence();
            const int prev = atomicAdd(&own->done, 1);
            if (prev == (int)gridDim.x - 1) {
                own->done = 0;
                __threadfence();
                *(volatile int*)&own->epoch = e + 1;
            }
        }
    }
}

cudaError_t launch_ep_exchange(const EpExchangeArgs& a, int rows, cudaStream_t stream) {
    if (a.spin_limit < 1 || a.world < 2 || a.world > EP_MAX_WORLD || a.rank < 0 || a.rank >= a.world || (a.width & 1) || !a.grouped ||
        !(a.phase & (EP_PHASE_PUSH | EP_PHASE_PULL)) || rows < 1)
        return cudaErrorInvalidValue;
    for (int p = 0; p < a.world; p++)
        if (!a.region[p]) return cudaErrorInvalidValue;
    // two slots per thread when the whole batch fits one wave, never more than one block per SM
    const long long work = (long long)rows * (a.width >> 1);
    long long blocks = (work + 2 * EP_THREADS - 1) / (2 * EP_THREADS);
    blocks = blocks < 8 ? 8 : (blocks > 148 ? 148 : blocks);
    return launch_pdl(ep_exchange_kernel, dim3((unsigned)blocks), dim3(EP_THREADS), 0, stream, a);
}

}  // namespace sb
