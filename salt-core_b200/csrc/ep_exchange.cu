// Expert-parallel exchange of the grouped expert outputs over peer memory (NVLink), one
// launch per layer, no host round trip and no library collective.
//
// Every rank owns a contiguous expert range and therefore a contiguous range of rows of the
// grouped output (the grouping is computed from a replicated router, so all ranks agree on
// it).  The kernel PUSHES its own rows into a landing buffer in every peer's memory, raises
// one flag per (source rank, block) there, waits for the peers' flags on its own landing
// buffer, and copies the rows it does not own into its grouped buffer.  Each row is produced
// by exactly one rank and copied unchanged, so the result does not depend on the number of
// ranks.  Remote data is only ever written into the consumer's memory and then read locally.
//
// Landing buffers alternate with the parity of an epoch counter that lives on the device and
// advances once per exchange, so a replayed CUDA graph needs no host-side state.  A peer may
// be one epoch ahead (it pushes epoch e + 1 into the other buffer while this rank still reads
// epoch e); it cannot be two ahead, because passing epoch e + 1 needs this rank's push of
// e + 1, which this rank issues after it has finished reading epoch e.
//
// Every wait is bounded: when a flag does not arrive within about a second the kernel sets
// SB_ERR_TIMEOUT in the status word, skips the copy and still advances the epoch.
#include "internal.h"

namespace sb {

struct EpHeader {
    int epoch;
    int done;
    int pad[62];
    int flags[EP_MAX_WORLD][EP_BLOCKS];
};
static_assert(sizeof(EpHeader) <= EP_HEADER_BYTES, "header area too small");

size_t ep_region_bytes(int rows_cap, int width) {
    return (size_t)EP_HEADER_BYTES + 2 * (size_t)rows_cap * width * sizeof(float);
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

constexpr int EP_SPIN_LIMIT = 1 << 21;   // polls of >= 0.3 us each
constexpr int EP_ROW_PIECES = 4;         // a row is moved by up to four blocks

__global__ void __launch_bounds__(EP_THREADS) ep_exchange_kernel(EpExchangeArgs a) {
    __shared__ int s_timed_out;
    EpHeader* own = (EpHeader*)a.region[a.rank];
    const int e = *(volatile const int*)&own->epoch;
    int lo = a.group_offsets[a.expert_begin], hi = a.group_offsets[a.expert_end];
    int total = a.group_offsets[a.n_experts];
    if (lo < 0 || lo > hi || hi > total || total > a.rows_cap) {
        // still raise the flags, so that no peer waits for this rank in vain
        if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(a.status, SB_ERR_CAPACITY);
        lo = hi = total = 0;
    }
    const int w4 = a.width >> 2;
    const int piece = (w4 + EP_ROW_PIECES - 1) / EP_ROW_PIECES;
    const size_t buf_off = (size_t)EP_HEADER_BYTES + (size_t)(e & 1) * a.rows_cap * a.width * sizeof(float);
    const int peers = a.world - 1;

    if (a.phase & EP_PHASE_PUSH) {
        const int items = (hi - lo) * peers * EP_ROW_PIECES;
        for (int it = blockIdx.x; it < items; it += gridDim.x) {
            const int pc = it % EP_ROW_PIECES;
            const int rp = it / EP_ROW_PIECES;
            const int pi = rp % peers;
            const int r = lo + rp / peers;
            const int p = pi + (pi >= a.rank ? 1 : 0);
            const float4* src = (const float4*)(a.grouped + (size_t)r * a.width);
            float4* dst = (float4*)(a.region[p] + buf_off) + (size_t)r * w4;
            const int end = min((pc + 1) * piece, w4);
            for (int i = pc * piece + threadIdx.x; i < end; i += blockDim.x) dst[i] = src[i];
        }
        __threadfence_system();
        __syncthreads();
        if ((int)threadIdx.x < a.world && (int)threadIdx.x != a.rank)
            st_release_sys(&((EpHeader*)a.region[threadIdx.x])->flags[a.rank][blockIdx.x], e + 1);
    }

    if (a.phase & EP_PHASE_PULL) {
        if (threadIdx.x == 0) s_timed_out = 0;
        __syncthreads();
        for (int f = threadIdx.x; f < peers * (int)gridDim.x; f += blockDim.x) {
            const int pi = f / (int)gridDim.x, b = f - pi * (int)gridDim.x;
            const int p = pi + (pi >= a.rank ? 1 : 0);
            const int* flag = &own->flags[p][b];
            int spins = 0;
            while (ld_acquire_sys(flag) - (e + 1) < 0) {
                if (++spins > EP_SPIN_LIMIT) {
                    s_timed_out = 1;
                    break;
                }
                __nanosleep(200);
            }
        }
        __threadfence_system();
        __syncthreads();
        if (s_timed_out) {
            if (threadIdx.x == 0) atomicOr(a.status, SB_ERR_TIMEOUT);
        } else {
            // rows below lo and from hi on came from the peers; the landing buffer was written by
            // another device, so it is read past the L1 cache
            const int nown = hi - lo;
            const int items = (total - nown) * EP_ROW_PIECES;
            for (int it = blockIdx.x; it < items; it += gridDim.x) {
                const int pc = it % EP_ROW_PIECES;
                const int q = it / EP_ROW_PIECES;
                const int r = q < lo ? q : q + nown;
                const float4* src = (const float4*)(a.region[a.rank] + buf_off) + (size_t)r * w4;
                float4* dst = (float4*)(a.grouped + (size_t)r * a.width);
                const int end = min((pc + 1) * piece, w4);
                for (int i = pc * piece + threadIdx.x; i < end; i += blockDim.x) dst[i] = __ldcg(src + i);
            }
        }
        // the last block to get here has seen every block read the epoch: advance it
        __syncthreads();
        if (threadIdx.x == 0) {
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

cudaError_t launch_ep_exchange(const EpExchangeArgs& a, cudaStream_t stream) {
    if (a.world < 2 || a.world > EP_MAX_WORLD || a.rank < 0 || a.rank >= a.world || (a.width & 3) || !a.grouped ||
        !(a.phase & (EP_PHASE_PUSH | EP_PHASE_PULL)))
        return cudaErrorInvalidValue;
    for (int p = 0; p < a.world; p++)
        if (!a.region[p]) return cudaErrorInvalidValue;
    ep_exchange_kernel<<<EP_BLOCKS, EP_THREADS, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace sb
