// Programmatic dependent launch (sm_90+): a kernel launched with the programmatic
// stream-serialisation attribute may begin while its predecessor in the stream is still
// running.  Inside such a kernel
//   pdl_wait()               returns once the predecessor grid has completed and its
//                            writes are visible (a no-op for an ordinary launch);
//   pdl_launch_dependents()  lets the NEXT kernel in the stream begin.
// Rules used throughout this library:
//   * before pdl_wait() a kernel only READS, and only data that no kernel launched less
//     than two launches earlier writes (weights, tables written two or more kernels ago);
//   * pdl_launch_dependents() is called right AFTER pdl_wait(), so when kernel K starts,
//     kernel K-2 has completed: the early section of K overlaps only the tail of K-1;
//   * early reads of anything a kernel of this stream ever rewrites (job tables, routing
//     maps) go through L2 (__ldcg): before the wait this SM's L1 may still hold the lines of
//     an earlier pass - observed as wrong results until those loads bypassed L1.
// The pay-off is at decode sizes, where a layer is five dependent kernels of 10-17 us and
// the launch latency, the first dependent global loads and the weight prefetch of the next
// kernel otherwise sit on the critical path.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace sb {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// SALT_B200_PDL=0 in the environment turns the attribute off (ordinary stream order).
inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("SALT_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// Launch `kernel` so that it may overlap the tail of the previous kernel in `stream`.
// Only for kernels that call pdl_wait() before touching their predecessor's output.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace sb
