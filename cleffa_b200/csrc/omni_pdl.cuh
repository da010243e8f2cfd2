// Programmatic dependent launch for the kernels of one MoE pass.
//
// The pass is a chain of seven kernels in one stream.  Launched the plain way, each kernel starts
// only after the previous one has drained and its memory is flushed, and pays its launch latency
// and prologue (barrier setup, tensor-memory allocation, descriptor prefetch) after that.  With
// the stream-serialization attribute below, a kernel's blocks may become resident as soon as
// every block of the previous kernel has either called dep_launch() or exited; they run their
// prologue and then block in dep_wait() until the previous kernel has completed and its writes
// are visible.
//
// Rules every kernel of the chain keeps:
//   * dep_wait() is executed by every thread before its first access to global memory and
//     before any exit path.  A block that left without waiting would let its grid count as
//     complete while an earlier grid still runs, and a later kernel could overtake that one.
//   * dep_launch() follows dep_wait() directly: by then the block is resident, so waiting
//     dependents can never hold resources a block of this grid still needs.
// Both instructions do nothing in a kernel that was launched without the attribute.
#pragma once
#include <cuda_runtime.h>

extern "C" int omni_dependent_launch_enabled(void);

__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t omni_launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                            Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = omni_dependent_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
