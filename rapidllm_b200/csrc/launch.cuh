// Kernel launch helper for the decode step: the same launch as <<< >>>, optionally marked for
// programmatic dependent launch so that consecutive kernels of a step overlap their heads and tails.
#pragma once
#include <cuda_runtime.h>

namespace rl {

// Set (per host thread) by the stack step around its launches.  Every kernel launched through
// launch_step() calls griddep_wait() before it touches anything an earlier kernel of the stream
// may have written.
extern thread_local bool g_step_overlap;
// Set at the start of a decode step: the step's first launch is a plain one, so it starts only when everything
// in front of it in the stream has completed.  Kernels further down the step may then read, before their
// griddep_wait(), data that only kernels of an earlier step (or of an earlier call) wrote.
extern thread_local bool g_step_first;

template <class... P, class... A>
inline cudaError_t launch_step(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_step_overlap && !g_step_first ? 1 : 0;
    g_step_first = false;
    return cudaLaunchKernelEx(&cfg, kernel, P(static_cast<A&&>(args))...);
}

}  // namespace rl
