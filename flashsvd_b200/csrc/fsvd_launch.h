// Launcher table shared by the C-ABI translation unit and the kernel instantiation units.
#pragma once
#include <cuda_runtime.h>

#include "fsvd_stage.h"

typedef cudaError_t (*LaunchFn)(const fsvd::Stage* prog, const fsvd::SmallProgram* small,
                                int use_small, int nstages, fsvd::SyncState* sync, int xstride,
                                unsigned long long* trace, int max_inflight, int grid,
                                size_t smem,
                                cudaStream_t stream);

struct KernelEntry {
  int dtype;  // FSVD_DTYPE_*
  int nb;     // compiled batch width
  int nw;     // warps per CTA
  int nd;     // ring slots per warp
  int bulk;   // 1: bulk-copy rings, 0: plain global loads
  LaunchFn fn;  // null terminates a table
};
