// Launcher table shared by the C-ABI translation unit and the kernel instantiation units.
#pragma once
#include <cuda_runtime.h>

#include "fsvd_stage.h"

typedef cudaError_t (*LaunchFn)(const fsvd::Stage* prog, const fsvd::SmallProgram* small,
                                int use_small, int nstages, fsvd::SyncState* sync, int xstride,
                                int part_bytes, int vec_bytes, unsigned long long* trace, int grid,
                                size_t smem,
                                cudaStream_t stream);

struct KernelEntry {
  int dtype;  // FSVD_DTYPE_*
  int nw;     // warps per CTA
  int depth;  // 16-byte loads in flight per lane
  LaunchFn fn;  // null terminates a table
};
