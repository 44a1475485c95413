// Launcher table shared by the C-ABI translation unit and the kernel instantiation units.
#pragma once
#include <cuda_runtime.h>

#include "fsvd_stage.h"

struct LaunchArgs {
  const fsvd::Stage* prog;            // device-resident program, or null with `small`
  const fsvd::SmallProgram* small;    // by-value program (per-op launches)
  const unsigned char* maps;          // device-resident TMA descriptors, 2 x 128 bytes per stage
  const fsvd::SmallMaps* small_maps;  // by-value descriptors of a by-value program
  int nstages;
  fsvd::SyncState* sync;
  int xstride, part_bytes, vec_bytes, nslots;
  int slot_bytes;                     // bytes of one ring slot: kBoxBytes, or kQ4BoxBytes with int4 stages
  unsigned long long* trace;
  long long wait_limit;               // budget of every device-side wait, in SM clocks
  int grid;
  size_t smem;
  cudaStream_t stream;
};
typedef cudaError_t (*LaunchFn)(const LaunchArgs& a);

struct KernelEntry {
  int dtype;    // FSVD_DTYPE_*
  LaunchFn fn;  // null terminates a table
};
