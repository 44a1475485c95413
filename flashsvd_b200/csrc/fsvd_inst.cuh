// Instantiates the interpreter for one element type; included by fsvd_inst_*.cu after defining
// FSVD_INST_T, FSVD_INST_DTYPE and FSVD_INST_TABLE (and FSVD_INST_Q4 = true for the instance that
// also understands int4 tile streams).
#ifndef FSVD_INST_Q4
#define FSVD_INST_Q4 false
#endif
#include <mutex>

#include "fsvd_kernel.cuh"
#include "fsvd_launch.h"

namespace {

template <typename T, bool Q4>
cudaError_t launch_impl(const LaunchArgs& a) {
  auto kern = fsvd::fsvd_decode_kernel<T, Q4>;
  // largest dynamic shared-memory size the kernel has been opted into, per device
  static size_t attr_smem[16] = {0};
  static std::mutex attr_mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  {
    std::lock_guard<std::mutex> lock(attr_mu);
    if (a.smem > attr_smem[dev]) {
      cudaError_t e =
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)a.smem);
      if (e != cudaSuccess) return e;
      attr_smem[dev] = a.smem;
    }
  }
  static const fsvd::SmallProgram empty_prog = {};
  static const fsvd::SmallMaps empty_maps = {};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.grid);
  cfg.blockDim = dim3(fsvd::kThreads);
  cfg.dynamicSmemBytes = a.smem;
  cfg.stream = a.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, a.prog, a.small ? *a.small : empty_prog, a.maps,
                            a.small_maps ? *a.small_maps : empty_maps, a.small ? 1 : 0, a.nstages,
                            a.sync, a.xstride, a.part_bytes, a.vec_bytes, a.nslots, a.slot_bytes, a.trace,
                            a.wait_limit);
}

}  // namespace

extern const KernelEntry FSVD_INST_TABLE[] = {{FSVD_INST_DTYPE, &launch_impl<FSVD_INST_T, FSVD_INST_Q4>}, {0, nullptr}};
