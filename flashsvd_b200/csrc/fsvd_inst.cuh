// Instantiates the interpreter for one element type; included by fsvd_inst_*.cu after defining
// FSVD_INST_T, FSVD_INST_DTYPE and FSVD_INST_TABLE.
#include "fsvd_kernel.cuh"
#include "fsvd_launch.h"

namespace {

template <typename T, int NW, int D>
cudaError_t launch_impl(const fsvd::Stage* prog, const fsvd::SmallProgram* small, int use_small,
                        int nstages, fsvd::SyncState* sync, int xstride, int part_bytes, int vec_bytes,
                        unsigned long long* trace, int grid, size_t smem, cudaStream_t stream) {
  auto kern = fsvd::fsvd_decode_kernel<T, NW, D>;
  static size_t attr_smem[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (smem > attr_smem[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_smem[dev] = smem;
  }
  static const fsvd::SmallProgram empty = {};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, prog, small ? *small : empty, use_small, nstages, sync,
                            xstride, part_bytes, vec_bytes, trace);
}

}  // namespace

#define FSVD_K(NW, D) {FSVD_INST_DTYPE, NW, D, &launch_impl<FSVD_INST_T, NW, D>}

extern const KernelEntry FSVD_INST_TABLE[] = {FSVD_K(8, 16), FSVD_K(8, 8), FSVD_K(8, 24),
                                              FSVD_K(16, 8), {0, 0, 0, nullptr}};
