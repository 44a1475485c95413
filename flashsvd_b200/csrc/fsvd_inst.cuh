// Instantiates the interpreter for one element type and batch width; included by fsvd_inst_*.cu
// after defining FSVD_INST_T, FSVD_INST_DTYPE, FSVD_INST_NB and FSVD_INST_TABLE.
#include "fsvd_kernel.cuh"
#include "fsvd_launch.h"

namespace {

template <typename T, int NB, int NW, int ND, bool BULK>
cudaError_t launch_impl(const fsvd::Stage* prog, const fsvd::SmallProgram* small, int use_small,
                        int nstages, fsvd::SyncState* sync, int xstride, unsigned long long* trace,
                        int max_inflight, int grid, size_t smem, cudaStream_t stream) {
  auto kern = fsvd::fsvd_decode_kernel<T, NB, NW, ND, BULK>;
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
                            xstride, trace, max_inflight);
}

}  // namespace

#define FSVD_K(NW, ND, BULK) \
  {FSVD_INST_DTYPE, FSVD_INST_NB, NW, ND, BULK, &launch_impl<FSVD_INST_T, FSVD_INST_NB, NW, ND, BULK != 0>}

extern const KernelEntry FSVD_INST_TABLE[] = {
    FSVD_K(16, 2, 1), FSVD_K(16, 3, 1), FSVD_K(8, 4, 1), FSVD_K(8, 6, 1),
    FSVD_K(16, 1, 0), FSVD_K(8, 1, 0),  {0, 0, 0, 0, 0, nullptr}};
