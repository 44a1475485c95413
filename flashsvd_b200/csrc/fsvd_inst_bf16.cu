// Interpreter instantiations: bf16 storage.
#define FSVD_INST_T __nv_bfloat16
#define FSVD_INST_DTYPE 0
#define FSVD_INST_TABLE g_kernels_bf16
#include "fsvd_inst.cuh"
