// Interpreter instantiations: element type __nv_bfloat16, batch width 1.
#define FSVD_INST_T __nv_bfloat16
#define FSVD_INST_DTYPE 0
#define FSVD_INST_NB 1
#define FSVD_INST_TABLE g_kernels_bf16_b1
#include "fsvd_inst.cuh"
