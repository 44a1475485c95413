// Interpreter instantiation: bf16 storage with int4-g128 factor tile streams.
#define FSVD_INST_T __nv_bfloat16
#define FSVD_INST_DTYPE 2
#define FSVD_INST_Q4 true
#define FSVD_INST_TABLE g_kernels_bf16_q4
#include "fsvd_inst.cuh"
