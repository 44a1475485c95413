// Interpreter instantiations: fp32 storage (parity mode).
#define FSVD_INST_T float
#define FSVD_INST_DTYPE 1
#define FSVD_INST_TABLE g_kernels_f32
#include "fsvd_inst.cuh"
