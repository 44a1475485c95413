// Interpreter instantiations: element type float, batch width 1.
#define FSVD_INST_T float
#define FSVD_INST_DTYPE 1
#define FSVD_INST_NB 1
#define FSVD_INST_TABLE g_kernels_f32_b1
#include "fsvd_inst.cuh"
