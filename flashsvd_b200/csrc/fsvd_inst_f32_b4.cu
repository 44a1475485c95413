// Interpreter instantiations: element type float, batch width 4.
#define FSVD_INST_T float
#define FSVD_INST_DTYPE 1
#define FSVD_INST_NB 4
#define FSVD_INST_TABLE g_kernels_f32_b4
#include "fsvd_inst.cuh"
