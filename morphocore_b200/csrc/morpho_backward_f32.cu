#define MC_T float
#include "morpho_backward_inst.cuh"
