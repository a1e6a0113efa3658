#define MC_T double
#include "morpho_backward_inst.cuh"
