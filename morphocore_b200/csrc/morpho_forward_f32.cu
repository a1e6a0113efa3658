#define MC_T float
#include "morpho_forward_inst.cuh"
