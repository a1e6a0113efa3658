#define MC_T double
#include "morpho_forward_inst.cuh"
