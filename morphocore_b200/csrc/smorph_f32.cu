#define MC_T float
#include "smorph_inst.cuh"
