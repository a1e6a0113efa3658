#define MC_T double
#include "smorph_inst.cuh"
