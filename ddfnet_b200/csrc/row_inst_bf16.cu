// Plane-ring kernel instantiations for __nv_bfloat16 elements.
#define DDF_INST_T __nv_bfloat16
#include "row_inst.inc"
