// Plane-ring kernel instantiations for __half elements.
#define DDF_INST_T __half
#include "row_inst.inc"
