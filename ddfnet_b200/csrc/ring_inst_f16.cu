// Plane-ring kernel instantiations for __half elements.
#define DDF_INST_T __half
#include "ring_inst.inc"
