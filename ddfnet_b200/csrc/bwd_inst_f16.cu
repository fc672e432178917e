// Filter-gradient streaming kernel instantiations for __half elements.
#define DDF_INST_T __half
#include "bwd_inst.inc"
