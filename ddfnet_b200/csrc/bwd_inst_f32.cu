// Filter-gradient streaming kernel instantiations for float elements.
#define DDF_INST_T float
#include "bwd_inst.inc"
