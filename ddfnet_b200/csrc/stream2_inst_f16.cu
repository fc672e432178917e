// Second-generation streaming kernel instantiations for __half elements.
#define DDF_INST_T __half
#include "stream2_inst.inc"
