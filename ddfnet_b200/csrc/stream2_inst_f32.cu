// Second-generation streaming kernel instantiations for float elements.
#define DDF_INST_T float
#include "stream2_inst.inc"
