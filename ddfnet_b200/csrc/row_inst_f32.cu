// Row kernel instantiations for float elements.
#define DDF_INST_T float
#include "row_inst.inc"
