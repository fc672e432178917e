// Plane-streaming kernel instantiations for float elements.
#define DDF_INST_T float
#include "stream_inst.inc"
