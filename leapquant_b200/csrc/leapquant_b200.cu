// Single translation unit of libleapquant_b200.so: the kernels share one device-side status word and a few host
// helpers, so they are compiled together (no relocatable device code needed).
#include "lq_abi.cu"
#include "lq_quant.cu"
#include "lq_flush.cu"
#include "lq_step.cu"
