// Single translation unit of libsvdq_b200.so: the device status word and the
// helpers in sm100.cuh are defined once for every kernel.
#include "tensormap.cu"
#include "quantize_generic.cu"
#include "quantize_fused.cu"
#include "quantize_stream.cu"
#include "gemm_w4a4.cu"
#include "capi.cu"
