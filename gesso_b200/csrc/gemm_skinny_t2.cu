// Skinny matrix product: the instantiations for 9 to 16 token rows, without the fused norm.
#include "gemm_skinny.cuh"

template int skinny_launch<2, false>(const void*, const float*, const float*, float, const void*, void*,
                                     const float*, int, int, int, int, void*, long long, const ConvEpi&,
                                     cudaStream_t);
