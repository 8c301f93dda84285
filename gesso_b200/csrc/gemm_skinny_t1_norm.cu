// Skinny matrix product: the instantiations for up to 8 token rows, with the fused norm.
#include "gemm_skinny.cuh"

template int skinny_launch<1, true>(const void*, const float*, const float*, float, const void*, void*,
                                     const float*, int, int, int, int, void*, long long, const ConvEpi&,
                                     cudaStream_t);
