// The fused GEMV kernel for 8-bit codes.
#include "linear_lut_kernel.cuh"

template int fdk::launch_bits<8>(const fdk::LinearParams&, const void*, int, int, unsigned, cudaStream_t);
template int fdk::norm_fits_bits<8>(int, int, int*);
