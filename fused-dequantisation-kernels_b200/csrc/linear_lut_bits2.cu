// The fused GEMV kernel for 2-bit codes.
#include "linear_lut_kernel.cuh"

template int fdk::launch_bits<2>(const fdk::LinearParams&, const void*, int, int, unsigned, cudaStream_t);
template int fdk::norm_fits_bits<2>(int, int, int*);
