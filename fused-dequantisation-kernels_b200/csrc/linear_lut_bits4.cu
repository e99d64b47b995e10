// The fused GEMV kernel for 4-bit codes.
#include "linear_lut_kernel.cuh"

template int fdk::launch_bits<4>(const fdk::LinearParams&, const void*, int, int, unsigned, cudaStream_t);
template int fdk::norm_fits_bits<4>(int, int, int*);
