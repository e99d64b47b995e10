// Small device/host helpers shared by every translation unit of libfdk_b200.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/fdk_b200.h"
#include "fdk_layout.cuh"

namespace fdk {

// ---- status plumbing -------------------------------------------------------
void set_error_detail(const char* fmt, ...);
int cuda_status(cudaError_t e, const char* what);

#define FDK_CHECK_ARG(cond, code, ...)       \
  do {                                       \
    if (!(cond)) {                           \
      ::fdk::set_error_detail(__VA_ARGS__);  \
      return (code);                         \
    }                                        \
  } while (0)

#define FDK_CUDA(expr)                                         \
  do {                                                         \
    cudaError_t _e = (expr);                                   \
    if (_e != cudaSuccess) return ::fdk::cuda_status(_e, #expr); \
  } while (0)

inline bool bits_supported(int bits) { return bits == 1 || bits == 2 || bits == 3 || bits == 4 || bits == 8; }

struct DeviceInfo {
  int sm_count;
  int cc_major;
  int cc_minor;
  int max_smem_optin;
};
// Cached per device; returns a status code.
int device_info(DeviceInfo* out);

// ---- 16-bit float helpers --------------------------------------------------
template <bool FP16>
__device__ __forceinline__ float to_float(uint16_t v) {
  if constexpr (FP16) {
    return __half2float(__ushort_as_half(v));
  } else {
    return __uint_as_float(((uint32_t)v) << 16);
  }
}

template <bool FP16>
__device__ __forceinline__ uint16_t from_float(float f) {
  if constexpr (FP16) {
    return __half_as_ushort(__float2half_rn(f));
  } else {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  }
}

// Low / high 16-bit halves of a packed pair, as float.
template <bool FP16>
__device__ __forceinline__ float pair_lo(uint32_t w) {
  if constexpr (FP16) {
    return __half2float(__ushort_as_half((uint16_t)(w & 0xFFFFu)));
  } else {
    return __uint_as_float(w << 16);
  }
}
template <bool FP16>
__device__ __forceinline__ float pair_hi(uint32_t w) {
  if constexpr (FP16) {
    return __half2float(__ushort_as_half((uint16_t)(w >> 16)));
  } else {
    return __uint_as_float(w & 0xFFFF0000u);
  }
}

// ---- 3-bit helpers ----------------------------------------------------------
// Source format for 3 bits: one MSB-first bit stream per row, element j at
// stream bits [3j, 3j+3).  16 elements = 48 bits = 6 bytes.  The tiled buffer
// stores the same 6 bytes re-encoded as a little-endian 48-bit integer whose
// bits [6p, 6p+6) hold (code[2p] << 3) | code[2p+1], so that a pair index is
// one shift-and-mask away.
__host__ __device__ inline uint64_t encode3_pairs(const uint8_t* src6) {
  uint64_t be = 0;
  for (int i = 0; i < 6; ++i) be = (be << 8) | src6[i];
  uint64_t out = 0;
  for (int p = 0; p < 8; ++p) {
    uint64_t pair = (be >> (42 - 6 * p)) & 0x3F;  // codes 2p (high 3 bits) and 2p+1
    out |= pair << (6 * p);
  }
  return out;
}
__host__ __device__ inline void decode3_pairs(uint64_t enc, uint8_t* dst6) {
  uint64_t be = 0;
  for (int p = 0; p < 8; ++p) be |= ((enc >> (6 * p)) & 0x3F) << (42 - 6 * p);
  for (int i = 0; i < 6; ++i) dst6[i] = (uint8_t)(be >> (40 - 8 * i));
}

}  // namespace fdk
