// Offline repacker between the reference's packed tensors and the tiled buffer,
// plus the bit-exact dequantisers.  One-time / test-time work: simple grid-stride
// kernels bounded by HBM traffic (every byte is read and written once).
#include "fdk_common.cuh"

namespace fdk {
namespace {

// One thread per (padded row, padded 64-block, t in 0..3): moves the 2*bits
// bytes that hold 16 consecutive elements, and (t == 0) the block's scale.
__global__ void repack_kernel(const uint8_t* __restrict__ codes, const uint16_t* __restrict__ scale,
                              uint8_t* __restrict__ tiled, int n, int k, int bits, int block_size,
                              TiledDims d) {
  const int blocks_padded = d.k_slabs * d.ksb;
  const int rows_padded = d.row_tiles * kTileRows;
  const long long total = (long long)rows_padded * blocks_padded * 4;
  const int cb = 2 * bits;
  const int row_bytes = k / 8 * bits;
  const int blocks = k / kBlock;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int t = (int)(idx & 3);
    long long rest = idx >> 2;
    int blk = (int)(rest % blocks_padded);
    int row = (int)(rest / blocks_padded);
    bool live = row < n && blk < blocks;
    uint8_t buf[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) buf[i] = 0;
    if (live) {
      const uint8_t* src = codes + (size_t)row * row_bytes + (size_t)blk * (8 * bits) + t * cb;
      for (int i = 0; i < cb; ++i) buf[i] = src[i];
      if (bits == 3) {
        uint64_t enc = encode3_pairs(buf);
        for (int i = 0; i < 6; ++i) buf[i] = (uint8_t)(enc >> (8 * i));
      }
    }
    for (int i = 0; i < cb; ++i) tiled[tiled_code_offset(row, blk, t * cb + i, bits, d)] = buf[i];
    if (t == 0) {
      uint16_t s = 0;
      if (live) s = scale[(size_t)row * (k / block_size) + (size_t)blk * kBlock / block_size];
      *reinterpret_cast<uint16_t*>(tiled + tiled_scale_offset(row, blk, d)) = s;
    }
  }
}

__global__ void unpack_kernel(const uint8_t* __restrict__ tiled, uint8_t* __restrict__ codes,
                              uint16_t* __restrict__ scale, int n, int k, int bits, int block_size,
                              TiledDims d) {
  const int blocks = k / kBlock;
  const long long total = (long long)n * blocks * 4;
  const int cb = 2 * bits;
  const int row_bytes = k / 8 * bits;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int t = (int)(idx & 3);
    long long rest = idx >> 2;
    int blk = (int)(rest % blocks);
    int row = (int)(rest / blocks);
    uint8_t buf[16];
    for (int i = 0; i < cb; ++i) buf[i] = tiled[tiled_code_offset(row, blk, t * cb + i, bits, d)];
    if (bits == 3) {
      uint64_t enc = 0;
      for (int i = 0; i < 6; ++i) enc |= (uint64_t)buf[i] << (8 * i);
      decode3_pairs(enc, buf);
    }
    uint8_t* dst = codes + (size_t)row * row_bytes + (size_t)blk * (8 * bits) + t * cb;
    for (int i = 0; i < cb; ++i) dst[i] = buf[i];
    if (t == 0 && (blk * kBlock) % block_size == 0) {
      scale[(size_t)row * (k / block_size) + (size_t)blk * kBlock / block_size] =
          *reinterpret_cast<const uint16_t*>(tiled + tiled_scale_offset(row, blk, d));
    }
  }
}

// Decodes 8 consecutive elements [k0, k0+8) of one row from `bits * 1` source
// bytes (8 elements always fill whole bytes) and writes one 16-byte vector.
template <bool FP16>
__device__ __forceinline__ void dequant8(const uint8_t* src, const uint16_t* __restrict__ lut, int bits,
                                         float s, uint16_t* dst) {
  uint16_t vals[8];
  if (bits == 3) {
    uint32_t be = ((uint32_t)src[0] << 16) | ((uint32_t)src[1] << 8) | src[2];
#pragma unroll
    for (int j = 0; j < 8; ++j) vals[j] = lut[(be >> (21 - 3 * j)) & 7];
  } else {
    const int e = 8 / bits;  // elements per byte
    for (int b = 0; b < bits; ++b) {
      const uint16_t* row = lut + (size_t)src[b] * e;
      for (int j = 0; j < e; ++j) vals[b * e + j] = row[j];
    }
  }
  uint4 out;
  uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint16_t lo = from_float<FP16>(to_float<FP16>(vals[2 * j]) * s);
    uint16_t hi = from_float<FP16>(to_float<FP16>(vals[2 * j + 1]) * s);
    o[j] = (uint32_t)lo | ((uint32_t)hi << 16);
  }
  *reinterpret_cast<uint4*>(dst) = out;
}

template <bool FP16>
__global__ void dequantise_kernel(const uint8_t* __restrict__ codes, const uint16_t* __restrict__ lut,
                                  const uint16_t* __restrict__ scale, uint16_t* __restrict__ w, int n,
                                  int k, int bits, int block_size) {
  const long long total = (long long)n * (k / 8);
  const int row_bytes = k / 8 * bits;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int oct = (int)(idx % (k / 8));
    int row = (int)(idx / (k / 8));
    int k0 = oct * 8;
    float s = to_float<FP16>(scale[(size_t)row * (k / block_size) + k0 / block_size]);
    uint8_t src[8];
    const uint8_t* p = codes + (size_t)row * row_bytes + (size_t)oct * bits;
    for (int b = 0; b < bits; ++b) src[b] = p[b];
    dequant8<FP16>(src, lut, bits, s, w + (size_t)row * k + k0);
  }
}

template <bool FP16>
__global__ void dequantise_tiled_kernel(const uint8_t* __restrict__ tiled, const uint16_t* __restrict__ lut,
                                        uint16_t* __restrict__ w, int n, int k, int bits, TiledDims d) {
  // one thread per 16 consecutive elements (the unit the tiled layout keeps together)
  const long long total = (long long)n * (k / 16);
  const int cb = 2 * bits;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int h = (int)(idx % (k / 16));
    int row = (int)(idx / (k / 16));
    int blk = h >> 2, t = h & 3;
    uint8_t buf[16];
    for (int i = 0; i < cb; ++i) buf[i] = tiled[tiled_code_offset(row, blk, t * cb + i, bits, d)];
    if (bits == 3) {
      uint64_t enc = 0;
      for (int i = 0; i < 6; ++i) enc |= (uint64_t)buf[i] << (8 * i);
      decode3_pairs(enc, buf);
    }
    float s = to_float<FP16>(*reinterpret_cast<const uint16_t*>(tiled + tiled_scale_offset(row, blk, d)));
    uint16_t* dst = w + (size_t)row * k + (size_t)h * 16;
    dequant8<FP16>(buf, lut, bits, s, dst);
    dequant8<FP16>(buf + bits, lut, bits, s, dst + 8);
  }
}

int grid_for(long long total, int threads) {
  long long g = (total + threads - 1) / threads;
  if (g > 148LL * 32) g = 148LL * 32;
  if (g < 1) g = 1;
  return (int)g;
}

int check_shape(int n, int k, int bits, int block_size) {
  FDK_CHECK_ARG(n > 0 && k > 0, FDK_ERR_BAD_ARG, "n=%d, k=%d must be positive", n, k);
  FDK_CHECK_ARG(bits_supported(bits), FDK_ERR_SHAPE, "bits=%d not in {1,2,3,4,8}", bits);
  FDK_CHECK_ARG(k % kBlock == 0, FDK_ERR_SHAPE, "k=%d must be a multiple of 64", k);
  FDK_CHECK_ARG(block_size > 0 && block_size % kBlock == 0 && k % block_size == 0, FDK_ERR_SHAPE,
                "block_size=%d must be a multiple of 64 that divides k=%d", block_size, k);
  return FDK_OK;
}

}  // namespace
}  // namespace fdk

using namespace fdk;

extern "C" int fdk_tiled_size(int n, int k, int bits, size_t* bytes_host) {
  FDK_CHECK_ARG(bytes_host != nullptr, FDK_ERR_BAD_ARG, "bytes_host is null");
  if (int st = check_shape(n, k, bits, kBlock)) return st;
  *bytes_host = tiled_bytes(n, k, bits);
  return FDK_OK;
}

extern "C" int fdk_repack(const void* codes, const void* scale, int n, int k, int bits, int block_size,
                          void* tiled, void* stream) {
  if (int st = check_shape(n, k, bits, block_size)) return st;
  FDK_CHECK_ARG(codes && scale && tiled, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(((uintptr_t)tiled & 15) == 0 && ((uintptr_t)scale & 1) == 0, FDK_ERR_ALIGN,
                "tiled must be 16-byte aligned, scale 2-byte aligned");
  TiledDims d = tiled_dims(n, k, bits);
  long long total = (long long)d.row_tiles * kTileRows * d.k_slabs * d.ksb * 4;
  repack_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)codes, (const uint16_t*)scale, (uint8_t*)tiled, n, k, bits, block_size, d);
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}

extern "C" int fdk_unpack(const void* tiled, int n, int k, int bits, int block_size, void* codes,
                          void* scale, void* stream) {
  if (int st = check_shape(n, k, bits, block_size)) return st;
  FDK_CHECK_ARG(codes && scale && tiled, FDK_ERR_BAD_ARG, "null pointer");
  TiledDims d = tiled_dims(n, k, bits);
  long long total = (long long)n * (k / kBlock) * 4;
  unpack_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)tiled, (uint8_t*)codes, (uint16_t*)scale, n, k, bits, block_size, d);
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}

extern "C" int fdk_dequantise(const void* codes, const void* lut, const void* scale, int n, int k,
                              int bits, int block_size, int dtype, void* w_out, void* stream) {
  FDK_CHECK_ARG(n > 0 && k > 0, FDK_ERR_BAD_ARG, "n=%d, k=%d must be positive", n, k);
  FDK_CHECK_ARG(bits_supported(bits), FDK_ERR_SHAPE, "bits=%d not in {1,2,3,4,8}", bits);
  FDK_CHECK_ARG(k % 8 == 0 && block_size > 0 && k % block_size == 0 && block_size % 8 == 0, FDK_ERR_SHAPE,
                "k=%d must be a multiple of 8 and of block_size=%d (itself a multiple of 8)", k, block_size);
  FDK_CHECK_ARG(codes && lut && scale && w_out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(dtype == FDK_DTYPE_BF16 || dtype == FDK_DTYPE_F16, FDK_ERR_BAD_ARG, "dtype=%d", dtype);
  FDK_CHECK_ARG(((uintptr_t)w_out & 15) == 0, FDK_ERR_ALIGN, "w_out must be 16-byte aligned");
  long long total = (long long)n * (k / 8);
  int grid = grid_for(total, 256);
  if (dtype == FDK_DTYPE_F16) {
    dequantise_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)codes, (const uint16_t*)lut, (const uint16_t*)scale, (uint16_t*)w_out, n, k, bits, block_size);
  } else {
    dequantise_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)codes, (const uint16_t*)lut, (const uint16_t*)scale, (uint16_t*)w_out, n, k, bits, block_size);
  }
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}

extern "C" int fdk_dequantise_tiled(const void* tiled, const void* lut, int n, int k, int bits, int dtype,
                                    void* w_out, void* stream) {
  if (int st = check_shape(n, k, bits, kBlock)) return st;
  FDK_CHECK_ARG(tiled && lut && w_out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(dtype == FDK_DTYPE_BF16 || dtype == FDK_DTYPE_F16, FDK_ERR_BAD_ARG, "dtype=%d", dtype);
  FDK_CHECK_ARG(((uintptr_t)w_out & 15) == 0, FDK_ERR_ALIGN, "w_out must be 16-byte aligned");
  TiledDims d = tiled_dims(n, k, bits);
  long long total = (long long)n * (k / 16);
  int grid = grid_for(total, 256);
  if (dtype == FDK_DTYPE_F16) {
    dequantise_tiled_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)tiled, (const uint16_t*)lut, (uint16_t*)w_out, n, k, bits, d);
  } else {
    dequantise_tiled_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)tiled, (const uint16_t*)lut, (uint16_t*)w_out, n, k, bits, d);
  }
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}
