// Glue kernels of the custom-llama decode step, around the quantised projections:
// RMSNorm fused with the residual add, rotary embedding fused with the KV-cache append,
// SiLU(gate) * up.  All are one pass over a [batch, width] bf16 activation (a few KB to a few
// MB), bound by launch latency at small batch and by HBM at large batch; they exist to
// replace ~10 framework launches per layer by 3.  The reference gets this arithmetic from
// transformers' LlamaForCausalLM (src/fdk/models.py:238-251); the formulas below follow that
// model's definition (RMSNorm in fp32 with the weight applied after the cast, rotate-half
// rotary embedding with cos/sin rounded to the activation type).
#include "fdk_common.cuh"

namespace fdk {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out[row] = weight * bf16(h[row] * rsqrt(mean(h[row]^2) + eps)), with h += delta first when
// delta is given (h is the residual stream, updated in place).
__global__ void rmsnorm_kernel(uint16_t* __restrict__ h, const uint16_t* __restrict__ delta,
                               const uint16_t* __restrict__ weight, uint16_t* __restrict__ out, int width,
                               float eps) {
  extern __shared__ float row_cache[];  // width floats
  __shared__ float partial[32];
  const int row = blockIdx.x;
  uint16_t* hr = h + (size_t)row * width;
  const uint16_t* dr = delta ? delta + (size_t)row * width : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
    uint4 hv = *reinterpret_cast<const uint4*>(hr + i);
    uint32_t* hw = reinterpret_cast<uint32_t*>(&hv);
    if (dr) {
      uint4 dv = *reinterpret_cast<const uint4*>(dr + i);
      const uint32_t* dw = reinterpret_cast<const uint32_t*>(&dv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the residual add is a bf16 add, as in the framework model
        uint16_t lo = from_float<false>(pair_lo<false>(hw[j]) + pair_lo<false>(dw[j]));
        uint16_t hi = from_float<false>(pair_hi<false>(hw[j]) + pair_hi<false>(dw[j]));
        hw[j] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      *reinterpret_cast<uint4*>(hr + i) = hv;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a = pair_lo<false>(hw[j]), b = pair_hi<false>(hw[j]);
      row_cache[i + 2 * j] = a;
      row_cache[i + 2 * j + 1] = b;
      ss += a * a + b * b;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) partial[0] = rsqrtf(v / width + eps);
  }
  __syncthreads();
  const float inv = partial[0];
  uint16_t* orow = out + (size_t)row * width;
  for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(weight + i);
    const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wv);
    uint4 ov;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a = to_float<false>(from_float<false>(row_cache[i + 2 * j] * inv)) * pair_lo<false>(ww[j]);
      float b = to_float<false>(from_float<false>(row_cache[i + 2 * j + 1] * inv)) * pair_hi<false>(ww[j]);
      ow[j] = (uint32_t)from_float<false>(a) | ((uint32_t)from_float<false>(b) << 16);
    }
    *reinterpret_cast<uint4*>(orow + i) = ov;
  }
}

// One CTA (64 threads) per (batch row, head of the fused q|k|v projection); head_dim = 128.
// q heads: rotated, written to q_out.  k heads: rotated, written to the cache at *pos.
// v heads: copied to the cache at *pos.
__global__ void rope_append_kernel(const uint16_t* __restrict__ qkv, const long long* __restrict__ pos_ptr,
                                   uint16_t* __restrict__ q_out, uint16_t* __restrict__ k_cache,
                                   uint16_t* __restrict__ v_cache, int q_heads, int kv_heads, int max_len,
                                   float theta) {
  const int row = blockIdx.y, head = blockIdx.x, i = threadIdx.x;  // i in 0..63: the pair (i, i + 64)
  const long long pos = *pos_ptr;
  const int heads_total = q_heads + 2 * kv_heads;
  const uint16_t* src = qkv + ((size_t)row * heads_total + head) * 128;
  if (head >= q_heads + kv_heads) {  // v
    const int kvh = head - q_heads - kv_heads;
    uint16_t* dst = v_cache + (((size_t)row * kv_heads + kvh) * max_len + pos) * 128;
    dst[i] = src[i];
    dst[i + 64] = src[i + 64];
    return;
  }
  const float inv_freq = powf(theta, -(float)(2 * i) / 128.f);
  const float angle = (float)pos * inv_freq;
  const float c = to_float<false>(from_float<false>(cosf(angle)));
  const float s = to_float<false>(from_float<false>(sinf(angle)));
  const float x0 = to_float<false>(src[i]), x1 = to_float<false>(src[i + 64]);
  // out = x * cos + rotate_half(x) * sin, each product and the sum rounded to bf16
  auto r = [](float v) { return to_float<false>(from_float<false>(v)); };
  const uint16_t o0 = from_float<false>(r(x0 * c) + r(-x1 * s));
  const uint16_t o1 = from_float<false>(r(x1 * c) + r(x0 * s));
  uint16_t* dst;
  if (head < q_heads) {
    dst = q_out + ((size_t)row * q_heads + head) * 128;
  } else {
    dst = k_cache + (((size_t)row * kv_heads + (head - q_heads)) * max_len + pos) * 128;
  }
  dst[i] = o0;
  dst[i + 64] = o1;
}

// out[row, j] = silu(gate_up[row, j]) * gate_up[row, width + j]
__global__ void silu_mul_kernel(const uint16_t* __restrict__ gate_up, uint16_t* __restrict__ out, int width,
                                long long total) {
  for (long long idx = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8; idx < total;
       idx += (long long)gridDim.x * blockDim.x * 8) {
    const long long row = idx / width;
    const int col = (int)(idx - row * width);
    const uint16_t* g = gate_up + row * 2 * width + col;
    uint4 gv = *reinterpret_cast<const uint4*>(g);
    uint4 uv = *reinterpret_cast<const uint4*>(g + width);
    const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gv);
    const uint32_t* uw = reinterpret_cast<const uint32_t*>(&uv);
    uint4 ov;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      auto act = [](float x) { return to_float<false>(from_float<false>(x / (1.f + __expf(-x)))); };
      float a = act(pair_lo<false>(gw[j])) * pair_lo<false>(uw[j]);
      float b = act(pair_hi<false>(gw[j])) * pair_hi<false>(uw[j]);
      ow[j] = (uint32_t)from_float<false>(a) | ((uint32_t)from_float<false>(b) << 16);
    }
    *reinterpret_cast<uint4*>(out + idx) = ov;
  }
}

}  // namespace
}  // namespace fdk

using namespace fdk;

extern "C" int fdk_rmsnorm(void* h, const void* delta, const void* weight, void* out, int rows, int width,
                           float eps, void* stream) {
  FDK_CHECK_ARG(h && weight && out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(rows > 0 && width > 0 && width % 8 == 0 && width <= 16384, FDK_ERR_SHAPE,
                "rows=%d, width=%d (width must be a multiple of 8, at most 16384)", rows, width);
  FDK_CHECK_ARG((((uintptr_t)h | (uintptr_t)weight | (uintptr_t)out | (uintptr_t)delta) & 15) == 0, FDK_ERR_ALIGN,
                "pointers must be 16-byte aligned");
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 48 * 1024) {
    static bool configured[64] = {};
    int dev = 0;
    FDK_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
      FDK_CUDA(cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
      configured[dev & 63] = true;
    }
  }
  rmsnorm_kernel<<<rows, 256, smem, (cudaStream_t)stream>>>((uint16_t*)h, (const uint16_t*)delta,
                                                             (const uint16_t*)weight, (uint16_t*)out, width, eps);
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}

extern "C" int fdk_rope_append(const void* qkv, const void* pos, void* q_out, void* k_cache, void* v_cache,
                               int rows, int q_heads, int kv_heads, int head_dim, int max_len, float theta,
                               void* stream) {
  FDK_CHECK_ARG(qkv && pos && q_out && k_cache && v_cache, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(head_dim == 128, FDK_ERR_SHAPE, "head_dim=%d: only 128 is supported", head_dim);
  FDK_CHECK_ARG(rows > 0 && q_heads > 0 && kv_heads > 0 && max_len > 0, FDK_ERR_BAD_ARG, "non-positive size");
  dim3 grid(q_heads + 2 * kv_heads, rows);
  rope_append_kernel<<<grid, 64, 0, (cudaStream_t)stream>>>((const uint16_t*)qkv, (const long long*)pos,
                                                            (uint16_t*)q_out, (uint16_t*)k_cache,
                                                            (uint16_t*)v_cache, q_heads, kv_heads, max_len, theta);
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}

extern "C" int fdk_silu_mul(const void* gate_up, void* out, int rows, int width, void* stream) {
  FDK_CHECK_ARG(gate_up && out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(rows > 0 && width > 0 && width % 8 == 0, FDK_ERR_SHAPE, "rows=%d, width=%d", rows, width);
  FDK_CHECK_ARG((((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0, FDK_ERR_ALIGN, "pointers must be 16-byte aligned");
  const long long total = (long long)rows * width;
  long long blocks = (total / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  silu_mul_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)gate_up, (uint16_t*)out, width, total);
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}
