// Glue kernels of the custom-llama decode step, around the quantised projections:
// RMSNorm fused with the residual add, rotary embedding fused with the KV-cache append,
// SiLU(gate) * up.  All are one pass over a [batch, width] bf16 activation (a few KB to a few
// MB), bound by launch latency at small batch and by HBM at large batch; they exist to
// replace ~10 framework launches per layer by 3.  The reference gets this arithmetic from
// transformers' LlamaForCausalLM (src/fdk/models.py:238-251); the formulas below follow that
// model's definition (RMSNorm in fp32 with the weight applied after the cast, rotate-half
// rotary embedding with cos/sin rounded to the activation type).
#include <cstring>
#include <type_traits>

#include "fdk_common.cuh"
#include "linear_lut_params.cuh"
#include "tp_exchange.cuh"

namespace fdk {
namespace {

// Every kernel here is launched with programmatic stream serialisation: it lets the next
// kernel on the stream be scheduled at once, and itself waits for the previous kernel before
// touching memory.  This only hides launch latency; ordering is that of the stream.
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <class... KArgs, class... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FDK_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
  return FDK_OK;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Where the partial sums of a tensor-parallel push are found (this rank's exchange buffer).
struct ReduceSource {
  const uint2* stage;  // words {two partial sums, tag} [2][tp][slot / 2]
  uint32_t* seq;       // reduces completed so far
  int* done;           // CTAs of this reduce that have finished
  int* status;
  long long slot;
  int tp;
};

__device__ __forceinline__ uint4 ld_words(const uint2* p) {  // two staging words
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Reads the two words again until both carry `tag` (bounded: two seconds).  Once a wait has
// run out on this rank (status bit set, by this or an earlier reduce) later words are taken as
// they are, so that a rank whose peer stopped pushing fails within seconds instead of waiting
// two seconds per word.
__device__ __forceinline__ void settle(uint4& v, const uint2* p, uint32_t tag, int* status) {
  unsigned long long t0 = 0;
  if ((v.y != tag || v.w != tag) && (*reinterpret_cast<volatile int*>(status) & 1)) {
    v = make_uint4(0u, tag, 0u, tag);
    return;
  }
  for (uint32_t i = 0; v.y != tag || v.w != tag; ++i) {
    v = ld_words(p);
    if ((i & 63u) == 63u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) {
        atomicOr(status, 1);
        v = make_uint4(0u, tag, 0u, tag);
      }
    }
  }
}

// out[row] = weight * bf16(h[row] * rsqrt(mean(h[row]^2) + eps)), with h += delta first when
// delta is given (h is the residual stream, updated in place).  REDUCE: delta is the sum over
// ranks (fp32, rank order, rounded to bf16) of the partial sums of the latest push, after
// every rank's arrival flag has been seen (bounded wait).
template <bool REDUCE>
__global__ void rmsnorm_kernel(uint16_t* __restrict__ h, const uint16_t* __restrict__ delta,
                               const uint16_t* __restrict__ weight, uint16_t* __restrict__ out, int width,
                               float eps, ReduceSource src) {
  extern __shared__ float row_cache[];  // width floats
  __shared__ float partial[32];
  pdl_prologue();
  const int row = blockIdx.x;
  uint16_t* hr = h + (size_t)row * width;
  const uint16_t* dr = delta ? delta + (size_t)row * width : nullptr;
  uint32_t c = 0;           // number of the push being reduced
  const uint2* words = nullptr;
  if constexpr (REDUCE) {
    c = *reinterpret_cast<const volatile uint32_t*>(src.seq);
    words = src.stage + ((size_t)(c & 1u) * src.tp * src.slot + (size_t)row * width) / 2;
  }
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
    uint4 hv = *reinterpret_cast<const uint4*>(hr + i);
    uint32_t* hw = reinterpret_cast<uint32_t*>(&hv);
    if (dr || REDUCE) {
      uint4 dv;
      if constexpr (REDUCE) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 v[2 * kTpMaxRanks];  // all ranks' words in flight at once
#pragma unroll
        for (int j = 0; j < kTpMaxRanks; ++j) {
          if (j < src.tp) {
            const uint2* w = words + ((size_t)j * src.slot + i) / 2;
            v[2 * j] = ld_words(w);
            v[2 * j + 1] = ld_words(w + 2);
          }
        }
#pragma unroll
        for (int j = 0; j < kTpMaxRanks; ++j) {  // added in rank order
          if (j < src.tp) {
            const uint2* w = words + ((size_t)j * src.slot + i) / 2;
            settle(v[2 * j], w, c + 1u, src.status);
            settle(v[2 * j + 1], w + 2, c + 1u, src.status);
            const uint4 lo = v[2 * j], hi = v[2 * j + 1];
            acc[0] += pair_lo<false>(lo.x); acc[1] += pair_hi<false>(lo.x);
            acc[2] += pair_lo<false>(lo.z); acc[3] += pair_hi<false>(lo.z);
            acc[4] += pair_lo<false>(hi.x); acc[5] += pair_hi<false>(hi.x);
            acc[6] += pair_lo<false>(hi.z); acc[7] += pair_hi<false>(hi.z);
          }
        }
        uint32_t* dwm = reinterpret_cast<uint32_t*>(&dv);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          dwm[j] = (uint32_t)from_float<false>(acc[2 * j]) | ((uint32_t)from_float<false>(acc[2 * j + 1]) << 16);
      } else {
        dv = *reinterpret_cast<const uint4*>(dr + i);
      }
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
  if constexpr (REDUCE) {  // the last CTA to get here counts this reduce as done
    __syncthreads();
    if (threadIdx.x == 0) {
      if (atomicAdd(src.done, 1) == (int)gridDim.x - 1) {
        *src.done = 0;
        *reinterpret_cast<volatile uint32_t*>(src.seq) = c + 1u;
      }
    }
  }
}

// One CTA (64 threads) per (batch row, head of the fused q|k|v projection); head_dim = 128.
// q heads: rotated, written to q_out.  k heads: rotated, written to the cache at *pos.
// v heads: copied to the cache at *pos.  A position outside [0, max_len) -- one decode step
// too many, a stale position buffer -- leaves the caches untouched (q is still written).
__global__ void rope_append_kernel(const uint16_t* __restrict__ qkv, const long long* __restrict__ pos_ptr,
                                   uint16_t* __restrict__ q_out, uint16_t* __restrict__ k_cache,
                                   uint16_t* __restrict__ v_cache, int q_heads, int kv_heads, int max_len,
                                   float theta, int paired) {
  pdl_prologue();
  const int row = blockIdx.y, head = blockIdx.x, i = threadIdx.x;  // i in 0..63: the pair (i, i + 64)
  const long long pos = *pos_ptr;
  const bool in_cache = pos >= 0 && pos < max_len;
  const int heads_total = q_heads + 2 * kv_heads;
  const uint16_t* src = qkv + ((size_t)row * heads_total + head) * 128;
  if (head >= q_heads + kv_heads) {  // v
    if (!in_cache) return;
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
  // paired: the head's values come in the order [0..31, 64..95, 32..63, 96..127] (the row order the
  // projection kernel's rotary output wants), so dimension i sits at i or i + 32, its partner 32 further on
  const int at = paired ? (i < 32 ? i : i + 32) : i;
  const float x0 = to_float<false>(src[at]), x1 = to_float<false>(src[at + (paired ? 32 : 64)]);
  // out = x * cos + rotate_half(x) * sin, each product and the sum rounded to bf16
  auto r = [](float v) { return to_float<false>(from_float<false>(v)); };
  const uint16_t o0 = from_float<false>(r(x0 * c) + r(-x1 * s));
  const uint16_t o1 = from_float<false>(r(x1 * c) + r(x0 * s));
  uint16_t* dst;
  if (head < q_heads) {
    dst = q_out + ((size_t)row * q_heads + head) * 128;
  } else {
    if (!in_cache) return;
    dst = k_cache + (((size_t)row * kv_heads + (head - q_heads)) * max_len + pos) * 128;
  }
  dst[i] = o0;
  dst[i + 64] = o1;
}

// table[i] = {bf16 cos, bf16 sin} of angle pos * theta^(-2 i / 128), i = 0 .. 63: what every
// rotary embedding of one decode step needs, computed once per step (the values of
// rope_append_kernel above).
__global__ void rope_table_kernel(const long long* __restrict__ pos_ptr, uint32_t* __restrict__ table, float theta) {
  pdl_prologue();
  const int i = threadIdx.x;
  const float inv_freq = powf(theta, -(float)(2 * i) / 128.f);
  const float angle = (float)(*pos_ptr) * inv_freq;
  table[i] = (uint32_t)from_float<false>(cosf(angle)) | ((uint32_t)from_float<false>(sinf(angle)) << 16);
}

// sumsq[row][t] = sum of squares of h[row][64 t .. 64 t + 63]; one warp per (row, tile), lane l
// taking elements l and l + 32, added in the order of the projection kernel's residual output.
// With `weight`: also x[row][col] = bf16(weight[col] * h[row][col]) (deferred RMSNorm).
__global__ void sumsq_tiles_kernel(const uint16_t* __restrict__ h, float* __restrict__ sumsq, int width, int tiles,
                                   const uint16_t* __restrict__ weight, uint16_t* __restrict__ x) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), row = blockIdx.y;
  if (t >= tiles) return;
  float sq = 0.f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int col = t * 64 + lane + 32 * half;
    if (col < width) {
      const float v = to_float<false>(h[(size_t)row * width + col]);
      sq = fmaf(v, v, sq);
      if (weight != nullptr) x[(size_t)row * width + col] = from_float<false>(v * to_float<false>(weight[col]));
    }
  }
  sq = warp_sum(sq);
  if (lane == 0) sumsq[(size_t)row * tiles + t] = sq;
}

// out[row] = index of the largest of x[row][0 .. n) (the lowest such index; a NaN counts as
// larger than any number, as torch.argmax has it): greedy decoding's token choice.  One CTA of
// 1024 threads per row; values are compared as keys whose unsigned order is the numeric order,
// packed with the complemented index so that one 64-bit maximum decides both.
template <bool FP16>
__global__ void __launch_bounds__(1024) argmax_kernel(const uint16_t* __restrict__ x, long long* __restrict__ out, int n) {
  pdl_prologue();
  __shared__ unsigned long long best_of_warp[32];
  const uint16_t* row = x + (size_t)blockIdx.x * n;
  auto key_of = [](uint16_t bits) -> uint32_t {
    // 16-bit floats order like sign-magnitude integers: flip negatives, lift positives
    const uint32_t b = bits;
    const uint32_t nan_limit = FP16 ? 0x7C00u : 0x7F80u;
    if ((b & 0x7FFFu) > nan_limit) return 0xFFFFu;  // NaN of either sign
    return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
  };
  unsigned long long best = 0;
  auto take = [&](uint16_t bits, int idx) {
    const unsigned long long cand = ((unsigned long long)key_of(bits) << 32) | (uint32_t)(~(uint32_t)idx);
    best = cand > best ? cand : best;
  };
  const int vecs = (((uintptr_t)row & 15) == 0) ? n / 8 : 0;  // 16-byte loads where the row allows them
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + (size_t)v * 8);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      take((uint16_t)(w[j] & 0xFFFFu), v * 8 + 2 * j);
      take((uint16_t)(w[j] >> 16), v * 8 + 2 * j + 1);
    }
  }
  for (int i = vecs * 8 + threadIdx.x; i < n; i += blockDim.x) take(row[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) best_of_warp[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? best_of_warp[threadIdx.x] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = (long long)(~(uint32_t)(best & 0xFFFFFFFFull));
  }
}

// out[row, j] = silu(gate) * up; the columns of gate_up alternate `group` gate values and the
// `group` matching up values.
__global__ void silu_mul_kernel(const uint16_t* __restrict__ gate_up, uint16_t* __restrict__ out, int width,
                                int group, long long total) {
  pdl_prologue();
  for (long long idx = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8; idx < total;
       idx += (long long)gridDim.x * blockDim.x * 8) {
    const long long row = idx / width;
    const int col = (int)(idx - row * width);
    const int tile = col / group;
    const uint16_t* g = gate_up + row * 2 * width + (size_t)tile * 2 * group + (col - tile * group);
    uint4 gv = *reinterpret_cast<const uint4*>(g);
    uint4 uv = *reinterpret_cast<const uint4*>(g + group);
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

static int rmsnorm_launch(void* h, const void* delta, const fdk_tp_exchange* ex, const void* weight, void* out,
                          int rows, int width, float eps, void* stream) {
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
      FDK_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
      FDK_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
      configured[dev & 63] = true;
    }
  }
  ReduceSource src{};
  if (ex == nullptr) {
    return launch_pdl(rmsnorm_kernel<false>, dim3(rows), dim3(256), smem, (cudaStream_t)stream, (uint16_t*)h,
                      (const uint16_t*)delta, (const uint16_t*)weight, (uint16_t*)out, width, eps, src);
  }
  FDK_CHECK_ARG(ex->tp >= 1 && ex->tp <= kTpMaxRanks && ex->rank >= 0 && ex->rank < ex->tp, FDK_ERR_BAD_ARG,
                "tp=%d, rank=%d", ex->tp, ex->rank);
  FDK_CHECK_ARG(ex->slot_elems % 8 == 0 && (long long)rows * width <= ex->slot_elems, FDK_ERR_SHAPE,
                "rows=%d x width=%d exceeds slots of %lld elements", rows, width, ex->slot_elems);
  uint8_t* local = (uint8_t*)ex->buffers[ex->rank];
  FDK_CHECK_ARG(local != nullptr && ((uintptr_t)local & 255) == 0, FDK_ERR_ALIGN,
                "the exchange buffer must be a 256-byte aligned device pointer");
  src.stage = (const uint2*)(local + kTpStageOffset);
  src.seq = (uint32_t*)(local + kTpSeqOffset);
  src.done = (int*)(local + kTpDoneOffset);
  src.status = (int*)(local + kTpStatusOffset);
  src.slot = ex->slot_elems;
  src.tp = ex->tp;
  return launch_pdl(rmsnorm_kernel<true>, dim3(rows), dim3(256), smem, (cudaStream_t)stream, (uint16_t*)h,
                    (const uint16_t*)nullptr, (const uint16_t*)weight, (uint16_t*)out, width, eps, src);
}

extern "C" int fdk_rmsnorm(void* h, const void* delta, const void* weight, void* out, int rows, int width,
                           float eps, void* stream) {
  return rmsnorm_launch(h, delta, nullptr, weight, out, rows, width, eps, stream);
}

extern "C" int fdk_rmsnorm_reduce(void* h, const fdk_tp_exchange* ex, const void* weight, void* out, int rows,
                                  int width, float eps, void* stream) {
  FDK_CHECK_ARG(ex != nullptr, FDK_ERR_BAD_ARG, "exchange is null");
  return rmsnorm_launch(h, nullptr, ex, weight, out, rows, width, eps, stream);
}

// ---- exchange buffers: device allocations shared between the ranks' processes by CUDA IPC ----
extern "C" size_t fdk_tp_exchange_bytes(int tp, long long slot_elems) {
  if (tp < 1 || tp > kTpMaxRanks || slot_elems <= 0) return 0;
  return tp_exchange_bytes(tp, slot_elems);
}

extern "C" int fdk_tp_buffer_create(size_t bytes, void** ptr_host, unsigned char* handle_host) {
  FDK_CHECK_ARG(bytes > 0 && ptr_host && handle_host, FDK_ERR_BAD_ARG, "null pointer or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64 bytes");
  void* ptr = nullptr;
  FDK_CUDA(cudaMalloc(&ptr, bytes));
  FDK_CUDA(cudaMemset(ptr, 0, bytes));
  FDK_CUDA(cudaDeviceSynchronize());
  cudaIpcMemHandle_t handle;
  FDK_CUDA(cudaIpcGetMemHandle(&handle, ptr));
  memcpy(handle_host, &handle, sizeof(handle));
  *ptr_host = ptr;
  return FDK_OK;
}

extern "C" int fdk_tp_buffer_open(const unsigned char* handle_host, void** ptr_host) {
  FDK_CHECK_ARG(handle_host && ptr_host, FDK_ERR_BAD_ARG, "null pointer");
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle_host, sizeof(handle));
  void* ptr = nullptr;
  FDK_CUDA(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess));
  *ptr_host = ptr;
  return FDK_OK;
}

extern "C" int fdk_tp_buffer_close(void* ptr) {
  FDK_CHECK_ARG(ptr != nullptr, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CUDA(cudaIpcCloseMemHandle(ptr));
  return FDK_OK;
}

extern "C" int fdk_tp_buffer_destroy(void* ptr) {
  FDK_CHECK_ARG(ptr != nullptr, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CUDA(cudaFree(ptr));
  return FDK_OK;
}

extern "C" int fdk_tp_exchange_status(const fdk_tp_exchange* ex, int* status_host) {
  FDK_CHECK_ARG(ex && status_host && ex->rank >= 0 && ex->rank < kTpMaxRanks && ex->buffers[ex->rank],
                FDK_ERR_BAD_ARG, "null pointer");
  FDK_CUDA(cudaMemcpy(status_host, (const uint8_t*)ex->buffers[ex->rank] + kTpStatusOffset, sizeof(int),
                      cudaMemcpyDeviceToHost));
  return FDK_OK;
}

static int rope_append_impl(const void* qkv, const void* pos, void* q_out, void* k_cache, void* v_cache, int rows,
                            int q_heads, int kv_heads, int head_dim, int max_len, float theta, int paired,
                            void* stream) {
  FDK_CHECK_ARG(qkv && pos && q_out && k_cache && v_cache, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(head_dim == 128, FDK_ERR_SHAPE, "head_dim=%d: only 128 is supported", head_dim);
  FDK_CHECK_ARG(rows > 0 && q_heads > 0 && kv_heads > 0 && max_len > 0, FDK_ERR_BAD_ARG, "non-positive size");
  dim3 grid(q_heads + 2 * kv_heads, rows);
  return launch_pdl(rope_append_kernel, grid, dim3(64), 0, (cudaStream_t)stream, (const uint16_t*)qkv,
                    (const long long*)pos, (uint16_t*)q_out, (uint16_t*)k_cache, (uint16_t*)v_cache, q_heads,
                    kv_heads, max_len, theta, paired);
}

extern "C" int fdk_rope_append(const void* qkv, const void* pos, void* q_out, void* k_cache, void* v_cache,
                               int rows, int q_heads, int kv_heads, int head_dim, int max_len, float theta,
                               void* stream) {
  return rope_append_impl(qkv, pos, q_out, k_cache, v_cache, rows, q_heads, kv_heads, head_dim, max_len, theta, 0, stream);
}

extern "C" int fdk_rope_append_paired(const void* qkv, const void* pos, void* q_out, void* k_cache, void* v_cache,
                                      int rows, int q_heads, int kv_heads, int head_dim, int max_len, float theta,
                                      void* stream) {
  return rope_append_impl(qkv, pos, q_out, k_cache, v_cache, rows, q_heads, kv_heads, head_dim, max_len, theta, 1, stream);
}

extern "C" int fdk_rope_table(const void* pos, void* table, float theta, void* stream) {
  FDK_CHECK_ARG(pos && table, FDK_ERR_BAD_ARG, "null pointer");
  return launch_pdl(rope_table_kernel, dim3(1), dim3(64), 0, (cudaStream_t)stream, (const long long*)pos,
                    (uint32_t*)table, theta);
}

extern "C" int fdk_sumsq_tiles(const void* h, float* sumsq, int rows, int width, void* stream) {
  FDK_CHECK_ARG(h && sumsq, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(rows > 0 && width > 0, FDK_ERR_BAD_ARG, "non-positive size");
  const int tiles = (width + 63) / 64;
  return launch_pdl(sumsq_tiles_kernel, dim3((tiles + 7) / 8, rows), dim3(256), 0, (cudaStream_t)stream,
                    (const uint16_t*)h, sumsq, width, tiles, (const uint16_t*)nullptr, (uint16_t*)nullptr);
}

extern "C" int fdk_norm_prepare(const void* h, const void* weight, void* x, float* sumsq, int rows, int width,
                                void* stream) {
  FDK_CHECK_ARG(h && weight && x && sumsq, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(rows > 0 && width > 0, FDK_ERR_BAD_ARG, "non-positive size");
  const int tiles = (width + 63) / 64;
  return launch_pdl(sumsq_tiles_kernel, dim3((tiles + 7) / 8, rows), dim3(256), 0, (cudaStream_t)stream,
                    (const uint16_t*)h, sumsq, width, tiles, (const uint16_t*)weight, (uint16_t*)x);
}

extern "C" int fdk_argmax(const void* x, void* out, int rows, int n, int dtype, void* stream) {
  FDK_CHECK_ARG(x && out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(rows > 0 && n > 0, FDK_ERR_BAD_ARG, "non-positive size");
  FDK_CHECK_ARG(dtype == FDK_DTYPE_BF16 || dtype == FDK_DTYPE_F16, FDK_ERR_BAD_ARG, "dtype=%d", dtype);
  FDK_CHECK_ARG(((uintptr_t)x & 1) == 0 && ((uintptr_t)out & 7) == 0, FDK_ERR_ALIGN, "x must be 2-byte, out 8-byte aligned");
  if (dtype == FDK_DTYPE_F16) {
    return launch_pdl(argmax_kernel<true>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, (const uint16_t*)x,
                      (long long*)out, n);
  }
  return launch_pdl(argmax_kernel<false>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, (const uint16_t*)x,
                    (long long*)out, n);
}

extern "C" int fdk_silu_mul(const void* gate_up, void* out, int rows, int width, int group, void* stream) {
  FDK_CHECK_ARG(gate_up && out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(rows > 0 && width > 0 && group > 0 && group % 8 == 0 && width % group == 0, FDK_ERR_SHAPE,
                "rows=%d, width=%d, group=%d (group a multiple of 8, width a multiple of group)", rows, width, group);
  FDK_CHECK_ARG((((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0, FDK_ERR_ALIGN, "pointers must be 16-byte aligned");
  const long long total = (long long)rows * width;
  long long blocks = (total / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch_pdl(silu_mul_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream,
                    (const uint16_t*)gate_up, (uint16_t*)out, width, group, total);
}

// ---- decode attention over the static KV cache ----------------------------------------------
// One query token per batch row, grouped-query attention, head_dim 128, bf16 cache
// [batch, kv_heads, max_len, 128].  Grid (splits, kv_heads, batch): a CTA of 8 warps takes one
// slice of the context for all the query heads that share a KV head (so every key/value byte
// is read once), keeps a running softmax per head, and leaves {max, sum, 128 weighted values}
// per head in scratch as tagged words; the CTA of slice 0 polls them (bounded), merges the
// slices and writes the bf16 output.  HBM-bound at large batch (2 x 256 B per position per KV head).
// Two kernels share that scheme: a scalar one for small grids (latency-bound: at most one CTA
// per SM, ratios up to 4) and a tensor-core one for everything else.
namespace fdk {
namespace {

constexpr int kAttnWarps = 8;
constexpr int kMaxSplits = 64;
constexpr int kMaxGroup = 8;

// What follows the key/value loop, shared by the two attention kernels: `part[w][j]` holds warp
// w's {128 weighted values, max, sum} of head j.  The warps are merged in a fixed order; an
// unsliced context writes the bf16 output directly, a slice leaves its numbers in scratch as
// tagged words and the CTA of slice 0 polls them (bounded), merges and writes the output.
template <int G>
__device__ __forceinline__ void attention_finish(const float (*part)[G][132], uint16_t* __restrict__ out,
                                                 float* __restrict__ scratch, int* __restrict__ counters, int split,
                                                 int splits, int b, int kvh, int kv_heads, int q_heads) {
  const int head0 = kvh * G;
  // threads 0..127: one output dimension each from here on
  const int d = threadIdx.x & 127;
  const bool writer = threadIdx.x < 128;
  // Every slice leaves its numbers in scratch as 8-byte words {value, tag}, tag = number of this
  // use of the (batch row, KV head) + 1: a word is valid once its tag is this launch's, so the
  // slices need no fence, counter or second trip through L2 to hand their sums over.
  const int group = b * kv_heads + kvh;
  const uint32_t uses = splits == 1 ? 0u : (uint32_t)ld_relaxed_s32(counters + group);
  const uint32_t tag = uses + 1u;
  uint2* mine = reinterpret_cast<uint2*>(scratch) + ((size_t)group * splits + split) * (G * 130);
  if (writer) {
    for (int j = 0; j < G; ++j) {
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) m = fmaxf(m, part[w][j][128]);
      float l = 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) {
        const float c = (part[w][j][128] == -INFINITY) ? 0.f : __expf(part[w][j][128] - m);
        l += part[w][j][129] * c;
        a += part[w][j][d] * c;
      }
      if (splits == 1) {
        out[((size_t)b * q_heads + head0 + j) * 128 + d] = from_float<false>(l > 0.f ? a / l : 0.f);
      } else {
        st_relaxed_v2(mine + j * 130 + d, make_uint2(__float_as_uint(a), tag));
        if (d == 0) {
          st_relaxed_v2(mine + j * 130 + 128, make_uint2(__float_as_uint(m), tag));
          st_relaxed_v2(mine + j * 130 + 129, make_uint2(__float_as_uint(l), tag));
        }
      }
    }
  }
  if (splits == 1 || split != 0) return;

  // The CTA of slice 0 merges.  Thread (d, half) takes output dimension d of every second
  // slice; its first words are requested before the slices' maxima and sums are polled, so
  // that the merge costs one trip to L2 once the last slice has written.  All polls are bounded.
  __shared__ float coef[G][kMaxSplits];
  __shared__ float lpart[G][kMaxSplits];
  __shared__ float denom[G];
  __shared__ float other_half[G][128];
  constexpr int SB = G <= 4 ? 8 : 4;  // slices per thread in flight (SB * G words)
  constexpr uint32_t kPollLimit = 1u << 20;
  const uint2* base = reinterpret_cast<const uint2*>(scratch) + (size_t)group * splits * (G * 130);
  const int half = threadIdx.x >> 7;
  bool ok = true;
  uint2 av[SB][G];
  auto request = [&](int s0) {  // slices s0 + half, s0 + half + 2, ...
#pragma unroll
    for (int i = 0; i < SB; ++i) {
      const int s2 = s0 + half + 2 * i;
#pragma unroll
      for (int j = 0; j < G; ++j)
        av[i][j] = s2 < splits ? ld_relaxed_v2(base + (size_t)s2 * (G * 130) + j * 130 + d) : make_uint2(0u, tag);
    }
  };
  request(0);
  for (int idx = threadIdx.x; idx < G * splits; idx += blockDim.x) {
    const int j = idx / splits, s2 = idx - j * splits;
    const uint2* w = base + (size_t)s2 * (G * 130) + j * 130 + 128;
    uint2 mm = ld_relaxed_v2(w), ll = ld_relaxed_v2(w + 1);
    for (uint32_t spins = 0; mm.y != tag || ll.y != tag; ++spins) {
      if (spins > kPollLimit) {
        ok = false;
        break;
      }
      __nanosleep(64);
      mm = ld_relaxed_v2(w);
      ll = ld_relaxed_v2(w + 1);
    }
    coef[j][s2] = __uint_as_float(mm.x);  // the slice's max for now
    lpart[j][s2] = __uint_as_float(ll.x);
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int j = threadIdx.x;
    float m = -INFINITY;
    for (int s2 = 0; s2 < splits; ++s2) m = fmaxf(m, coef[j][s2]);
    float l = 0.f;
    for (int s2 = 0; s2 < splits; ++s2) {
      const float c = (coef[j][s2] == -INFINITY) ? 0.f : __expf(coef[j][s2] - m);
      l += lpart[j][s2] * c;
      coef[j][s2] = c;
    }
    denom[j] = l;
  }
  __syncthreads();
  float total[G];
#pragma unroll
  for (int j = 0; j < G; ++j) total[j] = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 2 * SB) {
    if (s0 > 0) request(s0);
    for (uint32_t spins = 0;; ++spins) {  // a slice's maximum can land before its last sums
      bool fresh = true;
#pragma unroll
      for (int i = 0; i < SB; ++i)
#pragma unroll
        for (int j = 0; j < G; ++j) fresh = fresh && av[i][j].y == tag;
      if (fresh) break;
      if (spins > kPollLimit) {
        ok = false;
        break;
      }
      __nanosleep(64);
      request(s0);
    }
#pragma unroll
    for (int i = 0; i < SB; ++i) {
      const int s2 = s0 + half + 2 * i;
      if (s2 < splits) {
#pragma unroll
        for (int j = 0; j < G; ++j) total[j] += __uint_as_float(av[i][j].x) * coef[j][s2];
      }
    }
  }
  if (half == 1) {
#pragma unroll
    for (int j = 0; j < G; ++j) other_half[j][d] = total[j];
  }
  __syncthreads();
  if (half == 0) {
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const float a = total[j] + other_half[j][d];
      out[((size_t)b * q_heads + head0 + j) * 128 + d] = from_float<false>(denom[j] > 0.f ? a / denom[j] : 0.f);
    }
  }
  if (threadIdx.x == 0) counters[group] = (int)((uses + 1u) & 0x3FFFFFFFu);  // this use is done
  if (!ok) atomicOr(counters + gridDim.z * kv_heads, kStatusTimeout);
}

// This scalar kernel serves grids of at most one CTA per SM with grouped-query ratios up to 4
// (small batches: bound by latency, which its prefetch before the wait and its sixteen keys per
// warp in flight address); everything else goes to the tensor-core kernel below.
template <int G>
__global__ void __launch_bounds__(kAttnWarps * 32, 1)
    decode_attention_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k_cache,
                            const uint16_t* __restrict__ v_cache, const long long* __restrict__ pos_ptr,
                            uint16_t* __restrict__ out, float* __restrict__ scratch, int* __restrict__ counters,
                            int q_heads, int kv_heads, int max_len, int chunk) {
  static_assert(G >= 1 && G <= 4, "ratios above 4 take the tensor-core kernel");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ __align__(16) float part[kAttnWarps][G][132];
  __shared__ float wbuf[kAttnWarps][16 * G];  // softmax weights of a round, per warp: U * G
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, splits = gridDim.x;
  const int head0 = kvh * G;  // this CTA's first query head
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // The position only changes between decode steps, and the keys and values of earlier
  // positions were written in earlier steps: both may be read before the kernel that feeds
  // this one (it writes q and the current position's key and value) has finished.
  // A position outside the cache is clamped (no key at all gives zeros).
  const long long pos_now = *pos_ptr;
  const int len = pos_now < 0 ? 0 : (pos_now >= max_len ? max_len : (int)pos_now + 1);
  const int p0 = split * chunk, p1 = min(len, p0 + chunk);
  const uint16_t* kb = k_cache + ((size_t)b * kv_heads + kvh) * max_len * 128 + lane * 4;
  const uint16_t* vb = v_cache + ((size_t)b * kv_heads + kvh) * max_len * 128 + lane * 4;
  // U positions per warp and iteration, all their loads in flight together: with a slice of up
  // to 8 * U keys a warp pays the memory latency once -- and for its first U positions before
  // the wait, beside the previous kernel
  constexpr int U = 16;
  uint2 kk[U], vv[U];
  const int pb_first = p0 + warp * U;
  if (pb_first < p1) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int p = min(pb_first + u, p1 - 1);  // clamped reads, masked below
      if (p != len - 1) {  // the current position is read after the wait
        kk[u] = *reinterpret_cast<const uint2*>(kb + (size_t)p * 128);
        vv[u] = *reinterpret_cast<const uint2*>(vb + (size_t)p * 128);
      }
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float qf[G][4], acc[G][4], mx[G], sum[G];
  const float scale = 0.08838834764831845f;  // 1 / sqrt(128)
#pragma unroll
  for (int j = 0; j < G; ++j) {
    const uint2 qq = *reinterpret_cast<const uint2*>(q + ((size_t)b * q_heads + head0 + j) * 128 + lane * 4);
    qf[j][0] = pair_lo<false>(qq.x) * scale; qf[j][1] = pair_hi<false>(qq.x) * scale;
    qf[j][2] = pair_lo<false>(qq.y) * scale; qf[j][3] = pair_hi<false>(qq.y) * scale;
    acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    mx[j] = -INFINITY;
    sum[j] = 0.f;
  }
  for (int pb = pb_first; pb < p1; pb += kAttnWarps * U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int p = min(pb + u, p1 - 1);
      if (pb != pb_first || p == len - 1) {
        kk[u] = *reinterpret_cast<const uint2*>(kb + (size_t)p * 128);
        vv[u] = *reinterpret_cast<const uint2*>(vb + (size_t)p * 128);
      }
    }
    float s[U][G];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float k0 = pair_lo<false>(kk[u].x), k1 = pair_hi<false>(kk[u].x), k2 = pair_lo<false>(kk[u].y), k3 = pair_hi<false>(kk[u].y);
#pragma unroll
      for (int j = 0; j < G; ++j) s[u][j] = qf[j][0] * k0 + qf[j][1] * k1 + qf[j][2] * k2 + qf[j][3] * k3;
    }
    // Sum the 32 lanes' partial dot products.  Not U * G butterflies (5 shuffles each): the
    // position range is halved with the lane distance, so that after log2(U) rounds a group
    // of 32 / U lanes holds the G totals of ONE position (u_own), at a fifth of the shuffles.
    auto halve = [&](auto hc, int off) {
      constexpr int H = decltype(hc)::value;
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int u = 0; u < H; ++u)
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const float send = upper ? s[u][j] : s[u + H][j];
          const float keep = upper ? s[u + H][j] : s[u][j];
          s[u][j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    };
    static_assert(U == 16, "four halving rounds take sixteen positions down to one per pair of lanes");
    halve(std::integral_constant<int, 8>{}, 16);
    halve(std::integral_constant<int, 4>{}, 8);
    halve(std::integral_constant<int, 2>{}, 4);
    halve(std::integral_constant<int, 1>{}, 2);
#pragma unroll
    for (int j = 0; j < G; ++j) s[0][j] += __shfl_xor_sync(0xffffffffu, s[0][j], 1);
    const int u_own = lane / (32 / U);
    const bool live = pb + u_own < p1;
    float* wrow = wbuf[warp];
    float corr[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const float mine = live ? s[0][j] : -INFINITY;
      float m_new = mine;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, o));
      m_new = fmaxf(m_new, mx[j]);
      corr[j] = __expf(mx[j] - m_new);
      mx[j] = m_new;
      wrow[u_own * G + j] = __expf(mine - m_new);  // exp(-inf) = 0 for masked positions; every lane of the group writes the same value
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < G; ++j) {
      float l = sum[j] * corr[j], a0 = acc[j][0] * corr[j], a1 = acc[j][1] * corr[j], a2 = acc[j][2] * corr[j],
            a3 = acc[j][3] * corr[j];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float w = wrow[u * G + j];  // broadcast read
        l += w;
        a0 += w * pair_lo<false>(vv[u].x);
        a1 += w * pair_hi<false>(vv[u].x);
        a2 += w * pair_lo<false>(vv[u].y);
        a3 += w * pair_hi<false>(vv[u].y);
      }
      sum[j] = l; acc[j][0] = a0; acc[j][1] = a1; acc[j][2] = a2; acc[j][3] = a3;
    }
    __syncwarp();  // the weights are read before the next round overwrites them
  }
  // merge the warps of the CTA (fixed order)
#pragma unroll
  for (int j = 0; j < G; ++j) {
    *reinterpret_cast<float4*>(&part[warp][j][lane * 4]) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    if (lane == 0) {
      part[warp][j][128] = mx[j];
      part[warp][j][129] = sum[j];
    }
  }
  __syncthreads();
  attention_finish<G>(part, out, scratch, counters, split, splits, b, kvh, kv_heads, q_heads);
}

// ---- the same attention on the tensor cores, for grids larger than the GPU --------------------
// With every query head of a KV head in one CTA the scalar kernel above spends ~120 warp
// instructions per key at ratios 5 to 8 and is bound by instruction issue, not by HBM.  Here a
// warp takes 16 keys per step through two `mma.sync.m16n8k16`s:
//   S^T[head, key]  = Q[head, dim] . K[key, dim]^T   (A = Q, eight heads in rows 0-7, rows 8-15
//                                                     zero; B = K, read from global memory)
//   O^T[dim, head] += V[key, dim]^T . P^T[key, head] (A = V through `ldmatrix.trans` from a
//                                                     shared-memory tile; B = P as bf16)
// The accumulator layout of the first product is the B-operand layout of the second, so the
// softmax weights never leave their lane.  The contraction over the 128 dimensions does not
// care about their order: lane (g, t) reads 16 contiguous bytes (dimensions 32c + 8t .. + 7) of
// key g per 32-dimension chunk c and uses the four words as the b0/b1 operands of two
// contraction steps, q being read in the same order.
// Same grid, slices and hand-over between slices as the scalar kernel; ~25 instructions per key
// and warp step.  G = query heads per KV head (1..8).
constexpr int kMmaKeys = 16;                            // keys per warp and step
constexpr int kMmaPitch = 272;                          // bytes per key in the V tile (256 + 16: conflict-free ldmatrix)
constexpr int kMmaTile = kMmaKeys * kMmaPitch;          // one V tile
constexpr int kMmaSmem = kAttnWarps * 2 * kMmaTile;     // two stages per warp; the warps' partial results reuse it

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int G>
__global__ void __launch_bounds__(kAttnWarps * 32, 2)
    decode_attention_mma_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k_cache,
                                const uint16_t* __restrict__ v_cache, const long long* __restrict__ pos_ptr,
                                uint16_t* __restrict__ out, float* __restrict__ scratch, int* __restrict__ counters,
                                int q_heads, int kv_heads, int max_len, int chunk) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ __align__(16) unsigned char mma_smem[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, splits = gridDim.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  // As in the scalar kernel: the position and the keys and values of earlier positions may be
  // read before the kernel that feeds this one has finished; q and position len - 1 may not.
  const long long pos_now = *pos_ptr;
  const int len = pos_now < 0 ? 0 : (pos_now >= max_len ? max_len : (int)pos_now + 1);
  const int p0 = split * chunk, p1 = min(len, p0 + chunk);
  const uint16_t* kb = k_cache + ((size_t)b * kv_heads + kvh) * max_len * 128;
  const uint16_t* vb = v_cache + ((size_t)b * kv_heads + kvh) * max_len * 128;
  unsigned char* tile = mma_smem + warp * 2 * kMmaTile;
  const uint32_t tile_s = (uint32_t)__cvta_generic_to_shared(tile);

  uint4 k0[4], k1[4];  // keys base + g and base + 8 + g
  // which: 0 = every position, 1 = all but position len - 1, 2 = position len - 1 only
  auto load_keys = [&](int base, int which) {
    const int pa = min(base + g, p1 - 1), pb = min(base + 8 + g, p1 - 1);  // clamped, masked below
    const uint16_t* r0 = kb + (size_t)pa * 128 + t * 8;
    const uint16_t* r1 = kb + (size_t)pb * 128 + t * 8;
    const bool do0 = which == 0 || ((pa == len - 1) == (which == 2));
    const bool do1 = which == 0 || ((pb == len - 1) == (which == 2));
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (do0) k0[c] = *reinterpret_cast<const uint4*>(r0 + c * 32);
      if (do1) k1[c] = *reinterpret_cast<const uint4*>(r1 + c * 32);
    }
  };
  auto copy_values = [&](int base, int stage, int which) {  // 16 keys x 256 B, 16 B per lane and instruction
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = i * 32 + lane, key = idx >> 4, seg = idx & 15;
      const int pv = min(base + key, p1 - 1);
      const uint16_t* src = vb + (size_t)pv * 128 + seg * 8;
      const uint32_t dst = tile_s + stage * kMmaTile + key * kMmaPitch + seg * 16;
      if (which == 0 || ((pv == len - 1) == (which == 2)))
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
  };
  constexpr int kStride = kAttnWarps * kMmaKeys;
  int base = p0 + warp * kMmaKeys, stage = 0;
  if (base < p1) {
    load_keys(base, 1);
    copy_values(base, 0, 1);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (base < p1 && base + kMmaKeys >= len) {  // the step that holds the current position (clamped rows repeat it)
    load_keys(base, 2);
    copy_values(base, 0, 2);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  uint4 qa[4];  // head g, dimensions 32c + 8t .. + 7
#pragma unroll
  for (int c = 0; c < 4; ++c)
    qa[c] = g < G ? *reinterpret_cast<const uint4*>(q + ((size_t)b * q_heads + kvh * G + g) * 128 + c * 32 + t * 8)
                  : make_uint4(0u, 0u, 0u, 0u);

  float o[8][4];  // O^T: dimensions 16m + g (c0, c1) and 16m + 8 + g (c2, c3), heads 2t and 2t + 1
#pragma unroll
  for (int m = 0; m < 8; ++m) o[m][0] = o[m][1] = o[m][2] = o[m][3] = 0.f;
  float mx = -INFINITY, sum = 0.f;  // of head g; the sum is this lane's share (keys 2t, 2t+1, 8+2t, 9+2t of every step)
  const float scale = 0.08838834764831845f;  // 1 / sqrt(128)
  // ldmatrix.x4.trans row addresses: matrix (lane >> 3) = {keys 0-7 | 8-15} x {dims 0-7 | 8-15} of a 16-dimension column block
  const uint32_t ldm_off = (uint32_t)(((lane & 7) + ((lane >> 4) << 3)) * kMmaPitch + ((lane >> 3) & 1) * 16);

  for (; base < p1; base += kStride, stage ^= 1) {
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};  // heads g (c0, c1): keys 2t, 2t+1 | 8+2t, 9+2t
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      mma_bf16(sa, qa[c].x, 0u, qa[c].y, 0u, k0[c].x, k0[c].y);
      mma_bf16(sb, qa[c].x, 0u, qa[c].y, 0u, k1[c].x, k1[c].y);
      mma_bf16(sa, qa[c].z, 0u, qa[c].w, 0u, k0[c].z, k0[c].w);
      mma_bf16(sb, qa[c].z, 0u, qa[c].w, 0u, k1[c].z, k1[c].w);
    }
    // the next step's keys and values are requested while this step's are worked on
    if (base + kStride < p1) {
      load_keys(base + kStride, 0);
      copy_values(base + kStride, stage ^ 1, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int key0 = base + 2 * t;
    const float s0 = key0 < p1 ? sa[0] * scale : -INFINITY, s1 = key0 + 1 < p1 ? sa[1] * scale : -INFINITY;
    const float s2 = key0 + 8 < p1 ? sb[0] * scale : -INFINITY, s3 = key0 + 9 < p1 ? sb[1] * scale : -INFINITY;
    float m_new = fmaxf(fmaxf(s0, s1), fmaxf(s2, s3));
    m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 1));
    m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 2));
    m_new = fmaxf(m_new, mx);  // finite: the step has at least key `base` below p1
    const float corr = __expf(mx - m_new);
    mx = m_new;
    const float w0 = __expf(s0 - m_new), w1 = __expf(s1 - m_new), w2 = __expf(s2 - m_new), w3 = __expf(s3 - m_new);
    sum = sum * corr + ((w0 + w1) + (w2 + w3));
    uint32_t pb0, pb1;  // P^T as the B operand: keys 2t, 2t+1 | 8+2t, 9+2t of head g
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pb0) : "f"(w1), "f"(w0));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pb1) : "f"(w3), "f"(w2));
    // the accumulators hold heads 2t and 2t + 1: their correction factors sit in lanes 8t and 8t + 4
    const float c_even = __shfl_sync(0xffffffffu, corr, 8 * t), c_odd = __shfl_sync(0xffffffffu, corr, 8 * t + 4);
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      o[m][0] *= c_even; o[m][1] *= c_odd; o[m][2] *= c_even; o[m][3] *= c_odd;
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // this step's values have landed
    __syncwarp();
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      uint32_t a0, a1, a2, a3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                   : "r"(tile_s + stage * kMmaTile + ldm_off + m * 32));
      mma_bf16(o[m], a0, a1, a2, a3, pb0, pb1);
    }
    __syncwarp();  // the tile is read before the step after next overwrites it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // every warp is done with its tiles: the space now holds the warps' results
  float(*part)[G][132] = reinterpret_cast<float(*)[G][132]>(mma_smem);
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  if (t == 0 && g < G) {
    part[warp][g][128] = mx;
    part[warp][g][129] = sum;
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    if (2 * t < G) {
      part[warp][2 * t][16 * m + g] = o[m][0];
      part[warp][2 * t][16 * m + 8 + g] = o[m][2];
    }
    if (2 * t + 1 < G) {
      part[warp][2 * t + 1][16 * m + g] = o[m][1];
      part[warp][2 * t + 1][16 * m + 8 + g] = o[m][3];
    }
  }
  __syncthreads();
  attention_finish<G>(part, out, scratch, counters, split, splits, b, kvh, kv_heads, q_heads);
}

template <int G>
int launch_attention_mma(const void* q, const void* k_cache, const void* v_cache, const void* pos, void* out,
                         void* scratch, void* counters, int batch, int q_heads, int kv_heads, int max_len,
                         int splits, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    FDK_CUDA(cudaFuncSetAttribute(decode_attention_mma_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem));
    configured[dev & 63] = true;
  }
  const int chunk = (max_len + splits - 1) / splits;
  return launch_pdl(decode_attention_mma_kernel<G>, dim3(splits, kv_heads, batch), dim3(kAttnWarps * 32), (size_t)kMmaSmem,
                    stream, (const uint16_t*)q, (const uint16_t*)k_cache, (const uint16_t*)v_cache,
                    (const long long*)pos, (uint16_t*)out, (float*)scratch, (int*)counters, q_heads, kv_heads, max_len,
                    chunk);
}

template <int G>
int launch_attention(const void* q, const void* k_cache, const void* v_cache, const void* pos, void* out,
                     void* scratch, void* counters, int batch, int q_heads, int kv_heads, int max_len,
                     int splits, cudaStream_t stream) {
  const int chunk = (max_len + splits - 1) / splits;
  return launch_pdl(decode_attention_kernel<G>, dim3(splits, kv_heads, batch), dim3(kAttnWarps * 32), 0, stream,
                    (const uint16_t*)q, (const uint16_t*)k_cache, (const uint16_t*)v_cache, (const long long*)pos,
                    (uint16_t*)out, (float*)scratch, (int*)counters, q_heads, kv_heads, max_len, chunk);
}

}  // namespace
}  // namespace fdk

extern "C" int fdk_decode_attention_scratch(int batch, int q_heads, int kv_heads, int splits,
                                            size_t* scratch_bytes_host, size_t* counter_bytes_host) {
  FDK_CHECK_ARG(scratch_bytes_host && counter_bytes_host, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(batch > 0 && q_heads > 0 && kv_heads > 0 && splits > 0 && q_heads % kv_heads == 0, FDK_ERR_BAD_ARG,
                "bad sizes");
  *scratch_bytes_host = (size_t)batch * q_heads * splits * 130 * sizeof(uint2);  // {value, tag} words
  *counter_bytes_host = ((size_t)batch * kv_heads + 1) * sizeof(int);           // use counts + a status word
  return FDK_OK;
}

extern "C" int fdk_decode_attention_status(const void* counters, int batch, int kv_heads, int* status_host) {
  FDK_CHECK_ARG(counters != nullptr && status_host != nullptr && batch > 0 && kv_heads > 0, FDK_ERR_BAD_ARG, "bad argument");
  FDK_CUDA(cudaMemcpy(status_host, (const int*)counters + (size_t)batch * kv_heads, sizeof(int), cudaMemcpyDeviceToHost));
  return FDK_OK;
}

extern "C" int fdk_decode_attention(const void* q, const void* k_cache, const void* v_cache, const void* pos,
                                    void* out, void* scratch, void* counters, int batch, int q_heads,
                                    int kv_heads, int head_dim, int max_len, int splits, void* stream) {
  FDK_CHECK_ARG(q && k_cache && v_cache && pos && out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(head_dim == 128, FDK_ERR_SHAPE, "head_dim=%d: only 128 is supported", head_dim);
  FDK_CHECK_ARG(batch > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads / kv_heads <= kMaxGroup, FDK_ERR_SHAPE,
                "q_heads=%d must be 1..%d times kv_heads=%d", q_heads, kMaxGroup, kv_heads);
  FDK_CHECK_ARG(splits >= 1 && splits <= kMaxSplits && max_len > 0, FDK_ERR_BAD_ARG, "splits=%d (1..%d), max_len=%d", splits, kMaxSplits, max_len);
  FDK_CHECK_ARG(splits == 1 || (scratch && counters), FDK_ERR_WORKSPACE, "scratch and counters are needed when splits > 1");
  FDK_CHECK_ARG((((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) == 0, FDK_ERR_ALIGN,
                "q, caches and out must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const int group = q_heads / kv_heads;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  // Grids larger than the GPU and grouped-query ratios above 4: the tensor-core kernel.
  if ((long long)splits * kv_heads * batch > di.sm_count || group > 4) {
    switch (group) {
      case 1: return launch_attention_mma<1>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
      case 2: return launch_attention_mma<2>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
      case 3: return launch_attention_mma<3>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
      case 4: return launch_attention_mma<4>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
      case 5: return launch_attention_mma<5>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
      case 6: return launch_attention_mma<6>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
      case 7: return launch_attention_mma<7>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
      default: return launch_attention_mma<8>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
    }
  }
  switch (group) {
    case 1: return launch_attention<1>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
    case 2: return launch_attention<2>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
    case 3: return launch_attention<3>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
    default: return launch_attention<4>(q, k_cache, v_cache, pos, out, scratch, counters, batch, q_heads, kv_heads, max_len, splits, s);
  }
}
