// C entry points of the fused GEMV / skinny GEMM (the kernel itself: linear_lut_kernel.cuh,
// instantiated per code width in linear_lut_bits*.cu).
#include <cstring>
#include <mutex>

#include "linear_lut_params.cuh"
#include "tp_exchange.cuh"

namespace fdk {

static __device__ uint32_t g_smem_probe;  // where the probe kernel leaves its answer

namespace {
__global__ void probe_smem_base_kernel() {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  g_smem_probe = smem_addr(smem_raw);
}
}  // namespace

// Address, in the shared window, at which a kernel without static shared memory sees its
// dynamic shared memory.  Asked of the device once (the first call on a device runs a
// one-thread kernel and synchronises); nothing is allocated.
int dynamic_smem_base(uint32_t* out) {
  static uint32_t cache[64];
  static bool have[64] = {};
  static std::mutex mu;
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  dev &= 63;
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    probe_smem_base_kernel<<<1, 1, 1024>>>();
    FDK_CUDA(cudaGetLastError());
    FDK_CUDA(cudaMemcpyFromSymbol(&cache[dev], g_smem_probe, sizeof(uint32_t)));
    have[dev] = true;
  }
  *out = cache[dev];
  return FDK_OK;
}

}  // namespace fdk

using namespace fdk;

extern "C" int fdk_workspace_size(size_t* bytes_host) {
  FDK_CHECK_ARG(bytes_host != nullptr, FDK_ERR_BAD_ARG, "bytes_host is null");
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  *bytes_host = kWorkspaceBytes;
  return FDK_OK;
}

extern "C" int fdk_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  FDK_CHECK_ARG(workspace != nullptr, FDK_ERR_WORKSPACE, "workspace is null");
  FDK_CHECK_ARG(workspace_bytes >= kCounterBytes, FDK_ERR_WORKSPACE, "workspace of %zu bytes is too small", workspace_bytes);
  uint32_t base = 0;
  if (int st = dynamic_smem_base(&base)) return st;  // one-time device query, kept out of later captures
  FDK_CUDA(cudaMemsetAsync(workspace, 0, workspace_bytes, (cudaStream_t)stream));
  return FDK_OK;
}

extern "C" int fdk_workspace_status(const void* workspace, int* status_host) {
  FDK_CHECK_ARG(workspace != nullptr && status_host != nullptr, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CUDA(cudaMemcpy(status_host, (const int*)workspace + kStatusWord, sizeof(int), cudaMemcpyDeviceToHost));
  return FDK_OK;
}

static int linear_lut_impl(const void* x, const void* tiled, const void* lut, const void* lut_host, void* out,
                           int m, int n, int k, int bits, int dtype, void* workspace, size_t workspace_bytes,
                           unsigned flags, const fdk_tp_exchange* ex, const fdk_linear_fusion* fu, void* stream) {
  FDK_CHECK_ARG(m > 0 && n > 0 && k > 0, FDK_ERR_BAD_ARG, "m=%d, n=%d, k=%d must be positive", m, n, k);
  FDK_CHECK_ARG(bits_supported(bits), FDK_ERR_SHAPE, "bits=%d not in {1,2,3,4,8}", bits);
  FDK_CHECK_ARG(k % kBlock == 0, FDK_ERR_SHAPE, "k=%d must be a multiple of 64", k);
  const bool norm = fu != nullptr && fu->norm_h != nullptr;
  const bool resid = fu != nullptr && fu->resid_h != nullptr;
  const bool rope = fu != nullptr && fu->rope_pos != nullptr;
  FDK_CHECK_ARG((x || norm) && tiled && (lut || lut_host) && (out || ex || resid || rope), FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(dtype == FDK_DTYPE_BF16 || dtype == FDK_DTYPE_F16, FDK_ERR_BAD_ARG, "dtype=%d", dtype);
  FDK_CHECK_ARG((flags & ~(FDK_FLAG_PDL | FDK_FLAG_SILU_PAIRS)) == 0, FDK_ERR_BAD_ARG, "unknown flags 0x%x", flags);
  FDK_CHECK_ARG(!(flags & FDK_FLAG_SILU_PAIRS) || (ex == nullptr && m <= 16 && n % kTileRows == 0), FDK_ERR_SHAPE,
                "FDK_FLAG_SILU_PAIRS needs m <= 16 and n a multiple of 64 (m=%d, n=%d)", m, n);
  FDK_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)tiled & 15) == 0 && ((uintptr_t)lut & 15) == 0 &&
                    ((uintptr_t)out & 1) == 0,
                FDK_ERR_ALIGN, "x, tiled and lut must be 16-byte aligned");
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  FDK_CHECK_ARG(di.cc_major == 10, FDK_ERR_ARCH, "device has compute capability %d.%d", di.cc_major, di.cc_minor);
  const TiledDims d = tiled_dims(n, k, bits);
  FDK_CHECK_ARG(d.row_tiles < kStatusWord, FDK_ERR_SHAPE, "n=%d exceeds %d rows", n, kStatusWord * kTileRows);
  FDK_CHECK_ARG(di.sm_count <= 160, FDK_ERR_ARCH, "%d multiprocessors: the workspace layout provides for 160", di.sm_count);
  const size_t need = kCounterBytes + (size_t)di.sm_count * 1024 * sizeof(uint2);
  FDK_CHECK_ARG(workspace != nullptr && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                FDK_ERR_WORKSPACE, "workspace must be a 16-byte aligned buffer of at least %zu bytes", need);

  LinearParams p{};
  p.tiled = (const uint8_t*)tiled;
  p.lut = lut;
  p.counters = (int*)workspace;
  p.partial = (uint2*)((uint8_t*)workspace + kCounterBytes);
  p.n = n;
  p.k = k;
  p.k_slabs = d.k_slabs;
  p.total = d.row_tiles * d.k_slabs;
  p.k_magic = d.k_slabs > 1 ? (uint32_t)((((uint64_t)1 << 32) + d.k_slabs - 1) / d.k_slabs) : 0u;
  FDK_CHECK_ARG((uint64_t)p.total * d.k_slabs < ((uint64_t)1 << 32), FDK_ERR_SHAPE, "matrix of %d x %d slabs is too large", d.row_tiles, d.k_slabs);
  const int grid = di.sm_count;  // the launcher turns this into one or two CTAs per SM
  p.silu = (flags & FDK_FLAG_SILU_PAIRS) ? 1 : 0;
  if (ex != nullptr) {
    FDK_CHECK_ARG(ex->tp >= 1 && ex->tp <= kTpMaxRanks && ex->rank >= 0 && ex->rank < ex->tp, FDK_ERR_BAD_ARG,
                  "tp=%d, rank=%d", ex->tp, ex->rank);
    FDK_CHECK_ARG(m <= 16 && n % kTileRows == 0 && ex->slot_elems % 8 == 0 && (long long)m * n <= ex->slot_elems,
                  FDK_ERR_SHAPE, "push of m=%d, n=%d into slots of %lld elements (m <= 16, n %% 64 == 0)", m, n,
                  ex->slot_elems);
    p.tp = ex->tp;
    p.rank = ex->rank;
    p.stage_slot = ex->slot_elems;
    for (int j = 0; j < ex->tp; ++j) {
      FDK_CHECK_ARG(ex->buffers[j] != nullptr && ((uintptr_t)ex->buffers[j] & 255) == 0, FDK_ERR_ALIGN,
                    "exchange buffer %d must be a 256-byte aligned device pointer", j);
      p.peer_stage[j] = (uint2*)((uint8_t*)ex->buffers[j] + kTpStageOffset);
    }
    p.seq = (const uint32_t*)((const uint8_t*)ex->buffers[ex->rank] + kTpSeqOffset);
  }
  if (fu != nullptr) {
    FDK_CHECK_ARG(ex == nullptr && m <= 16 && dtype == FDK_DTYPE_BF16, FDK_ERR_SHAPE,
                  "the decode fusions take bf16 batches of up to 16 rows (m=%d)", m);
    FDK_CHECK_ARG(!(resid && rope) && !((resid || rope) && (flags & FDK_FLAG_SILU_PAIRS)), FDK_ERR_BAD_ARG,
                  "one output fusion at a time");
    if (norm) {
      FDK_CHECK_ARG(fu->norm_weight && fu->norm_sumsq && fu->norm_tiles > 0, FDK_ERR_BAD_ARG, "incomplete norm fusion");
      FDK_CHECK_ARG((((uintptr_t)fu->norm_h | (uintptr_t)fu->norm_weight) & 15) == 0, FDK_ERR_ALIGN,
                    "norm_h and norm_weight must be 16-byte aligned");
      p.norm_h = (const uint16_t*)fu->norm_h;
      p.norm_w = (const uint16_t*)fu->norm_weight;
      p.norm_ss = fu->norm_sumsq;
      p.norm_tiles = fu->norm_tiles;
      p.norm_eps = fu->norm_eps;
    }
    if (resid) {
      FDK_CHECK_ARG(fu->resid_sumsq != nullptr, FDK_ERR_BAD_ARG, "resid_sumsq is null");
      p.resid_h = (uint16_t*)fu->resid_h;
      p.resid_ss = fu->resid_sumsq;
      if (fu->resid_norm_weight != nullptr) {
        FDK_CHECK_ARG(fu->resid_x != nullptr, FDK_ERR_BAD_ARG, "resid_norm_weight without resid_x");
        p.resid_w = (const uint16_t*)fu->resid_norm_weight;
        p.resid_x = (uint16_t*)fu->resid_x;
      }
    } else {
      FDK_CHECK_ARG(fu->resid_norm_weight == nullptr, FDK_ERR_BAD_ARG, "resid_norm_weight goes with the residual output");
    }
    if (fu->scale_sumsq != nullptr) {
      FDK_CHECK_ARG(!norm, FDK_ERR_BAD_ARG, "the RMSNorm is applied to the input or to the output, not both");
      FDK_CHECK_ARG(fu->scale_tiles > 0, FDK_ERR_BAD_ARG, "scale_tiles=%d", fu->scale_tiles);
      p.scale_ss = fu->scale_sumsq;
      p.scale_tiles = fu->scale_tiles;
      p.scale_eps = fu->scale_eps;
    }
    if (rope) {
      FDK_CHECK_ARG(fu->rope_table && fu->q_out && fu->k_cache && fu->v_cache, FDK_ERR_BAD_ARG, "incomplete rotary fusion");
      FDK_CHECK_ARG(fu->q_heads > 0 && fu->kv_heads > 0 && fu->max_len > 0 && n == (fu->q_heads + 2 * fu->kv_heads) * 128,
                    FDK_ERR_SHAPE, "n=%d must be (q_heads + 2 kv_heads) * 128 (%d, %d)", n, fu->q_heads, fu->kv_heads);
      p.rope_pos = (const long long*)fu->rope_pos;
      p.rope_table = (const uint32_t*)fu->rope_table;
      p.q_out = (uint16_t*)fu->q_out;
      p.k_cache = (uint16_t*)fu->k_cache;
      p.v_cache = (uint16_t*)fu->v_cache;
      p.q_heads = fu->q_heads;
      p.kv_heads = fu->kv_heads;
      p.max_len = fu->max_len;
    }
  }
  // up to 16 rows the register path is the faster one (two n-tiles from 9 rows on: 19.5-21 us
  // at 8192^2 against 29-30 us for the tensor-core kernel and 26 us for bf16 cuBLAS)
  if (fu == nullptr && ex == nullptr && !(flags & FDK_FLAG_SILU_PAIRS) && m > 16) {
    return gemm_lut_tc(x, tiled, lut, lut_host, out, m, n, k, bits, dtype == FDK_DTYPE_F16, workspace, workspace_bytes,
                       di.sm_count,
                       (cudaStream_t)stream);
  }
  for (int m0 = 0; m0 < m; m0 += 16) {
    p.m = (m - m0) < 16 ? (m - m0) : 16;
    p.x = (const uint16_t*)x + (size_t)m0 * k;
    p.out = out ? (uint16_t*)out + (size_t)m0 * n : nullptr;
    int st;
    switch (bits) {
      case 1: st = launch_bits<1>(p, lut_host, grid, dtype, flags, (cudaStream_t)stream); break;
      case 2: st = launch_bits<2>(p, lut_host, grid, dtype, flags, (cudaStream_t)stream); break;
      case 3: st = launch_bits<3>(p, lut_host, grid, dtype, flags, (cudaStream_t)stream); break;
      case 4: st = launch_bits<4>(p, lut_host, grid, dtype, flags, (cudaStream_t)stream); break;
      default: st = launch_bits<8>(p, lut_host, grid, dtype, flags, (cudaStream_t)stream); break;
    }
    if (st) return st;
  }
  return FDK_OK;
}

extern "C" int fdk_linear_lut(const void* x, const void* tiled, const void* lut, const void* lut_host,
                              void* out, int m, int n, int k, int bits, int dtype, void* workspace,
                              size_t workspace_bytes, unsigned flags, void* stream) {
  FDK_CHECK_ARG(out != nullptr, FDK_ERR_BAD_ARG, "null pointer");
  return linear_lut_impl(x, tiled, lut, lut_host, out, m, n, k, bits, dtype, workspace, workspace_bytes, flags,
                         nullptr, nullptr, stream);
}

// fdk_linear_lut_host moves its few kilobytes of activations with a kernel of its own where it
// can: a DMA copy of 16 KB costs ~8 us on the stream, a kernel reading or writing page-locked
// host memory through its device mapping ~3 us, and it takes part in programmatic dependent
// launch (the projection's weight prefetch overlaps the copy in).  Host memory that is not
// page-locked and mapped (cudaPointerGetAttributes says so) is copied by cudaMemcpyAsync.
namespace fdk {
namespace hostcopy {

__global__ void host_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int vectors) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vectors; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// The device's address of page-locked, mapped host memory, or null.
void* mapped_host_pointer(const void* host) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

int launch_host_copy(const void* src, void* dst, size_t bytes, cudaStream_t stream) {
  const int vectors = (int)(bytes / 16);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((vectors + 255) / 256 < 8 ? (vectors + 255) / 256 : 8);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FDK_CUDA(cudaLaunchKernelEx(&cfg, host_copy_kernel, (const uint4*)src, (uint4*)dst, vectors));
  return FDK_OK;
}

constexpr size_t kHostCopyKernelLimit = 256 * 1024;  // larger activations: the DMA engine's bandwidth wins

}  // namespace hostcopy
}  // namespace fdk
using namespace fdk::hostcopy;

extern "C" int fdk_linear_lut_host(const void* x_host, const void* tiled, const void* lut, const void* lut_host,
                                   void* out_host, int m, int n, int k, int bits, int dtype, void* x_dev, void* out_dev,
                                   void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
  FDK_CHECK_ARG(x_host && out_host && x_dev && out_dev, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(m > 0 && n > 0 && k > 0, FDK_ERR_BAD_ARG, "m=%d, n=%d, k=%d must be positive", m, n, k);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t x_bytes = (size_t)m * k * 2, out_bytes = (size_t)m * n * 2;
  auto by_kernel = [](const void* host, const void* dev, size_t bytes) -> void* {
    if (bytes > kHostCopyKernelLimit || bytes % 16 != 0 || (((uintptr_t)host | (uintptr_t)dev) & 15) != 0) return nullptr;
    return mapped_host_pointer(host);
  };
  void* x_mapped = by_kernel(x_host, x_dev, x_bytes);
  void* out_mapped = by_kernel(out_host, out_dev, out_bytes);
  if (x_mapped != nullptr) {
    if (int st = launch_host_copy(x_mapped, x_dev, x_bytes, s)) return st;
  } else {
    FDK_CUDA(cudaMemcpyAsync(x_dev, x_host, x_bytes, cudaMemcpyHostToDevice, s));
  }
  // behind a kernel the projection may start early: it only reads weights before it waits
  const unsigned inner = (flags & ~FDK_FLAG_NO_SYNC) | (x_mapped != nullptr ? FDK_FLAG_PDL : 0u);
  // The result is written once and never read back by the kernels: into mapped host memory the
  // projection stores it itself (posted writes over PCIe), which saves a copy per call.  x is
  // read by every CTA and does need its copy in device memory.
  void* out = out_mapped != nullptr ? out_mapped : out_dev;
  if (int st = linear_lut_impl(x_dev, tiled, lut, lut_host, out, m, n, k, bits, dtype, workspace, workspace_bytes,
                               inner, nullptr, nullptr, stream)) {
    return st;
  }
  if (out_mapped == nullptr) FDK_CUDA(cudaMemcpyAsync(out_host, out_dev, out_bytes, cudaMemcpyDeviceToHost, s));
  if (!(flags & FDK_FLAG_NO_SYNC)) FDK_CUDA(cudaStreamSynchronize(s));
  return FDK_OK;
}

extern "C" int fdk_linear_lut_fused(const void* x, const void* tiled, const void* lut, const void* lut_host, void* out,
                                    int m, int n, int k, int bits, int dtype, void* workspace, size_t workspace_bytes,
                                    unsigned flags, const fdk_linear_fusion* fusion, void* stream) {
  FDK_CHECK_ARG(fusion != nullptr, FDK_ERR_BAD_ARG, "fusion is null");
  return linear_lut_impl(x, tiled, lut, lut_host, out, m, n, k, bits, dtype, workspace, workspace_bytes, flags,
                         nullptr, fusion, stream);
}

extern "C" int fdk_linear_norm_fits(int m, int k, int bits, int* fits_host) {
  FDK_CHECK_ARG(fits_host != nullptr, FDK_ERR_BAD_ARG, "fits_host is null");
  *fits_host = 0;
  if (m <= 0 || m > 16 || k <= 0 || k % kBlock != 0 || !bits_supported(bits)) return FDK_OK;
  switch (bits) {
    case 1: return norm_fits_bits<1>(m, k, fits_host);
    case 2: return norm_fits_bits<2>(m, k, fits_host);
    case 3: return norm_fits_bits<3>(m, k, fits_host);
    case 4: return norm_fits_bits<4>(m, k, fits_host);
    default: return norm_fits_bits<8>(m, k, fits_host);
  }
}

extern "C" int fdk_linear_lut_push(const void* x, const void* tiled, const void* lut, const void* lut_host, int m,
                                   int n, int k, int bits, int dtype, void* workspace, size_t workspace_bytes,
                                   unsigned flags, const fdk_tp_exchange* ex, void* stream) {
  FDK_CHECK_ARG(ex != nullptr, FDK_ERR_BAD_ARG, "exchange is null");
  return linear_lut_impl(x, tiled, lut, lut_host, nullptr, m, n, k, bits, dtype, workspace, workspace_bytes, flags,
                         ex, nullptr, stream);
}

// ---- entry point that allocates nothing ---------------------------------------------------
// Some callers cannot give fdk_linear_lut a workspace because they cannot allocate device
// memory at the point of the call: a plugin living inside a host runtime that owns every
// device allocation, or code that runs while a stream capture is open in a mode that
// forbids cudaMalloc.  For them the scratch lives in this library's own image: a file-scope
// device array, sized for GPUs of up to kStaticMaxSms multiprocessors, that every GPU which
// loads the library holds until the process exits.
constexpr int kStaticMaxSms = 160;
constexpr size_t kStaticScratchBytes = kCounterBytes + (size_t)kStaticMaxSms * 1024 * sizeof(uint2);  // 1,327,104
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// The array's address on the current device (looked up once per device; nothing is allocated).
static int static_scratch(void** out) {
  static void* scratch_of_device[64] = {};
  static std::mutex mu;
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  FDK_CHECK_ARG(dev >= 0 && dev < 64, FDK_ERR_BAD_ARG, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (scratch_of_device[dev] == nullptr) {
    // In host code `g_static_scratch` is only a handle for the symbol; the kernel needs the
    // array's address on the CURRENT device.
    void* ptr = nullptr;
    FDK_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    scratch_of_device[dev] = ptr;  // zero-filled when the module was loaded: nothing to clear
  }
  *out = scratch_of_device[dev];
  return FDK_OK;
}

extern "C" int fdk_linear_lut_static(const void* x, const void* tiled, const void* lut, const void* lut_host,
                                     void* out, int m, int n, int k, int bits, int dtype, unsigned flags,
                                     void* stream) {
  void* scratch = nullptr;
  if (int st = static_scratch(&scratch)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  const size_t need = kCounterBytes + (size_t)di.sm_count * 1024 * sizeof(uint2);
  FDK_CHECK_ARG(need <= kStaticScratchBytes, FDK_ERR_WORKSPACE,
                "this GPU has %d multiprocessors and needs %zu bytes of scratch; the built-in scratch holds %zu "
                "(up to %d multiprocessors): use fdk_linear_lut with a caller-allocated workspace",
                di.sm_count, need, kStaticScratchBytes, kStaticMaxSms);
  return fdk_linear_lut(x, tiled, lut, lut_host, out, m, n, k, bits, dtype, scratch, kStaticScratchBytes, flags, stream);
}

extern "C" int fdk_static_status(int* status_host) {
  FDK_CHECK_ARG(status_host != nullptr, FDK_ERR_BAD_ARG, "null pointer");
  void* scratch = nullptr;
  if (int st = static_scratch(&scratch)) return st;
  FDK_CUDA(cudaMemcpy(status_host, (const int*)scratch + kStatusWord, sizeof(int), cudaMemcpyDeviceToHost));
  return FDK_OK;
}
