// Device helpers shared by the fused kernels: shared-memory addressing, bulk asynchronous
// copies with bounded barrier waits, the per-lane replicated lookup table and the
// m16n8k16 MMA wrapper.
#pragma once
#include <type_traits>

#include "fdk_common.cuh"

namespace fdk {

constexpr uint32_t kWaitLimit = 1u << 22;  // try_wait rounds before giving up (seconds, not microseconds)

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

template <uint32_t SEL>
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "n"(SEL));
  return d;
}

// Table lookups: pure functions of the address once the table is filled (it never
// changes afterwards), so the compiler may schedule them freely.
__device__ __forceinline__ uint32_t lut32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lut64(uint32_t addr) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lut128(uint32_t addr) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// Ring reads: ordered after the barrier wait that precedes them.
__device__ __forceinline__ uint4 ring128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Waits for the phase with the given parity; gives up after kWaitLimit rounds or two seconds,
// whichever comes first.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((i & 1023u) == 1023u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) return false;
    }
  }
  return false;
}

template <bool FP16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                         const float (&c)[4]) {
  if constexpr (FP16) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
  }
}

template <int I>
__device__ __forceinline__ uint32_t word_of(const uint4& v) {
  if constexpr (I == 0) return v.x;
  else if constexpr (I == 1) return v.y;
  else if constexpr (I == 2) return v.z;
  else return v.w;
}
__device__ __forceinline__ uint32_t word_at(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// ---- lookup tables in shared memory -----------------------------------------
// Replicated so that lookups never conflict: entry e lives in the 128-byte row  base + 128 * e,
// once per lane of the group of lanes that one shared-memory wavefront serves -- 32 lanes for
// 4-byte entries, a half warp for 8-byte entries, a quarter warp for 16-byte entries -- at
// offset (lane % kReplicas) * kEntryBytes.  Whatever code bytes the lanes hold, the lanes of a
// wavefront read 128 different bytes' worth of banks.  A lookup address is one PRMT (extract
// the code byte) and one multiply-add.
//
// WIDE: rows 256 bytes apart (the second half of each row unused) in a table that starts at a
// multiple of 64 KB in the shared window.  The address of an entry is then the table's address
// with the code byte put into bits 8..15: one PRMT, no arithmetic (64 KB instead of 32 KB;
// not for 3 bits, whose 6-bit fields are not bytes).
template <int BITS, bool WIDE = false>
struct Table {
  static_assert(!(WIDE && BITS == 3), "3-bit codes use the compact table");
  static constexpr int kEntries = (BITS == 3) ? 64 : 256;
  static constexpr int kEntryBytes = (BITS == 2) ? 8 : (BITS == 1 ? 16 : 4);
  static constexpr int kReplicas = 128 / kEntryBytes;
  static constexpr int kStride = WIDE ? 256 : 128;
  static constexpr int kBytes = kEntries * kStride;  // 32 KB (64 KB wide), or 8 KB for 3 bits
  __device__ static __forceinline__ uint32_t lane_offset(int lane) { return (lane % kReplicas) * kEntryBytes; }
};

// The byte table may travel inside the kernel parameters (no memory latency at all) or be
// read from device memory.  16-bit entries, packed two per word.
template <int BITS>
struct InlineLut {
  static constexpr int kWords = (BITS == 3) ? 4 : 256 * (8 / BITS) / 2;
  uint32_t w[kWords];
};

// Fills the replicated table: one 128-byte row per warp and iteration, lane l writing word l
// of the row (replica l * 4 / kEntryBytes of the entry, its word l % (kEntryBytes / 4)).
// `threads` (a multiple of 32) threads numbered `tid` take part; word(i) returns 32-bit word
// i of the source table.
template <int BITS, bool WIDE = false, class WordFn>
__device__ __forceinline__ void fill_table(uint32_t table_base, int threads, WordFn word, int tid) {
  using T = Table<BITS, WIDE>;
  const int lane = tid & 31, warps = threads >> 5;
#pragma unroll 1
  for (int e = tid >> 5; e < T::kEntries; e += warps) {
    uint32_t v;
    if constexpr (BITS == 4) {
      v = word(e);
    } else if constexpr (BITS == 2) {
      v = word(2 * e + (lane & 1));
    } else if constexpr (BITS == 1) {
      v = word(4 * e + (lane & 3));
    } else if constexpr (BITS == 8) {
      const uint32_t pair = word(e >> 1);
      const uint32_t h = (e & 1) ? (pair >> 16) : (pair & 0xFFFFu);
      v = h | (h << 16);
    } else {  // 3 bits: pair table from the 8-entry codebook, first code in the high 3 index bits
      auto code = [&](int c) {
        const uint32_t pair = word(c >> 1);
        return (c & 1) ? (pair >> 16) : (pair & 0xFFFFu);
      };
      v = code(e >> 3) | (code(e & 7) << 16);
    }
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(table_base + e * T::kStride + lane * 4), "r"(v) : "memory");
  }
}

// The same with a thread count known at compile time: all the source words of a thread are
// fetched before the first is stored, so a thread pays the latency of the source once.
template <int BITS, bool WIDE, int THREADS, class WordFn>
__device__ __forceinline__ void fill_table_unrolled(uint32_t table_base, WordFn word, int tid) {
  using T = Table<BITS, WIDE>;
  static_assert(BITS == 4 || BITS == 2 || BITS == 1, "byte tables of 4-, 2- and 1-bit codes");
  constexpr int kWarps = THREADS / 32;
  constexpr int kRounds = (T::kEntries + kWarps - 1) / kWarps;
  constexpr int kWordsPerEntry = T::kEntryBytes / 4;
  const int lane = tid & 31, warp = tid >> 5;
  uint32_t v[kRounds];
#pragma unroll
  for (int i = 0; i < kRounds; ++i) {
    const int e = warp + i * kWarps;
    v[i] = e < T::kEntries ? word(kWordsPerEntry * e + (lane & (kWordsPerEntry - 1))) : 0u;
  }
#pragma unroll
  for (int i = 0; i < kRounds; ++i) {
    const int e = warp + i * kWarps;
    if (e < T::kEntries)
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(table_base + e * T::kStride + lane * 4), "r"(v[i]) : "memory");
  }
}

// Address of the table entry selected by byte J of `w` (lane_base = table base + lane offset).
template <int BITS, int J, bool WIDE = false>
__device__ __forceinline__ uint32_t entry_addr(uint32_t w, uint32_t lane_base) {
  if constexpr (WIDE) {  // byte J of w into byte 1 of the lane's table address
    return prmt<0x3200u | ((4u + J) << 4)>(lane_base, w);
  } else {
    const uint32_t b = prmt<0x4440u | J>(w, 0u);  // the byte alone
    return lane_base + b * (uint32_t)Table<BITS>::kStride;
  }
}

template <int BITS, bool WIDE = false, class WordFn>
__device__ __forceinline__ void fill_table(uint32_t table_base, WordFn word) {
  fill_table<BITS, WIDE>(table_base, (int)blockDim.x, word, (int)threadIdx.x);
}

__device__ __forceinline__ uint2 ld_relaxed_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.gpu.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_v2(uint2* p, uint2 v) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ int ld_relaxed_s32(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}


// ---- workspace layout (bytes) -----------------------------------------------------------------
//   [0, 16 KB)            use counts of split row tiles (4095 ints) + the status word
//   [16 KB, kGemvEnd)     tagged partial sums of the GEMV kernel, 8 KB per SM, room for 160 SMs
//   then 8 KB of flags and 8 KB of tile use counts of the tensor-core GEMM
//   then its fp32 partial tiles: up to 148 tiles of 128 rows x 256 batch columns
constexpr size_t kCounterBytes = 16384;
constexpr int kStatusWord = 4095;
constexpr size_t kGemvEnd = kCounterBytes + (size_t)160 * 1024 * sizeof(uint2);
constexpr size_t kTcFlagsOffset = kGemvEnd;
constexpr size_t kTcUsesOffset = kGemvEnd + 8192;
constexpr size_t kTcPartialOffset = kGemvEnd + 16384;
constexpr size_t kTcPartialTileBytes = (size_t)128 * 256 * sizeof(float);
constexpr size_t kWorkspaceBytes = kTcPartialOffset + 148 * kTcPartialTileBytes;

// Tensor-core GEMM for batches above 8 rows (gemm_lut_tc.cu).
int gemm_lut_tc(const void* x, const void* tiled, const void* lut, const void* lut_host, void* out, int m, int n,
                int k, int bits, bool fp16, void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream);

// The dynamic shared memory address seen by kernels without static shared memory, asked of
// the device once (linear_lut.cu).
int dynamic_smem_base(uint32_t* out);

}  // namespace fdk
