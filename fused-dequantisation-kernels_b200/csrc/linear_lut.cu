// Fused dequantise + GEMV / skinny GEMM for sm_100a:  out[m, n] = x[m, k] . W[n, k]^T,
// W given as tiled low-bit codes + block scales + a lookup table (fdk_layout.cuh).
//
// Shape of the kernel (one persistent CTA per SM, 16 warps):
//   * The weight stream is cut into slabs (64 rows x 64*KSB columns, ~2-6 KB).  The
//     slabs of the whole matrix form one linear sequence (row tile major); CTA c owns
//     a contiguous range of it ("stream-K"), its warps take slabs round-robin.  Every
//     SM therefore streams the same number of bytes (+-1 slab) whatever N and K are.
//   * A warp keeps kDepth slabs in flight as 16-byte-per-lane global loads straight
//     into registers (512 contiguous bytes per load instruction, no L1 allocation).
//   * Codes are turned into tensor-core A fragments by table lookup in shared memory:
//     one code byte indexes a per-lane replica of the byte table, so a lookup is one
//     PRMT (byte -> address) and one conflict-free LDS that returns 2 (4-bit), 4
//     (2-bit) or 8 (1-bit) 16-bit weights already in fragment order.  x is the B
//     operand (batch padded to 8 or 16 columns), read through L1.
//   * mma.sync m16n8k16 accumulates one 64-block in fp32; the block scale multiplies
//     the fp32 block sum (4 FMAs per 1024 weights), then running totals per row.
//     The tensor pipe is used because the FMA work would otherwise compete with the
//     lookups for issue slots; at m <= 16 it is far from being the limiter, so the
//     synchronous MMA form is enough and keeps the weights in registers (a tcgen05
//     MMA would need them written back to shared or tensor memory first).
//   * At a row-tile boundary the warps of a CTA reduce through shared memory in a
//     fixed order.  A CTA that owns only part of a row tile's K range writes its
//     partial sums to the workspace and bumps an arrival counter; the last arriver
//     adds the partials in CTA order and writes the result.  No spinning, and the
//     summation order never depends on timing, so results are reproducible.
#include <type_traits>

#include "fdk_common.cuh"

namespace fdk {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
// Slabs in flight per warp: as many as the register file allows for the slab size.
template <int BITS, int NB>
__host__ __device__ constexpr int depth_for() {
  if (BITS == 4) return NB == 1 ? 3 : 2;
  if (BITS == 2) return 2;
  if (BITS == 1) return NB == 1 ? 2 : 1;
  return 1;
}

struct LinearParams {
  const uint8_t* tiled;
  const void* lut;
  const uint16_t* x;
  uint16_t* out;
  float* partial;  // [grid][2][512 * NB]
  int* counters;   // [row_tiles], zero between launches
  int m, n, k;
  int k_slabs;     // slabs per row tile
  int total;       // row_tiles * k_slabs
  int base, rem;   // CTA c owns `base + (c < rem)` consecutive slabs
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ldg_l1(const void* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <uint32_t SEL>
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "n"(SEL));
  return d;
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

template <bool FP16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (FP16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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
// Per-lane replicas: entry e of lane l lives at  base + e * kStride + l * kEntryBytes,
// so that the 32 lanes of a warp always hit 32 different banks (or, for 8/16-byte
// entries, every quarter / half warp does).  For the 256-byte stride the base is
// 64 KB aligned inside the shared window: the address of entry `byte` is then the
// lane's base with `byte` dropped into bits 8..15, which is a single PRMT.
template <int BITS>
struct Table {
  static constexpr int kEntries = (BITS == 3) ? 64 : 256;
  static constexpr int kEntryBytes = (BITS == 2) ? 8 : (BITS == 1 ? 16 : 4);
  static constexpr int kStride = (BITS == 1) ? 512 : 256;
  static constexpr int kBytes = kEntries * kStride;
  static constexpr bool kAligned64K = (BITS != 1);
};

template <int BITS, bool FP16>
__device__ void fill_table(uint32_t table_base, const void* lut) {
  using T = Table<BITS>;
  for (int idx = threadIdx.x; idx < T::kEntries * 32; idx += kThreads) {
    int e = idx >> 5, l = idx & 31;
    uint32_t addr = table_base + e * T::kStride + l * T::kEntryBytes;
    if constexpr (BITS == 4) {
      uint32_t v = reinterpret_cast<const uint32_t*>(lut)[e];
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v));
    } else if constexpr (BITS == 2) {
      uint2 v = reinterpret_cast<const uint2*>(lut)[e];
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(v.x), "r"(v.y));
    } else if constexpr (BITS == 1) {
      uint4 v = reinterpret_cast<const uint4*>(lut)[e];
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w));
    } else if constexpr (BITS == 8) {
      uint32_t v = reinterpret_cast<const uint16_t*>(lut)[e];
      v |= v << 16;
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v));
    } else {  // 3 bits: pair table from the 8-entry codebook, first code in the high 3 index bits
      const uint16_t* cb = reinterpret_cast<const uint16_t*>(lut);
      uint32_t v = (uint32_t)cb[e >> 3] | ((uint32_t)cb[e & 7] << 16);
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v));
    }
  }
}

// Address of the table entry selected by byte J of `w` (lane_base = table base + lane offset).
template <int BITS, int J>
__device__ __forceinline__ uint32_t entry_addr(uint32_t w, uint32_t lane_base) {
  if constexpr (BITS == 1) {
    uint32_t b = prmt<0x4404u | (J << 4)>(w, 0u);  // byte << 8
    return lane_base + (b << 1);                    // stride 512
  } else {
    return prmt<0x7604u | (J << 4)>(w, lane_base);  // bits 8..15 <- byte
  }
}

// ---- one slab in registers ----------------------------------------------------
template <int BITS>
struct Slab {
  using L = Layout<BITS>;
  uint4 code[kSubTiles * L::V];
  uint4 sc[L::KSB];
};

template <int BITS>
__device__ __forceinline__ void load_slab(Slab<BITS>& s, const uint8_t* slab, int lane) {
  using L = Layout<BITS>;
#pragma unroll
  for (int i = 0; i < kSubTiles * L::V; ++i) s.code[i] = ldg_stream(slab + (i * 32 + lane) * 16);
#pragma unroll
  for (int jb = 0; jb < L::KSB; ++jb) s.sc[jb] = ldg_stream(slab + L::kCodeBytes + jb * 128 + (lane >> 2) * 16);
}

// A fragments of sub-tile R for the four MMA k-steps of 64-block JB.
//   a[s][0] = row g,   elements 4s, 4s+1      a[s][1] = row g+8, elements 4s, 4s+1
//   a[s][2] = row g,   elements 4s+2, 4s+3    a[s][3] = row g+8, elements 4s+2, 4s+3
// (elements counted inside the lane's 16-element share of the block; x is read
// with the same numbering, so the product does not depend on it).
template <int BITS, int R, int JB>
__device__ __forceinline__ void build_fragments(const Slab<BITS>& s, uint32_t lane_base, uint32_t (&a)[4][4]) {
  using L = Layout<BITS>;
  if constexpr (BITS == 4) {
    const uint4& c = s.code[R];
    a[0][0] = lds32(entry_addr<4, 0>(c.x, lane_base)); a[0][2] = lds32(entry_addr<4, 1>(c.x, lane_base));
    a[1][0] = lds32(entry_addr<4, 2>(c.x, lane_base)); a[1][2] = lds32(entry_addr<4, 3>(c.x, lane_base));
    a[2][0] = lds32(entry_addr<4, 0>(c.y, lane_base)); a[2][2] = lds32(entry_addr<4, 1>(c.y, lane_base));
    a[3][0] = lds32(entry_addr<4, 2>(c.y, lane_base)); a[3][2] = lds32(entry_addr<4, 3>(c.y, lane_base));
    a[0][1] = lds32(entry_addr<4, 0>(c.z, lane_base)); a[0][3] = lds32(entry_addr<4, 1>(c.z, lane_base));
    a[1][1] = lds32(entry_addr<4, 2>(c.z, lane_base)); a[1][3] = lds32(entry_addr<4, 3>(c.z, lane_base));
    a[2][1] = lds32(entry_addr<4, 0>(c.w, lane_base)); a[2][3] = lds32(entry_addr<4, 1>(c.w, lane_base));
    a[3][1] = lds32(entry_addr<4, 2>(c.w, lane_base)); a[3][3] = lds32(entry_addr<4, 3>(c.w, lane_base));
  } else if constexpr (BITS == 2) {
    const uint4& c = s.code[R];
    const uint32_t wg = word_of<2 * JB>(c), wh = word_of<2 * JB + 1>(c);
    uint2 q;
    q = lds64(entry_addr<2, 0>(wg, lane_base)); a[0][0] = q.x; a[0][2] = q.y;
    q = lds64(entry_addr<2, 1>(wg, lane_base)); a[1][0] = q.x; a[1][2] = q.y;
    q = lds64(entry_addr<2, 2>(wg, lane_base)); a[2][0] = q.x; a[2][2] = q.y;
    q = lds64(entry_addr<2, 3>(wg, lane_base)); a[3][0] = q.x; a[3][2] = q.y;
    q = lds64(entry_addr<2, 0>(wh, lane_base)); a[0][1] = q.x; a[0][3] = q.y;
    q = lds64(entry_addr<2, 1>(wh, lane_base)); a[1][1] = q.x; a[1][3] = q.y;
    q = lds64(entry_addr<2, 2>(wh, lane_base)); a[2][1] = q.x; a[2][3] = q.y;
    q = lds64(entry_addr<2, 3>(wh, lane_base)); a[3][1] = q.x; a[3][3] = q.y;
  } else if constexpr (BITS == 1) {
    const uint32_t w = word_of<JB>(s.code[R]);  // bytes 0,1: row g; bytes 2,3: row g+8
    uint4 q;
    q = lds128(entry_addr<1, 0>(w, lane_base)); a[0][0] = q.x; a[0][2] = q.y; a[1][0] = q.z; a[1][2] = q.w;
    q = lds128(entry_addr<1, 1>(w, lane_base)); a[2][0] = q.x; a[2][2] = q.y; a[3][0] = q.z; a[3][2] = q.w;
    q = lds128(entry_addr<1, 2>(w, lane_base)); a[0][1] = q.x; a[0][3] = q.y; a[1][1] = q.z; a[1][3] = q.w;
    q = lds128(entry_addr<1, 3>(w, lane_base)); a[2][1] = q.x; a[2][3] = q.y; a[3][1] = q.z; a[3][3] = q.w;
  } else if constexpr (BITS == 8) {
    const uint4& cg = s.code[R * 2];      // row g: 16 bytes = 16 elements
    const uint4& ch = s.code[R * 2 + 1];  // row g+8
#pragma unroll
    for (int st = 0; st < 4; ++st) {
      const uint32_t wg = word_at(cg, st), wh = word_at(ch, st);
      a[st][0] = prmt<0x7610>(lds32(entry_addr<8, 0>(wg, lane_base)), lds32(entry_addr<8, 1>(wg, lane_base)));
      a[st][2] = prmt<0x7610>(lds32(entry_addr<8, 2>(wg, lane_base)), lds32(entry_addr<8, 3>(wg, lane_base)));
      a[st][1] = prmt<0x7610>(lds32(entry_addr<8, 0>(wh, lane_base)), lds32(entry_addr<8, 1>(wh, lane_base)));
      a[st][3] = prmt<0x7610>(lds32(entry_addr<8, 2>(wh, lane_base)), lds32(entry_addr<8, 3>(wh, lane_base)));
    }
  } else {  // 3 bits: 96-bit little-endian group per block, pair field f at bits [6f, 6f+6)
    uint32_t w[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      constexpr int kWordsPerVec = 4;
      const int wi = 3 * JB + i;
      w[i] = word_at(s.code[R * L::V + wi / kWordsPerVec], wi % kWordsPerVec);
    }
#pragma unroll
    for (int f = 0; f < 16; ++f) {
      const int o = 6 * f;            // bit offset of the field
      const int wi = o >> 5, sh = o & 31;
      uint32_t v;
      if (sh + 6 <= 32) {
        // want field << 8: shift right by sh-8 (or left by 8-sh)
        v = (sh >= 8) ? (w[wi] >> (sh - 8)) : (w[wi] << (8 - sh));
      } else {
        v = __funnelshift_r(w[wi], w[wi + 1], sh - 8);
      }
      uint32_t addr = (v & 0x3F00u) | lane_base;
      const int p = f & 7, half = f >> 3;
      a[p >> 1][(p & 1) * 2 + half] = lds32(addr);
    }
  }
}

// ---- the kernel -------------------------------------------------------------------
template <int NB, bool FP16>
__device__ __noinline__ void segment_reduce(const LinearParams& p, float* slots, int rt, int c0, int c1,
                                            int* flag) {
  constexpr int E = 512 * NB;  // outputs of one row tile: 64 rows x (8 * NB) batch columns
  const int seg_lo = rt * p.k_slabs, seg_hi = seg_lo + p.k_slabs;
  const bool full = (c0 <= seg_lo) && (c1 >= seg_hi);
  __syncthreads();  // every warp has deposited its totals
  float sums[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    // element e = nb * 512 + threadIdx.x  <->  slot word (r * NB + nb) * 128 + lane * 4 + c
    const int r = threadIdx.x >> 7, rem = threadIdx.x & 127;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) acc += slots[((w * kSubTiles + r) * NB + nb) * 128 + rem];
    sums[nb] = acc;
  }
  bool write_out = full;
  if (!full) {
    const int cta = blockIdx.x;
    const int slot = (rt == c0 / p.k_slabs) ? 0 : 1;
    float* mine = p.partial + ((size_t)cta * 2 + slot) * E;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) __stcg(mine + nb * 512 + threadIdx.x, sums[nb]);
    __threadfence();
    __syncthreads();
    // which CTAs share this row tile: those owning slab seg_lo .. seg_hi-1
    const int big = p.rem * (p.base + 1);
    auto owner = [&](int item) { return item < big ? item / (p.base + 1) : p.rem + (item - big) / p.base; };
    const int first = owner(seg_lo), last = owner(seg_hi - 1);
    if (threadIdx.x == 0) {
      int old = atomicAdd(p.counters + rt, 1);
      *flag = (old == last - first) ? 1 : 0;
    }
    __syncthreads();
    if (*flag) {
      __threadfence();
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) sums[nb] = 0.f;
      for (int c = first; c <= last; ++c) {
        const int cs = c * p.base + min(c, p.rem);  // first slab of CTA c
        const int sl = (rt == cs / p.k_slabs) ? 0 : 1;
        const float* theirs = p.partial + ((size_t)c * 2 + sl) * E;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) sums[nb] += __ldcg(theirs + nb * 512 + threadIdx.x);
      }
      if (threadIdx.x == 0) p.counters[rt] = 0;  // leave the workspace clean for the next launch
      write_out = true;
    }
  }
  if (write_out) {
    const int r = threadIdx.x >> 7, lane = (threadIdx.x >> 2) & 31, c = threadIdx.x & 3;
    const int row = rt * kTileRows + 16 * r + (lane >> 2) + 8 * (c >> 1);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int b = 8 * nb + 2 * (lane & 3) + (c & 1);
      if (row < p.n && b < p.m) p.out[(size_t)b * p.n + row] = from_float<FP16>(sums[nb]);
    }
  }
  __syncthreads();  // slots may be overwritten after this
}

template <int BITS, int NB, bool FP16>
__global__ void __launch_bounds__(kThreads, 1) linear_lut_kernel(const __grid_constant__ LinearParams p) {
  using L = Layout<BITS>;
  using T = Table<BITS>;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ int flag;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  // shared-memory carve-up: [pad to 64 KB][table][reduction slots]
  const uint32_t raw = smem_addr(smem_raw);
  const uint32_t table_base = T::kAligned64K ? ((raw + 0xFFFFu) & ~0xFFFFu) : ((raw + 15u) & ~15u);
  float* slots = reinterpret_cast<float*>(smem_raw + (table_base - raw) + T::kBytes);
  const uint32_t lane_base = table_base + lane * T::kEntryBytes;

  // my slab range
  const int cta = blockIdx.x;
  const int c0 = cta * p.base + min(cta, p.rem);
  const int c1 = c0 + p.base + (cta < p.rem ? 1 : 0);

  // start streaming before anything else
  constexpr int kDepth = depth_for<BITS, NB>();
  Slab<BITS> buf[kDepth];
  int it = c0 + warp;
#pragma unroll
  for (int d = 0; d < kDepth; ++d) {
    const int i = it + d * kWarps;
    if (i < c1) load_slab<BITS>(buf[d], p.tiled + (size_t)i * L::kSlabBytes, lane);
  }
  fill_table<BITS, FP16>(table_base, p.lut);
  // everything above reads only weights; x, out and the workspace belong to the stream order
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();

  float tot[kSubTiles][NB][4];
#pragma unroll
  for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) tot[r][nb][i] = 0.f;

  const int rt_first = c0 / p.k_slabs;
  const int rt_last = (c1 - 1) / p.k_slabs;
  int cur_rt = rt_first;

  auto flush_until = [&](int target) {
    while (cur_rt < target) {
#pragma unroll
      for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          float4 v = make_float4(tot[r][nb][0], tot[r][nb][1], tot[r][nb][2], tot[r][nb][3]);
          *reinterpret_cast<float4*>(slots + ((warp * kSubTiles + r) * NB + nb) * 128 + lane * 4) = v;
          tot[r][nb][0] = tot[r][nb][1] = tot[r][nb][2] = tot[r][nb][3] = 0.f;
        }
      segment_reduce<NB, FP16>(p, slots, cur_rt, c0, c1, &flag);
      ++cur_rt;
    }
  };

  auto compute = [&](const Slab<BITS>& s, int ks) {
    auto block = [&](auto jbc) {
      constexpr int JB = decltype(jbc)::value;
      const int kb = (ks * L::KSB + JB) * kBlock;
      uint32_t xb[NB][8];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const int b = g + 8 * nb;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (b < p.m && kb < p.k) {
          const uint16_t* src = p.x + (size_t)b * p.k + kb + 16 * t;
          lo = ldg_l1(src);
          hi = ldg_l1(src + 8);
        }
        xb[nb][0] = lo.x; xb[nb][1] = lo.y; xb[nb][2] = lo.z; xb[nb][3] = lo.w;
        xb[nb][4] = hi.x; xb[nb][5] = hi.y; xb[nb][6] = hi.z; xb[nb][7] = hi.w;
      }
      auto sub_tile = [&](auto rc) {
        constexpr int R = decltype(rc)::value;
        uint32_t a[4][4];
        build_fragments<BITS, R, JB>(s, lane_base, a);
        const uint32_t scw = word_of<R>(s.sc[JB]);
        const float s_lo = pair_lo<FP16>(scw), s_hi = pair_hi<FP16>(scw);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int st = 0; st < 4; ++st) mma16816<FP16>(acc, a[st], xb[nb][2 * st], xb[nb][2 * st + 1]);
          tot[R][nb][0] += acc[0] * s_lo;
          tot[R][nb][1] += acc[1] * s_lo;
          tot[R][nb][2] += acc[2] * s_hi;
          tot[R][nb][3] += acc[3] * s_hi;
        }
      };
      sub_tile(std::integral_constant<int, 0>{});
      sub_tile(std::integral_constant<int, 1>{});
      sub_tile(std::integral_constant<int, 2>{});
      sub_tile(std::integral_constant<int, 3>{});
    };
    block(std::integral_constant<int, 0>{});
    if constexpr (L::KSB > 1) block(std::integral_constant<int, 1>{});
    if constexpr (L::KSB > 2) {
      block(std::integral_constant<int, 2>{});
      block(std::integral_constant<int, 3>{});
    }
  };

  while (it < c1) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      if (it < c1) {
        const int rt = it / p.k_slabs;
        const int ks = it - rt * p.k_slabs;
        if (rt != cur_rt) flush_until(rt);
        compute(buf[d], ks);
        const int nx = it + kDepth * kWarps;
        if (nx < c1) load_slab<BITS>(buf[d], p.tiled + (size_t)nx * L::kSlabBytes, lane);
        it += kWarps;
      }
    }
  }
  flush_until(rt_last + 1);
}

constexpr size_t kCounterBytes = 16384;  // 4096 row tiles = 262144 output rows

template <int BITS, int NB, bool FP16>
int launch(const LinearParams& p, int grid, unsigned flags, cudaStream_t stream) {
  using T = Table<BITS>;
  const size_t smem = (T::kAligned64K ? 65536 : 16) + T::kBytes + (size_t)kWarps * kSubTiles * NB * 128 * sizeof(float);
  auto kernel = linear_lut_kernel<BITS, NB, FP16>;
  static bool configured[64] = {};
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    FDK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & FDK_FLAG_PDL) ? 1 : 0;
  FDK_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return FDK_OK;
}

template <int BITS>
int launch_bits(const LinearParams& p, int grid, int dtype, unsigned flags, cudaStream_t stream) {
  const bool wide = p.m > 8;
  if (dtype == FDK_DTYPE_F16) {
    return wide ? launch<BITS, 2, true>(p, grid, flags, stream) : launch<BITS, 1, true>(p, grid, flags, stream);
  }
  return wide ? launch<BITS, 2, false>(p, grid, flags, stream) : launch<BITS, 1, false>(p, grid, flags, stream);
}

}  // namespace
}  // namespace fdk

using namespace fdk;

extern "C" int fdk_workspace_size(size_t* bytes_host) {
  FDK_CHECK_ARG(bytes_host != nullptr, FDK_ERR_BAD_ARG, "bytes_host is null");
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  *bytes_host = kCounterBytes + (size_t)di.sm_count * 2 * 1024 * sizeof(float);
  return FDK_OK;
}

extern "C" int fdk_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  FDK_CHECK_ARG(workspace != nullptr, FDK_ERR_WORKSPACE, "workspace is null");
  FDK_CHECK_ARG(workspace_bytes >= kCounterBytes, FDK_ERR_WORKSPACE, "workspace of %zu bytes is too small", workspace_bytes);
  FDK_CUDA(cudaMemsetAsync(workspace, 0, kCounterBytes, (cudaStream_t)stream));
  return FDK_OK;
}

extern "C" int fdk_linear_lut(const void* x, const void* tiled, const void* lut, void* out, int m, int n,
                              int k, int bits, int dtype, void* workspace, size_t workspace_bytes,
                              unsigned flags, void* stream) {
  FDK_CHECK_ARG(m > 0 && n > 0 && k > 0, FDK_ERR_BAD_ARG, "m=%d, n=%d, k=%d must be positive", m, n, k);
  FDK_CHECK_ARG(bits_supported(bits), FDK_ERR_SHAPE, "bits=%d not in {1,2,3,4,8}", bits);
  FDK_CHECK_ARG(k % kBlock == 0, FDK_ERR_SHAPE, "k=%d must be a multiple of 64", k);
  FDK_CHECK_ARG(x && tiled && lut && out, FDK_ERR_BAD_ARG, "null pointer");
  FDK_CHECK_ARG(dtype == FDK_DTYPE_BF16 || dtype == FDK_DTYPE_F16, FDK_ERR_BAD_ARG, "dtype=%d", dtype);
  FDK_CHECK_ARG((flags & ~FDK_FLAG_PDL) == 0, FDK_ERR_BAD_ARG, "unknown flags 0x%x", flags);
  FDK_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)tiled & 15) == 0 && ((uintptr_t)lut & 15) == 0 &&
                    ((uintptr_t)out & 1) == 0,
                FDK_ERR_ALIGN, "x, tiled and lut must be 16-byte aligned");
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  FDK_CHECK_ARG(di.cc_major == 10, FDK_ERR_ARCH, "device has compute capability %d.%d", di.cc_major, di.cc_minor);
  const TiledDims d = tiled_dims(n, k, bits);
  FDK_CHECK_ARG((size_t)d.row_tiles * sizeof(int) <= kCounterBytes, FDK_ERR_SHAPE, "n=%d exceeds %d rows", n,
                (int)(kCounterBytes / sizeof(int)) * kTileRows);
  const size_t need = kCounterBytes + (size_t)di.sm_count * 2 * 1024 * sizeof(float);
  FDK_CHECK_ARG(workspace != nullptr && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                FDK_ERR_WORKSPACE, "workspace must be a 16-byte aligned buffer of at least %zu bytes", need);

  LinearParams p{};
  p.tiled = (const uint8_t*)tiled;
  p.lut = lut;
  p.counters = (int*)workspace;
  p.partial = (float*)((uint8_t*)workspace + kCounterBytes);
  p.n = n;
  p.k = k;
  p.k_slabs = d.k_slabs;
  p.total = d.row_tiles * d.k_slabs;
  const int grid = p.total < di.sm_count ? p.total : di.sm_count;
  p.base = p.total / grid;
  p.rem = p.total % grid;
  for (int m0 = 0; m0 < m; m0 += 16) {
    p.m = (m - m0) < 16 ? (m - m0) : 16;
    p.x = (const uint16_t*)x + (size_t)m0 * k;
    p.out = (uint16_t*)out + (size_t)m0 * n;
    int st;
    switch (bits) {
      case 1: st = launch_bits<1>(p, grid, dtype, flags, (cudaStream_t)stream); break;
      case 2: st = launch_bits<2>(p, grid, dtype, flags, (cudaStream_t)stream); break;
      case 3: st = launch_bits<3>(p, grid, dtype, flags, (cudaStream_t)stream); break;
      case 4: st = launch_bits<4>(p, grid, dtype, flags, (cudaStream_t)stream); break;
      default: st = launch_bits<8>(p, grid, dtype, flags, (cudaStream_t)stream); break;
    }
    if (st) return st;
  }
  return FDK_OK;
}
