// Fused dequantise + GEMM for batches of 17 and more rows, on the fifth-generation tensor
// cores:  out[m, n] = x[m, k] . W[n, k]^T  with W = bf16(table value * block scale), the
// reference's dense W (src/fdk/kernels.py:23-24) bit for bit (fp16(...) for fp16 inputs), built tile by tile in shared
// memory and never written to HBM.
//
// One CTA per 128 weight rows (the MMA M dimension; the batch is the MMA N dimension, so a
// weight tile is dequantised once for the whole batch).  Six warps, specialised:
//   warp 0      copy producer: per 64-column block, the [batch, 64] slice of x by a tiled TMA
//               load (128-byte swizzle) into a ring of stages, and the two code slabs of the
//               tile by cp.async.bulk -- with the stage where a slab holds one block (4 and 8
//               bits), into a two-slot ring of their own where it holds two or four (1, 2,
//               3 bits); completion on mbarriers;
//   warps 2..9  dequantise: code bytes -> replicated table lookup -> multiply by the
//               block scale in bf16 -> the 128 x 64 bf16 A tile of the stage, written in the
//               K-major 128-byte-swizzled layout the MMA reads; afterwards the epilogue;
//   warp 1      one thread issues tcgen05.mma (M = 128, N = batch padded to 16, K = 16, four
//               per block) accumulating in tensor memory, and tcgen05.commit hands the stage
//               back to the producer; it also owns the tensor-memory allocation.
// Epilogue: tcgen05.ld brings the fp32 accumulators to registers (one tile row per thread),
// converted to bf16 and stored transposed into out[batch, n].
// Every barrier wait is bounded; a wait that runs out sets a status bit, and the kernel still
// frees its tensor memory and returns.
#include <cuda.h>

#include <cstring>

#include "fdk_common.cuh"
#include "lut_table.cuh"

namespace fdk {
namespace {

constexpr int kTcDequantWarps = 8;
constexpr int kTcThreads = 64 + 32 * kTcDequantWarps;
constexpr int kTcMaxSplits = 8;
constexpr int kTcTileRows = 128;
constexpr int kTcMaxStages = 4;
constexpr int kTcStatusTimeout = 1;
constexpr int kTcStatusSmemLayout = 2;

struct TcParams {
  const uint8_t* tiled;
  const void* lut;   // device byte table, or null when it travels in the parameters
  uint16_t* out;
  int* status;       // device-side error bits
  int m, m_pad, n, k;
  int row_tiles;     // 64-row tiles of the tiled buffer
  int k_blocks;      // k / 64
  int stages;
  int splits;        // CTAs sharing one 128-row tile, each with a contiguous range of 64-column blocks
  float* partial;    // [tile][split - 1][m_pad][128] fp32 sums of the non-owning CTAs
  int* flags;        // [tile][kTcMaxSplits] tag of the last published partial
  int* uses;         // [tile] how often the tile has been finished through this workspace
  uint32_t tmem_cols;
  uint32_t smem_base, table_addr, bar_addr, tmem_slot_addr;
  uint32_t a_addr[kTcMaxStages], b_addr[kTcMaxStages], c_addr[kTcMaxStages];
  int k_slabs;            // slabs per 64-row tile
  uint32_t cc_addr[2];    // code slots of the formats whose slabs span several blocks
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);        // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // descriptor version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t ring32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

template <bool FP16>
__device__ __forceinline__ uint32_t mul_pair(uint32_t a, uint32_t b) {  // two 16-bit products, rounded to nearest
  uint32_t d;
  if constexpr (FP16) asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// The 16 elements (eight bf16 pairs) of one row's share of a 64-block, in element order.
// w: the row's code words -- 4 bits: two words; 8 bits: four; 2 bits: one; 1 bit: the two
// bytes starting at byte 2 * HH of w[0]; 3 bits: the 48-bit field group starting at bit 48 * HH
// of the 96 bits w[0..2].
template <int BITS, int HH>
__device__ __forceinline__ void decode_row16(const uint32_t (&w)[4], uint32_t lane_base, uint32_t (&v)[8]) {
  if constexpr (BITS == 4) {
    v[0] = lut32(entry_addr<4, 0>(w[0], lane_base)); v[1] = lut32(entry_addr<4, 1>(w[0], lane_base));
    v[2] = lut32(entry_addr<4, 2>(w[0], lane_base)); v[3] = lut32(entry_addr<4, 3>(w[0], lane_base));
    v[4] = lut32(entry_addr<4, 0>(w[1], lane_base)); v[5] = lut32(entry_addr<4, 1>(w[1], lane_base));
    v[6] = lut32(entry_addr<4, 2>(w[1], lane_base)); v[7] = lut32(entry_addr<4, 3>(w[1], lane_base));
  } else if constexpr (BITS == 8) {  // sixteen single lookups, merged in pairs
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = prmt<0x7610>(lut32(entry_addr<8, 0>(w[i], lane_base)), lut32(entry_addr<8, 1>(w[i], lane_base)));
      v[2 * i + 1] = prmt<0x7610>(lut32(entry_addr<8, 2>(w[i], lane_base)), lut32(entry_addr<8, 3>(w[i], lane_base)));
    }
  } else if constexpr (BITS == 2) {  // one byte = four elements = one 8-byte entry
    uint2 q;
    q = lut64(entry_addr<2, 0>(w[0], lane_base)); v[0] = q.x; v[1] = q.y;
    q = lut64(entry_addr<2, 1>(w[0], lane_base)); v[2] = q.x; v[3] = q.y;
    q = lut64(entry_addr<2, 2>(w[0], lane_base)); v[4] = q.x; v[5] = q.y;
    q = lut64(entry_addr<2, 3>(w[0], lane_base)); v[6] = q.x; v[7] = q.y;
  } else if constexpr (BITS == 1) {  // one byte = eight elements = one 16-byte entry
    uint4 q;
    q = lut128(entry_addr<1, 2 * HH>(w[0], lane_base)); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    q = lut128(entry_addr<1, 2 * HH + 1>(w[0], lane_base)); v[4] = q.x; v[5] = q.y; v[6] = q.z; v[7] = q.w;
  } else {  // 3 bits: eight 6-bit pair fields, field f at bits [6f, 6f + 6) of the 96-bit group
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      constexpr int kStrideLog2 = 7;  // Table<3>::kStride
      const int o = 6 * (8 * HH + i), wi = o >> 5, sh = o & 31;
      uint32_t f;  // the field moved to bits 7..12: field * 128
      if (sh + 6 <= 32) {
        f = (sh >= kStrideLog2) ? (w[wi] >> (sh - kStrideLog2)) : (w[wi] << (kStrideLog2 - sh));
      } else {
        f = __funnelshift_r(w[wi], w[wi + 1], sh - kStrideLog2);
      }
      v[i] = lut32(lane_base + (f & (63u << kStrideLog2)));
    }
  }
}

template <int BITS, bool FP16>
__global__ void __launch_bounds__(kTcThreads, 2)
    gemm_lut_tc_kernel(const __grid_constant__ TcParams p, const __grid_constant__ InlineLut<BITS> inl,
                       const __grid_constant__ CUtensorMap x_map) {
  using L = Layout<BITS>;
  using T = Table<BITS>;
  static_assert(T::kStride == 128, "3-bit field extraction assumes 128-byte table rows");
  constexpr bool kOwnCodeRing = L::KSB > 1;  // slabs spanning several blocks live in a ring of their own
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_addr(smem_raw);
  if (raw != p.smem_base) {
    if (threadIdx.x == 0) atomicOr(p.status, kTcStatusSmemLayout);
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int S = p.stages;
  // barriers: tma_full[S], a_full[S], empty[S], accum_full
  const uint32_t tma_full = p.bar_addr, a_full = p.bar_addr + 8 * S, empty = p.bar_addr + 16 * S,
                 accum_full = p.bar_addr + 24 * S;
  const uint32_t c_full = p.bar_addr + 8 * (3 * kTcMaxStages + 2), c_empty = c_full + 16;  // two slots each
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (p.tmem_slot_addr - raw));
  const int tile = blockIdx.x / p.splits;         // 128 rows = 64-row tiles 2*tile, 2*tile + 1
  const int sp = blockIdx.x - tile * p.splits;    // this CTA's share of the 64-column blocks
  const int kb_begin = (int)((long long)p.k_blocks * sp / p.splits);
  const int kb_end = (int)((long long)p.k_blocks * (sp + 1) / p.splits);
  const int n_kb = kb_end - kb_begin;
  const bool second_half = (2 * tile + 1) < p.row_tiles;
  bool timed_out = false;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(tma_full + 8 * s, 1);
      mbar_init(a_full + 8 * s, kTcDequantWarps);  // one arrival per dequantising warp
      mbar_init(empty + 8 * s, 1);
    }
    mbar_init(accum_full, 1);
    for (int c = 0; c < 2; ++c) {
      mbar_init(c_full + 8 * c, 1);
      mbar_init(c_empty + 8 * c, kTcDequantWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory for the accumulator: 128 lanes x tmem_cols columns of fp32
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(p.tmem_slot_addr),
                 "r"(p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp >= 2) {
    if (p.lut == nullptr) {
      fill_table<BITS>(p.table_addr, 32 * kTcDequantWarps, [&](int i) { return inl.w[i]; }, threadIdx.x - 64);
    } else {
      fill_table<BITS>(p.table_addr, 32 * kTcDequantWarps,
                       [&](int i) { return __ldg(reinterpret_cast<const uint32_t*>(p.lut) + i); }, threadIdx.x - 64);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- copy producer ----------------
    if (lane == 0) {
      const uint32_t code_bytes = L::kSlabBytes * (second_half ? 2 : 1);
      const uint32_t x_bytes = (uint32_t)p.m_pad * 128;
      auto load_codes = [&](int slab, uint32_t dst, uint32_t bar) {
        const uint8_t* slab0 = p.tiled + ((size_t)(2 * tile) * p.k_slabs + slab) * L::kSlabBytes;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                     "l"(slab0), "r"((uint32_t)L::kSlabBytes), "r"(bar)
                     : "memory");
        if (second_half) {
          const uint8_t* slab1 = p.tiled + ((size_t)(2 * tile + 1) * p.k_slabs + slab) * L::kSlabBytes;
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           dst + (uint32_t)L::kSlabBytes),
                       "l"(slab1), "r"((uint32_t)L::kSlabBytes), "r"(bar)
                       : "memory");
        }
      };
      int loaded_slab = -1, slabs_loaded = 0;
      for (int i = 0; i < n_kb; ++i) {
        const int kb = kb_begin + i;
        const int s = i % S;
        const uint32_t phase = (i / S) & 1;
        if constexpr (kOwnCodeRing) {
          const int slab = kb / L::KSB;
          if (slab != loaded_slab) {  // next slab into the slot freed two slabs ago
            const int c = slabs_loaded & 1;
            if (!mbar_wait(c_empty + 8 * c, ((slabs_loaded >> 1) & 1) ^ 1)) { timed_out = true; break; }
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(c_full + 8 * c), "r"(code_bytes) : "memory");
            load_codes(slab, p.cc_addr[c], c_full + 8 * c);
            loaded_slab = slab;
            ++slabs_loaded;
          }
        }
        if (!mbar_wait(empty + 8 * s, phase ^ 1)) { timed_out = true; break; }
        const uint32_t bar = tma_full + 8 * s;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                     "r"((kOwnCodeRing ? 0u : code_bytes) + x_bytes)
                     : "memory");
        if constexpr (!kOwnCodeRing) load_codes(kb, p.c_addr[s], bar);
        tma_load_2d(p.b_addr[s], &x_map, kb * 64, 0, bar);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, A and B both bf16 (format 1) or both fp16
      // (format 0), both K-major, N = m_pad, M = 128
      constexpr uint32_t kFormat = FP16 ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (kFormat << 7) | (kFormat << 10) | ((uint32_t)(p.m_pad >> 3) << 17) | ((128u >> 4) << 24);
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % S;
        const uint32_t phase = (i / S) & 1;
        if (!mbar_wait(tma_full + 8 * s, phase)) { timed_out = true; break; }
        if (!mbar_wait(a_full + 8 * s, phase)) { timed_out = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // one descriptor pair per stage; the four K = 16 slices of the 64-column block lie 32
        // bytes apart, i.e. 2 in the descriptors' 16-byte address units
        const uint64_t a_desc = umma_desc(p.a_addr[s]), b_desc = umma_desc(p.b_addr[s]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          umma_bf16(tmem_base, a_desc + 2 * j, b_desc + 2 * j, idesc, (i > 0 || j > 0) ? 1u : 0u);
        }
        umma_commit(empty + 8 * s);  // the stage may be refilled once these MMAs have read it
      }
      umma_commit(accum_full);
    }
  } else {
    // ---------------- dequantise, then epilogue ----------------
    const int dw = warp - 2;          // 0..7: one of the eight 16-row sub-tiles each
    const int g = lane >> 2, t = lane & 3;
    const uint32_t lane_base = p.table_addr + T::lane_offset(lane);
    int cur_slab = -1, slabs_seen = 0;
    uint32_t code_slot = 0;
    for (int i = 0; i < n_kb; ++i) {
      const int s = i % S;
      const uint32_t phase = (i / S) & 1;
      const int kb = kb_begin + i;
      const int jb = kOwnCodeRing ? kb % L::KSB : 0;  // block inside its slab
      if constexpr (kOwnCodeRing) {
        const int slab_index = kb / L::KSB;
        if (slab_index != cur_slab) {
          const int c = slabs_seen & 1;
          if (!mbar_wait(c_full + 8 * c, (slabs_seen >> 1) & 1)) { timed_out = true; break; }
          code_slot = p.cc_addr[c];
          cur_slab = slab_index;
          ++slabs_seen;
        }
      }
      if (!mbar_wait(tma_full + 8 * s, phase)) { timed_out = true; break; }  // also: the stage's A tile is free
      {
        const int u = dw, half = u >> 2, r = u & 3;
        if (!(half == 1 && !second_half)) {
        const uint32_t slab = (kOwnCodeRing ? code_slot : p.c_addr[s]) + half * L::kSlabBytes;
        const uint32_t scw = ring32(slab + L::kCodeBytes + jb * 128 + g * 16 + r * 4);
        const uint32_t s_lo = prmt<0x1010>(scw, 0u), s_hi = prmt<0x3232>(scw, 0u);  // scale of row g / g+8 in both halves
        uint32_t wg[4] = {0u, 0u, 0u, 0u}, wh[4] = {0u, 0u, 0u, 0u};  // code words of row g and of row g+8
        if constexpr (BITS == 4) {
          const uint4 c = ring128(slab + (r * 32 + lane) * 16);
          wg[0] = c.x; wg[1] = c.y; wh[0] = c.z; wh[1] = c.w;
        } else if constexpr (BITS == 8) {
          const uint4 cg = ring128(slab + ((r * 2) * 32 + lane) * 16), ch = ring128(slab + ((r * 2 + 1) * 32 + lane) * 16);
          wg[0] = cg.x; wg[1] = cg.y; wg[2] = cg.z; wg[3] = cg.w;
          wh[0] = ch.x; wh[1] = ch.y; wh[2] = ch.z; wh[3] = ch.w;
        } else if constexpr (BITS == 2) {  // the lane's 16 bytes: per block one word for row g, one for row g+8
          const uint32_t at = slab + (r * 32 + lane) * 16 + jb * 8;
          wg[0] = ring32(at);
          wh[0] = ring32(at + 4);
        } else if constexpr (BITS == 1) {  // per block one word: bytes 0,1 row g, bytes 2,3 row g+8
          wg[0] = wh[0] = ring32(slab + (r * 32 + lane) * 16 + jb * 4);
        } else {  // 3 bits: 48 bytes per lane in three 16-byte vectors, 12 bytes per block
#pragma unroll
          for (int i3 = 0; i3 < 3; ++i3) {
            const int wi = 3 * jb + i3;
            wg[i3] = wh[i3] = ring32(slab + ((r * 3 + (wi >> 2)) * 32 + lane) * 16 + (wi & 3) * 4);
          }
        }
        auto write_row = [&](auto hhc) {
          constexpr int HH = decltype(hhc)::value;
          uint32_t v[8];
          decode_row16<BITS, HH>(HH == 0 ? wg : wh, lane_base, v);
          const uint32_t sc = HH == 0 ? s_lo : s_hi;
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = mul_pair<FP16>(v[i], sc);
          const int row = 16 * u + g + 8 * HH;  // row % 8 == g
          const uint32_t row_addr = p.a_addr[s] + row * 128;
          const uint32_t c0 = ((2 * t) ^ g) * 16, c1 = ((2 * t + 1) ^ g) * 16;
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row_addr + c0), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row_addr + c1), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
        };
        write_row(std::integral_constant<int, 0>{});
        write_row(std::integral_constant<int, 1>{});
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a_full + 8 * s) : "memory");
        if constexpr (kOwnCodeRing) {  // last block read from this code slot: hand it back
          if (jb == L::KSB - 1 || i == n_kb - 1) {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(c_empty + 8 * ((slabs_seen - 1) & 1)) : "memory");
          }
        }
      }
    }
    // epilogue (first four of these warps): each reads the 32 accumulator rows of its
    // tensor-memory lane quarter.  A CTA that does not own the tile parks its fp32 sums in the
    // workspace; the owner (share 0) adds the parked sums in share order and writes bf16.
    if (dw < 4) {
      if (!mbar_wait(accum_full, 0)) timed_out = true;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int quarter = warp & 3;
      const int row_in_tile = quarter * 32 + lane;
      const int row = tile * kTcTileRows + row_in_tile;
      int tag = 0;
      if (p.splits > 1) tag = ld_relaxed_s32(p.uses + tile) + 1;
      if (sp == 0 && p.splits > 1) {  // wait until every other share has been published
        for (int o = 1; o < p.splits; ++o) {
          unsigned long long t0 = 0;
          for (uint32_t spin = 0;; ++spin) {
            int f;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(p.flags + tile * kTcMaxSplits + o) : "memory");
            if (f == tag) break;
            if ((spin & 255u) == 255u) {
              unsigned long long now;
              asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
              if (t0 == 0) t0 = now;
              else if (now - t0 > 2000000000ull) { timed_out = true; break; }
            }
          }
        }
      }
      for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
        uint32_t acc[16];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]), "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7]),
              "=r"(acc[8]), "=r"(acc[9]), "=r"(acc[10]), "=r"(acc[11]), "=r"(acc[12]), "=r"(acc[13]), "=r"(acc[14]), "=r"(acc[15])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (sp != 0) {
          float* mine = p.partial + ((size_t)(tile * (p.splits - 1) + sp - 1) * p.m_pad + c0) * 128 + row_in_tile;
#pragma unroll
          for (int j = 0; j < 16; ++j) __stcg(mine + j * 128, __uint_as_float(acc[j]));
        } else {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(acc[j]);
          for (int o = 1; o < p.splits; ++o) {  // share order; the sixteen loads of a share are independent
            const float* theirs = p.partial + ((size_t)(tile * (p.splits - 1) + o - 1) * p.m_pad + c0) * 128 + row_in_tile;
            float t[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) t[j] = __ldcg(theirs + j * 128);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += t[j];
          }
          if (row < p.n) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int b = c0 + j;
              if (b < p.m) p.out[(size_t)b * p.n + row] = from_float<FP16>(v[j]);
            }
          }
        }
      }
      if (p.splits > 1) {
        __threadfence();
        // the four epilogue warps meet on a named barrier, then one thread publishes
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (dw == 0 && lane == 0) {
          if (sp != 0) {
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.flags + tile * kTcMaxSplits + sp), "r"(tag) : "memory");
          } else {
            p.uses[tile] = tag;  // the next use of this tile waits for tags one higher
          }
        }
      }
    }
  }
  if (timed_out && lane == 0) atomicOr(p.status, kTcStatusTimeout);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
  }
}

// ---- host side ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_fn(EncodeTiledFn* out) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    FDK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
    FDK_CHECK_ARG(qres == cudaDriverEntryPointSuccess && sym != nullptr, FDK_ERR_CUDA, "cuTensorMapEncodeTiled not found");
    fn = (EncodeTiledFn)sym;
  }
  *out = fn;
  return FDK_OK;
}

inline uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }
inline bool two_per_sm(int m_pad) { return m_pad <= 64; }

// Shared memory: barriers, the table, then the stage buffers (1024-byte aligned for the
// swizzled tiles).  Returns the dynamic size, or 0 if `stages` do not fit in `limit`.
template <int BITS>
size_t plan_tc_smem(uint32_t base, uint32_t limit, int stages, TcParams& p) {
  using L = Layout<BITS>;
  using T = Table<BITS>;
  uint32_t cursor = round_up(base, 128);
  p.smem_base = base;
  p.bar_addr = cursor;
  p.tmem_slot_addr = cursor + 8 * (3 * kTcMaxStages + 1);  // then the four code-ring barriers
  cursor += 256;
  p.table_addr = cursor;
  cursor += T::kBytes;
  p.stages = stages;
  const uint32_t b_bytes = (uint32_t)p.m_pad * 128;
  cursor = round_up(cursor, 1024);
  for (int s = 0; s < stages; ++s) { p.b_addr[s] = cursor; cursor += b_bytes; }
  for (int s = 0; s < stages; ++s) { p.a_addr[s] = cursor; cursor += 16384; }
  if (L::KSB == 1) {
    for (int s = 0; s < stages; ++s) { p.c_addr[s] = cursor; cursor += round_up(2 * L::kSlabBytes, 128); }
  } else {
    for (int c = 0; c < 2; ++c) { p.cc_addr[c] = cursor; cursor += round_up(2 * L::kSlabBytes, 128); }
  }
  return (cursor - base <= limit) ? cursor - base : 0;
}

template <int BITS, bool FP16>
int launch_tc(TcParams p, const void* lut_host, const CUtensorMap& map, int tiles, cudaStream_t stream) {
  InlineLut<BITS> inl;
  if (lut_host != nullptr) {
    memcpy(inl.w, lut_host, sizeof(inl.w));
    p.lut = nullptr;
  } else {
    memset(inl.w, 0, sizeof(inl.w));
  }
  uint32_t base = 0;
  if (int st = dynamic_smem_base(&base)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  size_t smem = 0;
  // small batches: two CTAs per SM (twice the warps to hide the latencies of the per-block
  // hand-offs), each within half the shared memory; tensor memory holds both accumulators
  const uint32_t limit = two_per_sm(p.m_pad) ? ((uint32_t)di.max_smem_optin + 1024) / 2 - 1024 : (uint32_t)di.max_smem_optin;
  for (int s = kTcMaxStages; s >= 1 && smem == 0; --s) smem = plan_tc_smem<BITS>(base, limit, s, p);
  FDK_CHECK_ARG(smem != 0, FDK_ERR_CUDA, "no shared-memory plan fits %d bytes", di.max_smem_optin);
  auto kernel = gemm_lut_tc_kernel<BITS, FP16>;
  static size_t configured[64] = {};
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  if (configured[dev & 63] < smem) {
    FDK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev & 63] = smem;
  }
  kernel<<<tiles, kTcThreads, smem, stream>>>(p, inl, map);
  FDK_CUDA(cudaGetLastError());
  return FDK_OK;
}

}  // namespace

// Batches above 16 rows.  Called by fdk_linear_lut.
int gemm_lut_tc(const void* x, const void* tiled, const void* lut, const void* lut_host, void* out, int m, int n,
                int k, int bits, bool fp16, void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream) {
  EncodeTiledFn encode = nullptr;
  if (int st = encode_fn(&encode)) return st;
  const TiledDims d = tiled_dims(n, k, bits);
  const int tiles = (n + kTcTileRows - 1) / kTcTileRows;
  const int k_blocks = k / kBlock;
  // few tiles: several CTAs share a tile, each with its own range of 64-column blocks, so that
  // the whole GPU is busy; all of them must be resident at once (the owner waits for the others)
  const int m_pad_max = ((m < 256 ? m : 256) + 15) / 16 * 16;
  const int resident = sm_count * (two_per_sm(m_pad_max) ? 2 : 1);
  int splits = 1;
  if (tiles * 2 <= resident) {
    splits = resident / tiles;
    if (splits > kTcMaxSplits) splits = kTcMaxSplits;
    if (splits > k_blocks / 4) splits = k_blocks / 4;
    if (splits < 1) splits = 1;
  }
  // the parked partial tiles (128 rows x m_pad columns of fp32 each) must fit the workspace
  const size_t partial_room = workspace_bytes > kTcPartialOffset ? workspace_bytes - kTcPartialOffset : 0;
  while (splits > 1 && ((size_t)tiles * (splits - 1) * 128 * m_pad_max * sizeof(float) > partial_room || tiles > 2048)) --splits;
  for (int m0 = 0; m0 < m; m0 += 256) {
    const int mc = (m - m0) < 256 ? (m - m0) : 256;
    TcParams p{};
    p.tiled = (const uint8_t*)tiled;
    p.lut = lut;
    p.out = (uint16_t*)out + (size_t)m0 * n;
    p.status = (int*)workspace + kStatusWord;
    p.m = mc;
    p.m_pad = (mc + 15) / 16 * 16;
    p.n = n;
    p.k = k;
    p.row_tiles = d.row_tiles;
    p.k_blocks = k_blocks;
    p.k_slabs = d.k_slabs;
    p.splits = splits;
    p.flags = (int*)((uint8_t*)workspace + kTcFlagsOffset);
    p.uses = (int*)((uint8_t*)workspace + kTcUsesOffset);
    p.partial = (float*)((uint8_t*)workspace + kTcPartialOffset);
    uint32_t cols = 32;
    while ((int)cols < p.m_pad) cols *= 2;
    p.tmem_cols = cols;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)mc};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)p.m_pad};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = encode(&map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)((const uint16_t*)x + (size_t)m0 * k), dims,
                        strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FDK_CHECK_ARG(r == CUDA_SUCCESS, FDK_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    int st;
    switch (bits) {
      case 1: st = fp16 ? launch_tc<1, true>(p, lut_host, map, tiles * splits, stream) : launch_tc<1, false>(p, lut_host, map, tiles * splits, stream); break;
      case 2: st = fp16 ? launch_tc<2, true>(p, lut_host, map, tiles * splits, stream) : launch_tc<2, false>(p, lut_host, map, tiles * splits, stream); break;
      case 3: st = fp16 ? launch_tc<3, true>(p, lut_host, map, tiles * splits, stream) : launch_tc<3, false>(p, lut_host, map, tiles * splits, stream); break;
      case 4: st = fp16 ? launch_tc<4, true>(p, lut_host, map, tiles * splits, stream) : launch_tc<4, false>(p, lut_host, map, tiles * splits, stream); break;
      default: st = fp16 ? launch_tc<8, true>(p, lut_host, map, tiles * splits, stream) : launch_tc<8, false>(p, lut_host, map, tiles * splits, stream); break;
    }
    if (st) return st;
  }
  return FDK_OK;
}

}  // namespace fdk
