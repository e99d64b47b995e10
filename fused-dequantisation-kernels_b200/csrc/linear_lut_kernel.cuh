// Fused dequantise + GEMV / skinny GEMM for sm_100a:  out[m, n] = x[m, k] . W[n, k]^T,
// W given as tiled low-bit codes + block scales + a lookup table (fdk_layout.cuh).
//
// Shape of the kernel (persistent CTAs of 12, 8 or 4 warps, sized so that two fit on an SM):
//   * The weight stream is cut into slabs (64 rows x 64*KSB columns, 2-6 KB).  The
//     slabs of the whole matrix form one linear sequence (row tile major); CTA c owns
//     a contiguous range of it ("stream-K"), its warps take slabs round-robin.  Every
//     SM therefore streams the same number of bytes (+-1 slab) whatever N and K are.
//     A large matrix runs two CTAs per SM; a small one runs one, and the other half of
//     the SM is free for the next kernel on the stream, which under programmatic
//     dependent launch fills its table and prefetches weights while this one runs.
//   * Every warp owns a small ring of slab-sized stages in shared memory.  Lane 0
//     fills them with one bulk asynchronous copy per slab (cp.async.bulk, completion
//     on an mbarrier), so the data in flight costs no registers and the loads need
//     no issue slots.  x is staged whole once per CTA when it is small, otherwise
//     its rows travel with each slab.  All waits on the barriers are bounded.
//   * Codes are turned into tensor-core A fragments by table lookup in shared memory:
//     one code byte indexes a replicated byte table (lut_table.cuh), so a lookup is one
//     PRMT (extract the byte), one multiply-add (address) and one conflict-free LDS
//     that returns 2 (4-bit), 4 (2-bit) or 8 (1-bit) 16-bit weights already in
//     fragment order.  The table itself arrives inside the kernel parameters.
//   * mma.sync m16n8k16 accumulates one 64-block in fp32; the block scale multiplies
//     the fp32 block sum (4 FMAs per 1024 weights), then running totals per row.
//     The tensor pipe is used because the FMA work would otherwise compete with the
//     lookups for issue slots; at m <= 16 it is far from being the limiter, so the
//     synchronous MMA form is enough and keeps the weights in registers (a tcgen05
//     MMA would need them written back to shared or tensor memory first).  What
//     bounds the main loop is the shared-memory pipe: one 128-byte wavefront per 32
//     code bytes looked up, plus the wavefronts that bring codes and x in.
//   * At a row-tile boundary the warps of a CTA deposit their totals in shared memory
//     and the last to arrive adds them in warp order (no CTA barrier).  A row tile
//     split over several CTAs is finished by the CTA holding its first slabs: the
//     others publish their sums to the workspace as {value, tag} words, which the
//     finisher reads (bounded polling) and adds in CTA order.  The summation order
//     never depends on timing, so results are reproducible bit for bit.
//   * Epilogue variants: plain store; silu(gate) * up for a gate|up weight stored in
//     32 + 32 row groups; or, in tensor-parallel decode, tagged stores of the partial
//     sums into every rank's exchange buffer.#pragma once
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "linear_lut_params.cuh"
#include "tp_exchange.cuh"

namespace fdk {
namespace {


// A fragments of one sub-tile for the four MMA k-steps of 64-block JB, from the lane's
// code vectors `code[0..V)` of that sub-tile.
//   a[s][0] = row g,   elements 4s, 4s+1      a[s][1] = row g+8, elements 4s, 4s+1
//   a[s][2] = row g,   elements 4s+2, 4s+3    a[s][3] = row g+8, elements 4s+2, 4s+3
// (elements counted inside the lane's 16-element share of the block; x is read
// with the same numbering, so the product does not depend on it).
template <int BITS, int JB>
__device__ __forceinline__ void build_fragments(const uint4 (&code)[Layout<BITS>::V], uint32_t lane_base,
                                                uint32_t (&a)[4][4]) {
  if constexpr (BITS == 4) {
    const uint4& c = code[0];
    a[0][0] = lut32(entry_addr<4, 0>(c.x, lane_base)); a[0][2] = lut32(entry_addr<4, 1>(c.x, lane_base));
    a[1][0] = lut32(entry_addr<4, 2>(c.x, lane_base)); a[1][2] = lut32(entry_addr<4, 3>(c.x, lane_base));
    a[2][0] = lut32(entry_addr<4, 0>(c.y, lane_base)); a[2][2] = lut32(entry_addr<4, 1>(c.y, lane_base));
    a[3][0] = lut32(entry_addr<4, 2>(c.y, lane_base)); a[3][2] = lut32(entry_addr<4, 3>(c.y, lane_base));
    a[0][1] = lut32(entry_addr<4, 0>(c.z, lane_base)); a[0][3] = lut32(entry_addr<4, 1>(c.z, lane_base));
    a[1][1] = lut32(entry_addr<4, 2>(c.z, lane_base)); a[1][3] = lut32(entry_addr<4, 3>(c.z, lane_base));
    a[2][1] = lut32(entry_addr<4, 0>(c.w, lane_base)); a[2][3] = lut32(entry_addr<4, 1>(c.w, lane_base));
    a[3][1] = lut32(entry_addr<4, 2>(c.w, lane_base)); a[3][3] = lut32(entry_addr<4, 3>(c.w, lane_base));
  } else if constexpr (BITS == 2) {
    const uint4& c = code[0];
    const uint32_t wg = word_of<2 * JB>(c), wh = word_of<2 * JB + 1>(c);
    uint2 q;
    q = lut64(entry_addr<2, 0>(wg, lane_base)); a[0][0] = q.x; a[0][2] = q.y;
    q = lut64(entry_addr<2, 1>(wg, lane_base)); a[1][0] = q.x; a[1][2] = q.y;
    q = lut64(entry_addr<2, 2>(wg, lane_base)); a[2][0] = q.x; a[2][2] = q.y;
    q = lut64(entry_addr<2, 3>(wg, lane_base)); a[3][0] = q.x; a[3][2] = q.y;
    q = lut64(entry_addr<2, 0>(wh, lane_base)); a[0][1] = q.x; a[0][3] = q.y;
    q = lut64(entry_addr<2, 1>(wh, lane_base)); a[1][1] = q.x; a[1][3] = q.y;
    q = lut64(entry_addr<2, 2>(wh, lane_base)); a[2][1] = q.x; a[2][3] = q.y;
    q = lut64(entry_addr<2, 3>(wh, lane_base)); a[3][1] = q.x; a[3][3] = q.y;
  } else if constexpr (BITS == 1) {
    const uint32_t w = word_of<JB>(code[0]);  // bytes 0,1: row g; bytes 2,3: row g+8
    uint4 q;
    q = lut128(entry_addr<1, 0>(w, lane_base)); a[0][0] = q.x; a[0][2] = q.y; a[1][0] = q.z; a[1][2] = q.w;
    q = lut128(entry_addr<1, 1>(w, lane_base)); a[2][0] = q.x; a[2][2] = q.y; a[3][0] = q.z; a[3][2] = q.w;
    q = lut128(entry_addr<1, 2>(w, lane_base)); a[0][1] = q.x; a[0][3] = q.y; a[1][1] = q.z; a[1][3] = q.w;
    q = lut128(entry_addr<1, 3>(w, lane_base)); a[2][1] = q.x; a[2][3] = q.y; a[3][1] = q.z; a[3][3] = q.w;
  } else if constexpr (BITS == 8) {
    const uint4& cg = code[0];  // row g: 16 bytes = 16 elements
    const uint4& ch = code[1];  // row g+8
#pragma unroll
    for (int st = 0; st < 4; ++st) {
      const uint32_t wg = word_at(cg, st), wh = word_at(ch, st);
      a[st][0] = prmt<0x7610>(lut32(entry_addr<8, 0>(wg, lane_base)), lut32(entry_addr<8, 1>(wg, lane_base)));
      a[st][2] = prmt<0x7610>(lut32(entry_addr<8, 2>(wg, lane_base)), lut32(entry_addr<8, 3>(wg, lane_base)));
      a[st][1] = prmt<0x7610>(lut32(entry_addr<8, 0>(wh, lane_base)), lut32(entry_addr<8, 1>(wh, lane_base)));
      a[st][3] = prmt<0x7610>(lut32(entry_addr<8, 2>(wh, lane_base)), lut32(entry_addr<8, 3>(wh, lane_base)));
    }
  } else {  // 3 bits: 96-bit little-endian group per block, pair field f at bits [6f, 6f+6)
    uint32_t w[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int wi = 3 * JB + i;
      w[i] = word_at(code[wi / 4], wi % 4);
    }
#pragma unroll
    for (int f = 0; f < 16; ++f) {
      const int o = 6 * f;  // bit offset of the field
      const int wi = o >> 5, sh = o & 31;
      uint32_t v;  // field moved to bits 7..12: field * 128, the table stride
      if (sh + 6 <= 32) {
        v = (sh >= 7) ? (w[wi] >> (sh - 7)) : (w[wi] << (7 - sh));
      } else {
        v = __funnelshift_r(w[wi], w[wi + 1], sh - 7);
      }
      const int p = f & 7, half = f >> 3;
      a[p >> 1][(p & 1) * 2 + half] = lut32((v & 0x1F80u) + lane_base);
    }
  }
}


// ---- row-tile epilogue ----------------------------------------------------------
// No CTA-wide barrier anywhere: a warp that has finished its slabs of a row tile deposits its
// totals in shared memory and moves on; the LAST warp of the CTA to do so adds the deposits
// up in warp order and finishes the tile (tile_finish).
//
// A row tile whose K range is split over several CTAs is finished by its OWNER, the CTA that
// holds the tile's first slabs (for that CTA the tile is the last thing it works on).  The
// other CTAs hold later slabs of the tile at the START of their ranges, so they are done with
// it early: each stores its partial sums as {value, tag} 8-byte words into its own area of
// the workspace and never waits.  The owner polls those words (bounded) until they carry this
// use's tag, adds them to its own sums in CTA order, writes the outputs and bumps the tile's
// use count.  tag = (use count + 1) * 4096 + row tile: a word left by an earlier launch or
// another tile can never match.  No fences, no atomics, one memory round trip at the end;
// and every sum has a fixed order, so results do not depend on timing.
//
// Reduction slots keep, per warp, sub-tile and n-tile, the float4 accumulator fragments of
// the lanes that hold live batch columns only: lanes with t < TT, TT = ceil(min(m, 8) / 2),
// stored densely as [t][g][4].  SW = 32 * TT floats per (warp, sub-tile, n-tile).
// There are two sets of slots; consecutive row tiles of a CTA alternate between them.
struct EpilogueSync {
  int count[2];  // deposits so far in each slot set
  int gen[2];    // reductions completed on each slot set
};

constexpr uint32_t kSpinLimit = 1u << 24;  // polls of a memory word before giving up

// Run by one warp.  `slots` is the slot set of this row tile: per warp one block of
// E = NB * 4 * SW floats laid out [sub-tile][n-tile][t][g][4].  Plain loops on purpose (this
// runs once or twice per CTA, so its cost is mostly instruction fetches).  Returns false if a
// bounded poll ran out.
// EPI: what is done with a finished row tile -- kEpiStore: written to `out`; kEpiSilu:
// silu(gate) * up written to `out`; kEpiPush: stored into every rank's exchange buffer.  A
// template parameter so that the plain kernel carries none of the other two's code (code that
// runs once per CTA costs mostly its instruction fetches).
constexpr int kEpiStore = 0, kEpiSilu = 1, kEpiPush = 2;

template <int NB, int WARPS, bool FP16, int EPI>
__device__ __forceinline__ bool tile_finish(const LinearParams& p, float* slots, int rt, int c0, int c1, uint32_t push_seq) {
  constexpr int EMAX = 512 * NB;  // outputs of one row tile at TT = 4
  const int lane = threadIdx.x & 31;
  const int tt = p.slot_t, sw = 32 * tt;
  const int E = NB * kSubTiles * sw;
  const int seg_lo = rt * p.k_slabs, seg_hi = seg_lo + p.k_slabs;
  const bool full = (c0 <= seg_lo) && (c1 >= seg_hi);
  const bool owner = (c0 <= seg_lo);  // holds the tile's first slab
  int uses = 0;
  if (!full) uses = ld_relaxed_s32(p.counters + rt);  // in flight while the slots are summed
  const uint32_t tag = ((uint32_t)(uses + 1) << 12) | (uint32_t)rt;
  uint2* mine = p.partial + (size_t)blockIdx.x * EMAX;
  bool ok = true;

  // 1. add the warps' deposits in a fixed order (even and odd warps in two chains, four
  //    elements per lane in flight); keep the sums in warp 0's block, or (not the owner of a
  //    split tile) publish them as tagged words and be done.  E is a multiple of 128.
#pragma unroll 1
  for (int e0 = lane; e0 < E; e0 += 128) {
    float even[4] = {0.f, 0.f, 0.f, 0.f}, odd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
    for (int w = 0; w < WARPS; w += 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        even[j] += slots[w * E + e0 + 32 * j];
        odd[j] += slots[(w + 1) * E + e0 + 32 * j];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float acc = even[j] + odd[j];
      if (!full && !owner) {
        st_relaxed_v2(mine + e0 + 32 * j, make_uint2(__float_as_uint(acc), tag));
      } else {
        slots[e0 + 32 * j] = acc;
      }
    }
  }
  if (!full && !owner) return true;

  // 2. owner of a split tile: add the words of the CTAs after this one, up to the one holding
  //    the tile's last slab, in CTA order
  if (!full) {
    const int big = p.rem * (p.base + 1);
    const int last_item = seg_hi - 1;
    const int last = last_item < big ? last_item / (p.base + 1) : p.rem + (last_item - big) / p.base;
#pragma unroll 1
    for (int e0 = lane; e0 < E; e0 += 128) {        // four words per lane ...
#pragma unroll 1
      for (int cb = blockIdx.x + 1; cb <= last; cb += 4) {  // ... of up to four CTAs in flight
        uint2 v[4][4];
#pragma unroll
        for (int ci = 0; ci < 4; ++ci)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[ci][j] = (cb + ci <= last) ? ld_relaxed_v2(p.partial + (size_t)(cb + ci) * EMAX + e0 + 32 * j)
                                         : make_uint2(0u, tag);
#pragma unroll
        for (int ci = 0; ci < 4; ++ci)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t spins = 0;
            while (v[ci][j].y != tag) {
              if (++spins > kSpinLimit) {
                ok = false;
                break;
              }
              v[ci][j] = ld_relaxed_v2(p.partial + (size_t)(cb + ci) * EMAX + e0 + 32 * j);
            }
          }
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // added in CTA order
          float acc = slots[e0 + 32 * j];
#pragma unroll
          for (int ci = 0; ci < 4; ++ci) acc += __uint_as_float(v[ci][j].x);
          slots[e0 + 32 * j] = acc;
        }
      }
    }
  }

  // 3. write the outputs: element (blk, tq, lane) with blk = sub-tile * NB + n-tile.  In a
  //    tensor-parallel push they are first gathered as bf16 in the slot block of warp 1 (summed
  //    above, free now), [batch row][64 tile rows], then stored into this rank's slot of the
  //    current half of every rank's exchange buffer (plain peer stores) as 8-byte words {two
  //    outputs, tag}: a word is valid once its tag is that of this push, so no fence, flag or
  //    second crossing of the link is needed.
  {
    const int g = lane >> 2, c = lane & 3;
    uint16_t* gathered = reinterpret_cast<uint16_t*>(slots + E);
#pragma unroll 1
    for (int blk = 0; blk < kSubTiles * NB; ++blk) {
      const int r = blk / NB, nb = blk - r * NB;
      const int lrow = 16 * r + g + 8 * (c >> 1);
      const int row = rt * kTileRows + lrow;
#pragma unroll 1
      for (int tq = 0; tq < tt; ++tq) {
        const int b = 8 * nb + 2 * tq + (c & 1);
        if (row < p.n && b < p.m) {
          const uint16_t v = from_float<FP16>(slots[blk * sw + tq * 32 + lane]);
          if constexpr (EPI == kEpiPush) gathered[b * kTileRows + lrow] = v;
          else if constexpr (EPI == kEpiStore) p.out[(size_t)b * p.n + row] = v;
        }
      }
    }
    if constexpr (EPI == kEpiSilu) {  // sub-tiles 0,1 hold gate rows, 2,3 the matching up rows
      auto rnd = [](float v) { return to_float<FP16>(from_float<FP16>(v)); };
#pragma unroll 1
      for (int blk = 0; blk < 2 * NB; ++blk) {
        const int r = blk / NB, nb = blk - r * NB;
        const int col = rt * (kTileRows / 2) + 16 * r + g + 8 * (c >> 1);
#pragma unroll 1
        for (int tq = 0; tq < tt; ++tq) {
          const int b = 8 * nb + 2 * tq + (c & 1);
          if (b < p.m) {
            const float gate = rnd(slots[blk * sw + tq * 32 + lane]);
            const float up = rnd(slots[(blk + 2 * NB) * sw + tq * 32 + lane]);
            const float act = rnd(gate / (1.f + __expf(-gate)));
            p.out[(size_t)b * (p.n / 2) + col] = from_float<FP16>(act * up);
          }
        }
      }
    }
    if constexpr (EPI == kEpiPush) {
      __syncwarp();
      const uint32_t tag = push_seq + 1u;
      const size_t base = ((size_t)((push_seq & 1u) * p.tp + p.rank) * p.stage_slot + (size_t)rt * kTileRows) / 2;
#pragma unroll 1
      for (int ch = lane; ch < p.m * (kTileRows / 4); ch += 32) {  // four outputs and two tags per store
        const int b = ch / (kTileRows / 4), part = ch % (kTileRows / 4);
        const uint2 d = *reinterpret_cast<const uint2*>(gathered + b * kTileRows + part * 4);
        const size_t off = base + ((size_t)b * p.n) / 2 + part * 2;
#pragma unroll 1
        for (int j = 0; j < p.tp; ++j) {
          asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p.peer_stage[j] + off), "r"(d.x),
                       "r"(tag), "r"(d.y), "r"(tag)
                       : "memory");
        }
      }
    }
  }
  if (!full) {
    __syncwarp();
    if (lane == 0) p.counters[rt] = (uses + 1) & 0x7FFFF;  // this use of the split tile is done
  }
  return ok;
}

// ---- the kernel -------------------------------------------------------------------
constexpr int kXRowPad = 16;  // x rows in a stage are 16 bytes apart from a 128-byte multiple: no bank conflicts

template <int BITS, int NB, int WARPS, bool FP16, int EPI, bool XRES>
__global__ void __launch_bounds__(WARPS * 32, (NB == 1 || WARPS <= 8) ? 2 : 1)
    linear_lut_kernel(const __grid_constant__ LinearParams p, const __grid_constant__ InlineLut<BITS> inl) {
  using L = Layout<BITS>;
  using T = Table<BITS>;
  constexpr uint32_t kXRow = 128 * L::KSB + kXRowPad;  // bytes between x rows inside a stage
  extern __shared__ __align__(128) uint8_t smem_raw[];

  // The host planned the shared-memory layout for a known window address; refuse to run on
  // anything else (uniform exit before any barrier).
  const uint32_t raw = smem_addr(smem_raw);
  if (raw != p.smem_base) {
    if (threadIdx.x == 0) atomicOr(p.counters + kStatusWord, kStatusSmemLayout);
    return;
  }
#ifdef FDK_TRACE
  const long long tr0 = clock64();
  long long tr_wait = 0, tr_comp = 0, tr_flush = 0, tr_refill = 0, tr_finish = 0;
#define FDK_T(var) var
#else
#define FDK_T(var)
#endif
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int W = WARPS;
  const int S = p.stages;
  const int g = lane >> 2, t = lane & 3;
  float* slots = reinterpret_cast<float*>(smem_raw + (p.slots_addr - raw));
  EpilogueSync* esync = reinterpret_cast<EpilogueSync*>(smem_raw + (p.mbar_addr - raw) + W * S * 8);
  if (threadIdx.x == 0) {
    esync->count[0] = esync->count[1] = 0;
    esync->gen[0] = esync->gen[1] = 0;
    if (XRES) mbar_init(p.xres_bar, 1);
  }
  const uint32_t lane_base = p.table_addr + T::lane_offset(lane);


  // my slab range
  const int cta = blockIdx.x;
  const int c0 = cta * p.base + min(cta, p.rem);
  const int c1 = c0 + p.base + (cta < p.rem ? 1 : 0);

  // this warp's ring: stage s lives at stage_addr(s), its barrier at bar_addr(s)
  auto stage_addr = [&](int s) -> uint32_t {
    const uint32_t q = warp * S + s;
    return q < p.stage_a_count ? p.stage_a_addr + q * p.stage_bytes
                               : p.stage_b_addr + (q - p.stage_a_count) * p.stage_bytes;
  };
  auto bar_addr = [&](int s) -> uint32_t { return p.mbar_addr + (warp * S + s) * 8; };
  // valid x bytes per row for the slab at position kpos of its row tile
  auto x_bytes = [&](int kpos) -> uint32_t {
    const int left = p.k - kpos * L::kSlabK;
    return 2u * (uint32_t)(left < L::kSlabK ? left : L::kSlabK);
  };
  // lane 0: announce the bytes of slab i and start its weight copy
  auto issue_weights = [&](int i, int kpos, int s) {
    const uint32_t bar = bar_addr(s);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                 "r"((uint32_t)L::kSlabBytes + (XRES ? 0u : (uint32_t)p.m * x_bytes(kpos)))
                 : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            stage_addr(s)),
        "l"(p.tiled + (size_t)i * L::kSlabBytes), "r"((uint32_t)L::kSlabBytes), "r"(bar)
        : "memory");
  };
  // lanes 0..m-1: one x row each, for the same slab
  auto issue_x = [&](int kpos, int s) {
    if (!XRES && lane < p.m) {
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
              stage_addr(s) + (uint32_t)L::kSlabBytes + lane * kXRow),
          "l"(p.x + (size_t)lane * p.k + (size_t)kpos * L::kSlabK), "r"(x_bytes(kpos)), "r"(bar_addr(s))
          : "memory");
    }
  };

  int it = c0 + warp;               // next slab of this warp
  int rt = it / p.k_slabs;          // its row tile and position inside the tile
  int ks = it - rt * p.k_slabs;
  // the prefetch cursor runs S slabs ahead
  int pf_it = it, pf_ks = ks;
  auto pf_advance = [&]() {
    pf_it += W;
    pf_ks += W;
    while (pf_ks >= p.k_slabs) pf_ks -= p.k_slabs;
  };

  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(bar_addr(s), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // start streaming before anything else: these copies read weights only
    int i = it, kp = ks;
    for (int s = 0; s < S && i < c1; ++s) {
      issue_weights(i, kp, s);
      i += W;
      kp += W;
      while (kp >= p.k_slabs) kp -= p.k_slabs;
    }
  }
  if (p.lut == nullptr) {
    fill_table<BITS>(p.table_addr, [&](int i) { return inl.w[i]; });
  } else {
    fill_table<BITS>(p.table_addr, [&](int i) { return __ldg(reinterpret_cast<const uint32_t*>(p.lut) + i); });
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // everything above touched only weights; x, out and the workspace follow stream order
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // number of this push = reduces completed before this launch (the reduce kernel counts)
  const uint32_t push_seq = EPI == kEpiPush ? (uint32_t)ld_relaxed_s32(reinterpret_cast<const int*>(p.seq)) : 0u;
  __syncwarp();
  if (XRES && warp == 0) {  // small x: one copy per batch row for the whole kernel
    if (lane == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(p.xres_bar),
                   "r"((uint32_t)p.m * (uint32_t)p.k * 2u)
                   : "memory");
    }
    __syncwarp();
    if (lane < p.m) {
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
              p.xres_addr + lane * p.xres_row),
          "l"(p.x + (size_t)lane * p.k), "r"((uint32_t)p.k * 2u), "r"(p.xres_bar)
          : "memory");
    }
  }
  for (int s = 0; s < S && pf_it < c1; ++s) {
    issue_x(pf_ks, s);
    pf_advance();
  }
  FDK_T(const long long tr1 = clock64();)
  __syncthreads();
  FDK_T(const long long tr2 = clock64();)

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
  bool timed_out = false;
  const int tt = p.slot_t, sw = 32 * tt;

  const uint32_t slot_set_floats = W * kSubTiles * NB * sw;
  auto flush_until = [&](int target) {
    while (cur_rt < target) {
      const int seg = cur_rt - rt_first;
      const int set = p.slot_sets == 2 ? (seg & 1) : 0, turn = p.slot_sets == 2 ? (seg >> 1) : seg;
      float* my_slots = slots + set * slot_set_floats;
      // the slot set is free once the reduction of two row tiles ago has read it
      {
        volatile int* gen = &esync->gen[set];
        uint32_t spins = 0;
        while (*gen != turn) {
          if (++spins > kSpinLimit) {
            timed_out = true;
            break;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          if (t < tt) {
            float4 v = make_float4(tot[r][nb][0], tot[r][nb][1], tot[r][nb][2], tot[r][nb][3]);
            *reinterpret_cast<float4*>(my_slots + ((warp * kSubTiles + r) * NB + nb) * sw + t * 32 + g * 4) = v;
          }
          tot[r][nb][0] = tot[r][nb][1] = tot[r][nb][2] = tot[r][nb][3] = 0.f;
        }
      __threadfence_block();
      __syncwarp();
      int old = 0;
      if (lane == 0) old = atomicAdd(&esync->count[set], 1);
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old == W - 1) {  // every warp of the CTA has deposited: this warp finishes the tile
        __threadfence_block();
        FDK_T(long long tf = clock64();)
        if (!tile_finish<NB, WARPS, FP16, EPI>(p, my_slots, cur_rt, c0, c1, push_seq)) timed_out = true;
        FDK_T(tr_finish += clock64() - tf;)
        __syncwarp();
        if (lane == 0) {
          esync->count[set] = 0;
          __threadfence_block();
          atomicAdd(&esync->gen[set], 1);
        }
      }
      ++cur_rt;
    }
  };

  // One slab: stage address `sa`, slab position `kpos` inside its row tile.
  auto compute = [&](uint32_t sa, int kpos) {
    constexpr bool kPreload = (L::V == 1 && L::KSB > 1);
    uint4 pre[kPreload ? kSubTiles : 1];
    if constexpr (kPreload) {
#pragma unroll
      for (int r = 0; r < kSubTiles; ++r) pre[r] = ring128(sa + (r * 32 + lane) * 16);
    }
    auto block = [&](auto jbc) {
      constexpr int JB = decltype(jbc)::value;
      if ((kpos * L::KSB + JB) * kBlock >= p.k) return;  // padded block: codes and scales are zero
      uint32_t xb[NB][8];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const int b = min(g + 8 * nb, p.m - 1);  // lanes of unused batch columns read a live row
        const uint32_t xa = XRES ? p.xres_addr + b * p.xres_row + (kpos * L::KSB + JB) * 128 + t * 32
                                        : sa + L::kSlabBytes + b * kXRow + JB * 128 + t * 32;
        const uint4 lo = ring128(xa), hi = ring128(xa + 16);
        xb[nb][0] = lo.x; xb[nb][1] = lo.y; xb[nb][2] = lo.z; xb[nb][3] = lo.w;
        xb[nb][4] = hi.x; xb[nb][5] = hi.y; xb[nb][6] = hi.z; xb[nb][7] = hi.w;
      }
      const uint4 sc = ring128(sa + L::kCodeBytes + JB * 128 + g * 16);
      auto sub_tile = [&](auto rc) {
        constexpr int R = decltype(rc)::value;
        uint4 code[L::V];
        if constexpr (kPreload) {
          code[0] = pre[R];
        } else {
#pragma unroll
          for (int v = 0; v < L::V; ++v) code[v] = ring128(sa + ((R * L::V + v) * 32 + lane) * 16);
        }
        uint32_t a[4][4];
        build_fragments<BITS, JB>(code, lane_base, a);
        const uint32_t scw = word_of<R>(sc);
        const float s_lo = pair_lo<FP16>(scw), s_hi = pair_hi<FP16>(scw);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          float acc[4];
          const float zero[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816<FP16>(acc, a[0], xb[nb][0], xb[nb][1], zero);
#pragma unroll
          for (int st = 1; st < 4; ++st) mma16816<FP16>(acc, a[st], xb[nb][2 * st], xb[nb][2 * st + 1], acc);
          tot[R][nb][0] = fmaf(acc[0], s_lo, tot[R][nb][0]);
          tot[R][nb][1] = fmaf(acc[1], s_lo, tot[R][nb][1]);
          tot[R][nb][2] = fmaf(acc[2], s_hi, tot[R][nb][2]);
          tot[R][nb][3] = fmaf(acc[3], s_hi, tot[R][nb][3]);
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

  if (XRES && it < c1) {
    if (!mbar_wait(p.xres_bar, 0)) timed_out = true;
  }
  int s = 0;
  uint32_t parity = 0;
  while (it < c1) {
    FDK_T(long long ta = clock64();)
    if (rt != cur_rt) flush_until(rt);
    FDK_T(long long tb = clock64(); tr_flush += tb - ta;)
    if (!mbar_wait(bar_addr(s), parity)) timed_out = true;  // carry on with whatever is there
    FDK_T(long long tc = clock64(); tr_wait += tc - tb;)
    compute(stage_addr(s), ks);
    __syncwarp();  // every lane has consumed its share of this stage
    FDK_T(long long td = clock64(); tr_comp += td - tc;)
    if (pf_it < c1) {
      if (lane == 0) issue_weights(pf_it, pf_ks, s);
      __syncwarp();
      issue_x(pf_ks, s);
      pf_advance();
    }
    FDK_T(tr_refill += clock64() - td;)
    it += W;
    ks += W;
    while (ks >= p.k_slabs) {
      ks -= p.k_slabs;
      ++rt;
    }
    if (++s == S) {
      s = 0;
      parity ^= 1;
    }
  }
  FDK_T(const long long tr3 = clock64();)
  flush_until(rt_last + 1);
  if (timed_out && lane == 0) atomicOr(p.counters + kStatusWord, kStatusTimeout);
#ifdef FDK_TRACE
  if (p.trace != nullptr && lane == 0) {
    unsigned long long* o = p.trace + ((size_t)blockIdx.x * W + warp) * 8;
    o[0] = tr1 - tr0; o[1] = tr_refill; o[2] = tr3 - tr2; o[3] = clock64() - tr3;
    o[4] = tr_wait; o[5] = tr_comp; o[6] = tr_flush; o[7] = tr_finish + 1;
  }
#endif
#undef FDK_T
}

// ---- host side ----------------------------------------------------------------------


inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

// Plans the shared-memory layout for `warps` warps with `stages` ring stages each; returns
// the dynamic size needed.
template <int BITS, int NB>
size_t plan_smem(uint32_t base, int warps, int stages, LinearParams& p) {
  using L = Layout<BITS>;
  using T = Table<BITS>;
  const uint32_t n_stages = warps * stages;
  const uint32_t tt = ((p.m < 8 ? p.m : 8) + 1) / 2;
  // two sets let a warp deposit its next row tile while the last one is being summed; large
  // deposits (batches of five rows and more) get one set and more warps instead
  const uint32_t sets = tt >= 3 ? 1 : 2;
  p.slot_sets = sets;
  const uint32_t slot_bytes = sets * warps * kSubTiles * NB * 32 * tt * sizeof(float);
  const uint32_t mbar_bytes = align_up(n_stages * 8 + 8 + sizeof(EpilogueSync), 128);  // barriers + epilogue sync words
  // x small enough is staged whole, once per CTA; otherwise its rows travel with each slab
  const uint32_t xres_row = (uint32_t)p.k * 2 + kXRowPad;
  const bool resident = (size_t)p.m * xres_row <= 36 * 1024;
  const uint32_t xres_bytes = resident ? align_up(p.m * xres_row, 128) : 0;
  const uint32_t stage_bytes =
      align_up(L::kSlabBytes + (resident ? 0 : p.m * (128 * L::KSB + kXRowPad)), 128);
  p.stage_bytes = stage_bytes;
  p.stages = stages;
  p.slot_t = tt;
  uint32_t cursor = align_up(base, 128);
  p.smem_base = base;
  p.mbar_addr = cursor;
  p.xres_bar = cursor + n_stages * 8 + sizeof(EpilogueSync);
  cursor += mbar_bytes;
  p.xres_row = xres_row;
  p.xres_addr = resident ? cursor : 0;
  cursor += xres_bytes;
  p.slots_addr = cursor;
  cursor = align_up(cursor + slot_bytes, 128);
  p.table_addr = cursor;
  cursor += T::kBytes;
  p.stage_a_addr = cursor;
  p.stage_a_count = n_stages;
  p.stage_b_addr = cursor;
  cursor += n_stages * stage_bytes;
  return cursor - base;
}

template <int BITS, int NB, int WARPS, bool FP16>
int launch_variant(LinearParams p, const InlineLut<BITS>& inl, size_t smem, int grid, unsigned flags,
                   cudaStream_t stream) {
  const int epi = p.tp > 0 ? kEpiPush : (p.silu ? kEpiSilu : kEpiStore);
  const bool xres = p.xres_addr != 0;
  auto kernel = epi == kEpiPush   ? (xres ? linear_lut_kernel<BITS, NB, WARPS, FP16, kEpiPush, true> : linear_lut_kernel<BITS, NB, WARPS, FP16, kEpiPush, false>)
                : epi == kEpiSilu ? (xres ? linear_lut_kernel<BITS, NB, WARPS, FP16, kEpiSilu, true> : linear_lut_kernel<BITS, NB, WARPS, FP16, kEpiSilu, false>)
                                  : (xres ? linear_lut_kernel<BITS, NB, WARPS, FP16, kEpiStore, true> : linear_lut_kernel<BITS, NB, WARPS, FP16, kEpiStore, false>);
  static size_t configured[6][64] = {};
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  if (configured[2 * epi + xres][dev & 63] < smem) {
    FDK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[2 * epi + xres][dev & 63] = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & FDK_FLAG_PDL) ? 1 : 0;
  FDK_CUDA(cudaLaunchKernelEx(&cfg, kernel, p, inl));
  return FDK_OK;
}

// CTAs are sized so that two fit on an SM (12 or 8 warps, at most half the shared memory):
// with one CTA per SM the other half is free for the NEXT kernel on the stream, which under
// programmatic dependent launch starts its table fill and weight prefetch while this one is
// still running; a large matrix takes both halves itself (two CTAs per SM).  A plan that does
// not fit half an SM gets the whole SM.
template <int BITS, int NB, bool FP16>
int launch(LinearParams p, const void* lut_host, int sm_count, unsigned flags, cudaStream_t stream) {
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
  constexpr int kWide = 12;
  constexpr int kMid = 8;
  constexpr int kNarrow = 4;
  const size_t half_sm = ((size_t)di.max_smem_optin + 1024) / 2 - 1024;  // two CTAs, 1 KB reserved each
  const int widths[3] = {kWide, kMid, kNarrow};
  int best_w = 0, best_s = 0;
  size_t best_smem = 0;
  bool two_per_sm = true;
  bool env_free = true;  // no plan forced from the environment (development builds)
#ifdef FDK_TRACE
  static const char* env_s = getenv("FDK_STAGES");
  static const char* env_w = getenv("FDK_WARPS");
  if (env_s != nullptr) {
    const int want_w = env_w ? atoi(env_w) : kWide;
    LinearParams q = p;
    best_smem = plan_smem<BITS, NB>(base, want_w, atoi(env_s), q);
    best_w = want_w;
    best_s = atoi(env_s);
    two_per_sm = best_smem <= half_sm;
    env_free = false;
  }
#endif
  // Candidates: each width, in half an SM or all of it, with as many stages as fit.  The one
  // that keeps the most warps on an SM wins (two CTAs count double where the grid can be
  // doubled: NB == 1 and enough slabs); ties go to the half-SM plan, which leaves room for the
  // next kernel's prologue.  Plans with a single stage are taken only if nothing else fits.
  int best_score = -1;
  for (int wi = 0; wi < 3 && env_free; ++wi) {
    for (int pass = 0; pass < 2; ++pass) {
      const size_t limit = pass == 0 ? half_sm : (size_t)di.max_smem_optin;
      for (int s = kMaxStages; s >= 1; --s) {
        LinearParams q = p;
        const size_t smem = plan_smem<BITS, NB>(base, widths[wi], s, q);
        if (smem > limit) continue;
        const bool doubled = pass == 0 && NB == 1 && p.total >= 2 * widths[wi] * sm_count;
        const int score = (s >= 2 ? 1000 : 0) + widths[wi] * (doubled ? 2 : 1) * 10 + (pass == 0 ? 1 : 0);
        if (score > best_score) {
          best_score = score;
          best_w = widths[wi];
          best_s = s;
          best_smem = smem;
          two_per_sm = pass == 0;
        }
        break;  // fewer stages of the same plan are never better
      }
    }
  }
  FDK_CHECK_ARG(best_w != 0, FDK_ERR_CUDA, "no shared-memory plan fits %d bytes", di.max_smem_optin);
  plan_smem<BITS, NB>(base, best_w, best_s, p);
  // grid: one CTA per SM, or two when each would still have plenty of slabs (NB == 1 only: the
  // workspace holds one 4 KB partial per CTA for up to 320 CTAs)
  int grid = sm_count;
  if (two_per_sm && NB == 1 && p.total >= 2 * best_w * sm_count) grid = 2 * sm_count;
  if (grid > p.total) grid = p.total;
  p.base = p.total / grid;
  p.rem = p.total % grid;
  if (best_w == kWide) return launch_variant<BITS, NB, kWide, FP16>(p, inl, best_smem, grid, flags, stream);
  if (best_w == kMid) return launch_variant<BITS, NB, kMid, FP16>(p, inl, best_smem, grid, flags, stream);
  return launch_variant<BITS, NB, kNarrow, FP16>(p, inl, best_smem, grid, flags, stream);
}

}  // namespace

template <int BITS>
int launch_bits(const LinearParams& p, const void* lut_host, int grid, int dtype, unsigned flags,
                cudaStream_t stream) {
  const bool wide = p.m > 8;
  if (dtype == FDK_DTYPE_F16) {
    return wide ? launch<BITS, 2, true>(p, lut_host, grid, flags, stream)
                : launch<BITS, 1, true>(p, lut_host, grid, flags, stream);
  }
  return wide ? launch<BITS, 2, false>(p, lut_host, grid, flags, stream)
              : launch<BITS, 1, false>(p, lut_host, grid, flags, stream);
}


}  // namespace fdk
