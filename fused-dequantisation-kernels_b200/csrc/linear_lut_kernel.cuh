// Fused dequantise + GEMV / skinny GEMM for sm_100a:  out[m, n] = x[m, k] . W[n, k]^T,
// W given as tiled low-bit codes + block scales + a lookup table (fdk_layout.cuh).
//
// Shape of the kernel (one persistent CTA per SM: 19 compute warps and one finisher warp for
// batches up to 8 rows, 11 + 1 for 9 to 16 rows):
//   * The weight stream is cut into slabs (64 rows x 64*KSB columns, 2-6 KB).  The
//     slabs of the whole matrix form one linear sequence (row tile major); CTA c owns
//     a contiguous range of it ("stream-K"), its compute warps take slabs round-robin.
//     Every SM therefore streams the same number of bytes (+-1 slab) whatever N and K are.
//   * Weights go from global memory straight into registers: a lane's share of a slab
//     is a handful of 16-byte vectors that are contiguous across the warp (512 B per
//     load instruction, streaming loads that do not allocate in L1).  A warp holds two
//     slabs of registers, used alternately: while it works on one, the loads of its next
//     slab are in flight into the other, and L2 has been asked for the one after that
//     (prefetch.global.L2, a line per lane).  The codes never pass through shared
//     memory.  The first loads are issued before the kernel waits for its predecessor
//     on the stream (programmatic dependent launch): they read weights only.
//   * Every warp reads the x fragments of its slab from L2 as it needs them (x is small and
//     was just written); only the fused RMSNorm keeps a copy of x in shared memory, which
//     is otherwise left to the table lookups.
//   * Codes are turned into tensor-core A fragments by table lookup in shared memory:
//     one code byte indexes a byte table replicated per lane (lut_table.cuh) whose rows
//     are 256 bytes apart in a table that starts at a multiple of 64 KB of the shared
//     window, so a lookup is one PRMT (the code byte dropped into bits 8..15 of the
//     lane's table address) and one conflict-free LDS that returns 2 (4-bit), 4 (2-bit)
//     or 8 (1-bit) 16-bit weights already in fragment order.  The table itself arrives
//     inside the kernel parameters.
//   * mma.sync m16n8k16 accumulates one 64-block in fp32; the block scale multiplies
//     the fp32 block sum (4 FMAs per 1024 weights), then running totals per row.
//     The tensor pipe is used because the FMA work would otherwise compete with the
//     lookups for issue slots; the synchronous MMA form keeps the weights in registers
//     (a tcgen05 MMA would need them written to shared or tensor memory first).  What
//     bounds the main loop is instruction issue: about 130 lookup instructions, 16 MMAs
//     and 24 scale instructions per 4096 weights.
//   * At a row-tile boundary a compute warp deposits its totals in shared memory and moves
//     on; the finisher warp adds the deposits in warp order and writes the outputs.  A row
//     tile split over several CTAs is finished by the CTA holding its first slabs: the
//     others publish their sums to the workspace as {value, tag} words, which that CTA's
//     finisher fetches (bounded polling) while the compute warps are still busy, and adds
//     in CTA order.  The summation order never depends on timing, so results are
//     reproducible bit for bit.
//   * Epilogue variants: plain store; silu(gate) * up for a gate|up weight stored in
//     32 + 32 row groups; or, in tensor-parallel decode, tagged stores of the partial
//     sums into every rank's exchange buffer.
#pragma once
#include <atomic>
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
template <int BITS, int JB, bool WIDE>
__device__ __forceinline__ void build_fragments(const uint4 (&code)[Layout<BITS>::V], uint32_t lane_base,
                                                uint32_t (&a)[4][4]) {
  if constexpr (BITS == 4) {
    const uint4& c = code[0];
    a[0][0] = lut32(entry_addr<4, 0, WIDE>(c.x, lane_base)); a[0][2] = lut32(entry_addr<4, 1, WIDE>(c.x, lane_base));
    a[1][0] = lut32(entry_addr<4, 2, WIDE>(c.x, lane_base)); a[1][2] = lut32(entry_addr<4, 3, WIDE>(c.x, lane_base));
    a[2][0] = lut32(entry_addr<4, 0, WIDE>(c.y, lane_base)); a[2][2] = lut32(entry_addr<4, 1, WIDE>(c.y, lane_base));
    a[3][0] = lut32(entry_addr<4, 2, WIDE>(c.y, lane_base)); a[3][2] = lut32(entry_addr<4, 3, WIDE>(c.y, lane_base));
    a[0][1] = lut32(entry_addr<4, 0, WIDE>(c.z, lane_base)); a[0][3] = lut32(entry_addr<4, 1, WIDE>(c.z, lane_base));
    a[1][1] = lut32(entry_addr<4, 2, WIDE>(c.z, lane_base)); a[1][3] = lut32(entry_addr<4, 3, WIDE>(c.z, lane_base));
    a[2][1] = lut32(entry_addr<4, 0, WIDE>(c.w, lane_base)); a[2][3] = lut32(entry_addr<4, 1, WIDE>(c.w, lane_base));
    a[3][1] = lut32(entry_addr<4, 2, WIDE>(c.w, lane_base)); a[3][3] = lut32(entry_addr<4, 3, WIDE>(c.w, lane_base));
  } else if constexpr (BITS == 2) {
    const uint4& c = code[0];
    const uint32_t wg = word_of<2 * JB>(c), wh = word_of<2 * JB + 1>(c);
    uint2 q;
    q = lut64(entry_addr<2, 0, WIDE>(wg, lane_base)); a[0][0] = q.x; a[0][2] = q.y;
    q = lut64(entry_addr<2, 1, WIDE>(wg, lane_base)); a[1][0] = q.x; a[1][2] = q.y;
    q = lut64(entry_addr<2, 2, WIDE>(wg, lane_base)); a[2][0] = q.x; a[2][2] = q.y;
    q = lut64(entry_addr<2, 3, WIDE>(wg, lane_base)); a[3][0] = q.x; a[3][2] = q.y;
    q = lut64(entry_addr<2, 0, WIDE>(wh, lane_base)); a[0][1] = q.x; a[0][3] = q.y;
    q = lut64(entry_addr<2, 1, WIDE>(wh, lane_base)); a[1][1] = q.x; a[1][3] = q.y;
    q = lut64(entry_addr<2, 2, WIDE>(wh, lane_base)); a[2][1] = q.x; a[2][3] = q.y;
    q = lut64(entry_addr<2, 3, WIDE>(wh, lane_base)); a[3][1] = q.x; a[3][3] = q.y;
  } else if constexpr (BITS == 1) {
    const uint32_t w = word_of<JB>(code[0]);  // bytes 0,1: row g; bytes 2,3: row g+8
    uint4 q;
    q = lut128(entry_addr<1, 0, WIDE>(w, lane_base)); a[0][0] = q.x; a[0][2] = q.y; a[1][0] = q.z; a[1][2] = q.w;
    q = lut128(entry_addr<1, 1, WIDE>(w, lane_base)); a[2][0] = q.x; a[2][2] = q.y; a[3][0] = q.z; a[3][2] = q.w;
    q = lut128(entry_addr<1, 2, WIDE>(w, lane_base)); a[0][1] = q.x; a[0][3] = q.y; a[1][1] = q.z; a[1][3] = q.w;
    q = lut128(entry_addr<1, 3, WIDE>(w, lane_base)); a[2][1] = q.x; a[2][3] = q.y; a[3][1] = q.z; a[3][3] = q.w;
  } else if constexpr (BITS == 8) {
    const uint4& cg = code[0];  // row g: 16 bytes = 16 elements
    const uint4& ch = code[1];  // row g+8
#pragma unroll
    for (int st = 0; st < 4; ++st) {
      const uint32_t wg = word_at(cg, st), wh = word_at(ch, st);
      a[st][0] = prmt<0x7610>(lut32(entry_addr<8, 0, WIDE>(wg, lane_base)), lut32(entry_addr<8, 1, WIDE>(wg, lane_base)));
      a[st][2] = prmt<0x7610>(lut32(entry_addr<8, 2, WIDE>(wg, lane_base)), lut32(entry_addr<8, 3, WIDE>(wg, lane_base)));
      a[st][1] = prmt<0x7610>(lut32(entry_addr<8, 0, WIDE>(wh, lane_base)), lut32(entry_addr<8, 1, WIDE>(wh, lane_base)));
      a[st][3] = prmt<0x7610>(lut32(entry_addr<8, 2, WIDE>(wh, lane_base)), lut32(entry_addr<8, 3, WIDE>(wh, lane_base)));
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
// The warps that stream weights ("compute warps") never finish a row tile themselves: when a
// warp has worked through its slabs of a tile it deposits its totals in shared memory, bumps
// the tile's deposit count and moves on.  One extra warp of the CTA, the FINISHER, does the
// rest, so that every memory round trip of the epilogue runs beside the main loop instead of
// inside it: it waits for the deposits of a tile, adds them in warp order and
//   * writes the outputs, if the CTA holds the whole tile;
//   * publishes the sums, if the CTA holds a later part of a tile that starts in another CTA
//     (the tile is then the first thing the CTA works on): {value, tag} 8-byte words into the
//     CTA's own area of the workspace, never waiting for anybody;
//   * if the CTA holds the FIRST slabs of a tile that continues in the following CTAs (its
//     OWNER; the tile is then the last thing the CTA works on): fetches the words of those CTAs
//     -- as a rule published earlier, so the finisher has them before the compute warps are
//     done -- adds them in CTA order, writes the outputs and bumps the tile's use count.
// tag = (use count + 1) * 4096 + row tile: a word left by an earlier launch or another tile can
// never match.  No fences, no atomics on global memory; every sum has a fixed order, so results
// do not depend on timing.  All waits are bounded and report through the status word.
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

// EPI: what is done with a finished row tile -- kEpiStore: written to `out`; kEpiSilu:
// silu(gate) * up written to `out`; kEpiPush: stored into every rank's exchange buffer.  A
// template parameter so that the plain kernel carries none of the other two's code.
// kEpiResid: added to the residual stream in place, with the sums of squares the next RMSNorm
// needs; kEpiRope: rotary embedding of the q and k heads and the KV-cache append.
constexpr int kEpiStore = 0, kEpiSilu = 1, kEpiPush = 2, kEpiResid = 3, kEpiRope = 4;

// Shared-memory words ahead of everything else (offsets in bytes from the start of the dynamic
// shared memory): the epilogue's sync words, the RMSNorm factors of the batch rows, the
// position and the cos/sin table of the rotary epilogue.
constexpr uint32_t kSmemInv = 32, kSmemPos = 96, kSmemRope = 128, kSmemHead = 512;

// n / k_slabs for n * k_slabs < 2^32, by multiplication with k_magic = ceil(2^32 / k_slabs)
__device__ __forceinline__ int div_k(const LinearParams& p, int n) {
  return p.k_slabs == 1 ? n : (int)__umulhi((uint32_t)n, p.k_magic);
}
__device__ __forceinline__ int cta_begin(const LinearParams& p, int c) { return c * p.base + min(c, p.rem); }
__device__ __forceinline__ int cta_of(const LinearParams& p, int item) {
  const int big = p.rem * (p.base + 1);
  return item < big ? item / (p.base + 1) : p.rem + (item - big) / p.base;
}

// Owner of a split tile: adds the sums published by the CTAs after this one, up to the one
// holding the tile's last slab, in CTA order, into stash[0, E).  Run by one warp, lane l taking
// elements 4 l .. 4 l + 3 of every 128.  Every trip to L2 fetches sixteen words per lane (more
// for two n-tiles): four CTAs' words of one 128-element group where a tile has one group (small
// batches: several CTAs may share a tile), otherwise one CTA's words of four (eight) groups, so
// that the number of trips does not grow with the batch.  A round that finds a stale tag is
// repeated after a short sleep.  Returns false if that ran out.
template <int NB>
__device__ __forceinline__ bool fetch_foreign(const LinearParams& p, float* stash, int rt, uint32_t tag, int E) {
  constexpr int EMAX = 512 * NB;
  const int lane = threadIdx.x & 31;
  const int last = cta_of(p, (rt + 1) * p.k_slabs - 1);
  bool ok = true;
  if (E <= 128) {
    const int e0 = lane * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int cb0 = blockIdx.x + 1; cb0 <= last; cb0 += 4) {
      uint2 v[4][4];
      for (uint32_t round = 0;; ++round) {
        bool fresh = true;
#pragma unroll
        for (int ci = 0; ci < 4; ++ci) {
          const uint2* src = p.partial + (size_t)(cb0 + ci) * EMAX + e0;
#pragma unroll
          for (int j = 0; j < 4; ++j) v[ci][j] = cb0 + ci <= last ? ld_relaxed_v2(src + j) : make_uint2(0u, tag);
        }
#pragma unroll
        for (int ci = 0; ci < 4; ++ci)
#pragma unroll
          for (int j = 0; j < 4; ++j) fresh = fresh && v[ci][j].y == tag;
        if (__all_sync(0xffffffffu, fresh)) break;
        if (round > (kSpinLimit >> 4)) {
          ok = false;
          break;
        }
        __nanosleep(64);
      }
#pragma unroll
      for (int ci = 0; ci < 4; ++ci)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] += __uint_as_float(v[ci][j].x);  // CTA order
    }
    *reinterpret_cast<float4*>(stash + e0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    return ok;
  }
  constexpr int GROUPS = 4 * NB;  // 128-element groups fetched together
#pragma unroll 1
  for (int g0 = 0; g0 * 128 < E; g0 += GROUPS) {
    float acc[GROUPS][4];
#pragma unroll
    for (int gi = 0; gi < GROUPS; ++gi) acc[gi][0] = acc[gi][1] = acc[gi][2] = acc[gi][3] = 0.f;
#pragma unroll 1
    for (int cb = blockIdx.x + 1; cb <= last; ++cb) {
      uint2 v[GROUPS][4];
      const uint2* src = p.partial + (size_t)cb * EMAX + g0 * 128 + lane * 4;
      for (uint32_t round = 0;; ++round) {
        bool fresh = true;
#pragma unroll
        for (int gi = 0; gi < GROUPS; ++gi)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[gi][j] = (g0 + gi) * 128 < E ? ld_relaxed_v2(src + gi * 128 + j) : make_uint2(0u, tag);
#pragma unroll
        for (int gi = 0; gi < GROUPS; ++gi)
#pragma unroll
          for (int j = 0; j < 4; ++j) fresh = fresh && v[gi][j].y == tag;
        if (__all_sync(0xffffffffu, fresh)) break;
        if (round > (kSpinLimit >> 4)) {
          ok = false;
          break;
        }
        __nanosleep(64);
      }
#pragma unroll
      for (int gi = 0; gi < GROUPS; ++gi)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[gi][j] += __uint_as_float(v[gi][j].x);  // CTA order
    }
#pragma unroll
    for (int gi = 0; gi < GROUPS; ++gi)
      if ((g0 + gi) * 128 < E)
        *reinterpret_cast<float4*>(stash + (g0 + gi) * 128 + lane * 4) =
            make_float4(acc[gi][0], acc[gi][1], acc[gi][2], acc[gi][3]);
  }
  return ok;
}

// Run by the finisher warp once every compute warp has deposited.  `slots` is the slot set of
// this row tile: per warp one block of E = NB * 4 * SW floats laid out
// [sub-tile][n-tile][t][g][4].  `foreign`: stash holds the other CTAs' sums (owner of a split
// tile).  `publish`: the sums go to `mine` in the workspace as tagged words and nothing else is done.
template <int NB, int DEPOSITS, bool FP16, int EPI, bool SCALE>
__device__ __forceinline__ void tile_finish(const LinearParams& p, float* slots, uint16_t* gathered,
                                            const float* stash, uint2* mine, bool foreign, bool publish, uint32_t tag,
                                            int rt, uint32_t push_seq, const uint32_t (&hpre)[8 * NB], uint32_t wpre,
                                            const uint8_t* smem_head) {
  const int lane = threadIdx.x & 31;
  const int tt = p.slot_t, sw = 32 * tt;
  const int E = NB * kSubTiles * sw;

  // 1. add the warps' deposits in a fixed order (even and odd warps in two chains), then the
  //    other CTAs' sums.  Lane l takes elements 4 l .. 4 l + 3 of every 128: the four
  //    accumulators {row g: two batch columns, row g + 8: the same} of one lane of the
  //    depositing warps.  The sums are published, stored as outputs straight from the
  //    registers (plain epilogue), or kept in warp 0's block for step 2.
#pragma unroll 1
  for (int e0 = lane * 4; e0 < E; e0 += 128) {
    float4 even = make_float4(0.f, 0.f, 0.f, 0.f), odd = even;
#pragma unroll 5
    for (int w = 0; w + 1 < DEPOSITS; w += 2) {
      const float4 a = *reinterpret_cast<const float4*>(slots + w * E + e0);
      const float4 b = *reinterpret_cast<const float4*>(slots + (w + 1) * E + e0);
      even.x += a.x; even.y += a.y; even.z += a.z; even.w += a.w;
      odd.x += b.x; odd.y += b.y; odd.z += b.z; odd.w += b.w;
    }
    if (DEPOSITS & 1) {
      const float4 a = *reinterpret_cast<const float4*>(slots + (DEPOSITS - 1) * E + e0);
      even.x += a.x; even.y += a.y; even.z += a.z; even.w += a.w;
    }
    float acc[4] = {even.x + odd.x, even.y + odd.y, even.z + odd.z, even.w + odd.w};
    if (foreign) {
      const float4 f = *reinterpret_cast<const float4*>(stash + e0);
      acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
    }
    if (SCALE && !publish) {
      // deferred RMSNorm: the complete sums of batch row b are multiplied by the row's factor
      // (element e = ((blk * tt + tq) * 8 + g) * 4 + i holds batch row 8 nb + 2 tq + (i & 1))
      const float* inv = reinterpret_cast<const float*>(smem_head + kSmemInv);
      const int bt = e0 >> 5, blk = bt / tt, tq = bt - blk * tt, nb = blk % NB;
      const float f0 = inv[8 * nb + 2 * tq], f1 = inv[8 * nb + 2 * tq + 1];
      acc[0] *= f0; acc[1] *= f1; acc[2] *= f0; acc[3] *= f1;
    }
    if (publish) {
#pragma unroll
      for (int j = 0; j < 4; ++j) st_relaxed_v2(mine + e0 + j, make_uint2(__float_as_uint(acc[j]), tag));
    } else if constexpr (EPI == kEpiStore) {
      // element e = ((blk * tt + tq) * 8 + g) * 4 + i, blk = sub-tile * NB + n-tile
      const int idx = e0 >> 2, g = idx & 7, bt = idx >> 3;
      const int blk = bt / tt, tq = bt - blk * tt;
      const int r = blk / NB, nb = blk - r * NB;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = rt * kTileRows + 16 * r + g + 8 * (i >> 1);
        const int b = 8 * nb + 2 * tq + (i & 1);
        if (row < p.n && b < p.m) p.out[(size_t)b * p.n + row] = from_float<FP16>(acc[i]);
      }
    } else {
      *reinterpret_cast<float4*>(slots + e0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
  }
  if (publish || EPI == kEpiStore) return;
  __syncwarp();

  // 2. write the outputs: element (blk, tq, lane) with blk = sub-tile * NB + n-tile.  In a
  //    tensor-parallel push they are first gathered as bf16 in `gathered` (the slot block of warp
  //    1, summed above and free now, or a block of its own), [batch row][64 tile rows], then stored into this rank's slot of the
  //    current half of every rank's exchange buffer (plain peer stores) as 8-byte words {two
  //    outputs, tag}: a word is valid once its tag is that of this push, so no fence, flag or
  //    second crossing of the link is needed.
  {
    const int g = lane >> 2, c = lane & 3;
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
    if constexpr (EPI == kEpiResid) {
      // lane l takes rows l and l + 32 of the tile, for every batch row: y rounded as if stored,
      // added to the residual stream (the values of h were fetched before the deposits came in),
      // squares summed over the tile in a fixed order
      const int row_tiles = (p.n + kTileRows - 1) / kTileRows;
#pragma unroll
      for (int b = 0; b < 8 * NB; ++b) {
        if (b < p.m) {
          const int nb = b >> 3, tq = (b & 7) >> 1;
          float sq = 0.f;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int lrow = lane + 32 * half;
            const int r = lrow >> 4, gg = lrow & 7, hi = (lrow >> 3) & 1;
            const int e = (((r * NB + nb) * tt + tq) * 8 + gg) * 4 + 2 * hi + (b & 1);
            const int row = rt * kTileRows + lrow;
            if (row < p.n) {
              const float y = to_float<FP16>(from_float<FP16>(slots[e]));
              const float hold = to_float<FP16>((uint16_t)(half ? hpre[b] >> 16 : hpre[b] & 0xFFFFu));
              const uint16_t hnew = from_float<FP16>(hold + y);
              p.resid_h[(size_t)b * p.n + row] = hnew;
              const float hf = to_float<FP16>(hnew);
              sq = fmaf(hf, hf, sq);
              if (p.resid_w != nullptr) {  // the next RMSNorm's weight folded in: x of the next projection
                const float w = to_float<FP16>((uint16_t)(half ? wpre >> 16 : wpre & 0xFFFFu));
                p.resid_x[(size_t)b * p.n + row] = from_float<FP16>(hf * w);
              }
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
          if (lane == 0) p.resid_ss[(size_t)b * row_tiles + rt] = sq;
        }
      }
    }
    if constexpr (EPI == kEpiRope) {
      // tile rt is half t of head rt / 2; for q and k heads its sub-tiles 0,1 hold dimensions
      // 32 t .. 32 t + 31 and sub-tiles 2,3 their partners 64 further on
      auto rnd = [](float v) { return to_float<FP16>(from_float<FP16>(v)); };
      const int head = rt >> 1, th = rt & 1;
      const long long pos = *reinterpret_cast<const long long*>(smem_head + kSmemPos);
      const bool in_cache = pos >= 0 && pos < p.max_len;
      const uint32_t* table = reinterpret_cast<const uint32_t*>(smem_head + kSmemRope);
#pragma unroll 1
      for (int blk = 0; blk < 2 * NB; ++blk) {
        const int r = blk / NB, nb = blk - r * NB;
        const int lrow = 16 * r + g + 8 * (c >> 1);  // 0 .. 31
#pragma unroll 1
        for (int tq = 0; tq < tt; ++tq) {
          const int b = 8 * nb + 2 * tq + (c & 1);
          if (b < p.m) {
            const float x0 = rnd(slots[blk * sw + tq * 32 + lane]);
            const float x1 = rnd(slots[(blk + 2 * NB) * sw + tq * 32 + lane]);
            if (head < p.q_heads + p.kv_heads) {
              const uint32_t cs = table[32 * th + lrow];
              const float co = pair_lo<FP16>(cs), si = pair_hi<FP16>(cs);
              const uint16_t o0 = from_float<FP16>(rnd(x0 * co) + rnd(-x1 * si));
              const uint16_t o1 = from_float<FP16>(rnd(x1 * co) + rnd(x0 * si));
              uint16_t* dst = nullptr;
              if (head < p.q_heads) {
                dst = p.q_out + ((size_t)b * p.q_heads + head) * 128;
              } else if (in_cache) {
                dst = p.k_cache + (((size_t)b * p.kv_heads + (head - p.q_heads)) * p.max_len + pos) * 128;
              }
              if (dst != nullptr) {
                dst[32 * th + lrow] = o0;
                dst[32 * th + lrow + 64] = o1;
              }
            } else if (in_cache) {  // v: rows in their own order
              uint16_t* dst = p.v_cache + (((size_t)b * p.kv_heads + (head - p.q_heads - p.kv_heads)) * p.max_len + pos) * 128;
              dst[64 * th + lrow] = from_float<FP16>(x0);
              dst[64 * th + lrow + 32] = from_float<FP16>(x1);
            }
          }
        }
      }
    }
    if constexpr (EPI == kEpiPush) {
      __syncwarp();
      const uint32_t ptag = push_seq + 1u;
      const size_t base = ((size_t)((push_seq & 1u) * p.tp + p.rank) * p.stage_slot + (size_t)rt * kTileRows) / 2;
#pragma unroll 1
      for (int ch = lane; ch < p.m * (kTileRows / 4); ch += 32) {  // four outputs and two tags per store
        const int b = ch / (kTileRows / 4), part = ch % (kTileRows / 4);
        const uint2 d = *reinterpret_cast<const uint2*>(gathered + b * kTileRows + part * 4);
        const size_t off = base + ((size_t)b * p.n) / 2 + part * 2;
#pragma unroll 1
        for (int j = 0; j < p.tp; ++j) {
          asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p.peer_stage[j] + off), "r"(d.x),
                       "r"(ptag), "r"(d.y), "r"(ptag)
                       : "memory");
        }
      }
    }
  }
}

// ---- the kernel -------------------------------------------------------------------
template <int NB>
// compute warps per CTA; with the finisher a multiple of four.  One n-tile: 19 warps of 96
// registers.  Two n-tiles need ~160 registers: 11 warps of 168 (15 warps of 128 spilled in the
// loop and ran the 16-row case 4 us slower at every shape measured).
constexpr int kGemvWarps = NB == 1 ? 19 : 11;
constexpr int kXRowPad = 16;  // resident x rows are 16 bytes apart from a 128-byte multiple: no bank conflicts

// A lane's share of one slab: code vectors [sub-tile][v] and the scale vector of each block.
template <int BITS>
struct SlabRegs {
  uint4 code[kSubTiles][Layout<BITS>::V];
  uint4 sc[Layout<BITS>::KSB];
};

// Streaming load: weights are read once, so they are kept out of L1.
__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// x: written by the previous kernel on the stream, read through L2.
__device__ __forceinline__ uint4 ldg_l2(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Asks L2 for one whole slab, a 128-byte line per lane (a hint: no registers, no shared memory).
template <int BITS>
__device__ __forceinline__ void prefetch_slab_l2(const uint8_t* slab, int lane) {
  constexpr int kLines = Layout<BITS>::kSlabBytes / 128;
#pragma unroll
  for (int l = 0; l < kLines; l += 32)
    if (l + lane < kLines) asm volatile("prefetch.global.L2 [%0];" ::"l"(slab + (l + lane) * 128));
}

template <int BITS>
__device__ __forceinline__ void load_slab(SlabRegs<BITS>& s, const uint8_t* slab, int lane) {
  using L = Layout<BITS>;
  const uint8_t* c = slab + lane * 16;
#pragma unroll
  for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
    for (int v = 0; v < L::V; ++v) s.code[r][v] = ldg_stream(c + (r * L::V + v) * 512);
  const uint8_t* sp = slab + L::kCodeBytes + (lane >> 2) * 16;
#pragma unroll
  for (int jb = 0; jb < L::KSB; ++jb) s.sc[jb] = ldg_stream(sp + jb * 128);
}

// Spins (bounded, backing off) until *word == want.
__device__ __forceinline__ bool wait_shared_word(volatile int* word, int want) {
  for (uint32_t spins = 0; *word != want; ++spins) {
    if (spins > kSpinLimit) return false;
    if (spins > 8) __nanosleep(32);
  }
  return true;
}

// WARPS compute warps and one finisher warp (the last one).
// NORM: kNormNone; kNormInput: x is the RMSNorm of p.norm_h, applied while x is staged (needs
// resident x); kNormOutput: the deferred form -- x comes with the norm weight folded in and the
// complete sums are multiplied by the batch rows' norm factors.
constexpr int kNormNone = 0, kNormInput = 1, kNormOutput = 2;
// XM: where a warp finds x -- kXDirect: fragments read from L2 as they are needed (x is small
// and was just written by the kernel before this one); kXResident: all of x copied once per CTA
// into shared memory, which the fused RMSNorm needs.  Measured on a B200 at every batch size
// from 1 to 16 and every decode shape, reading the fragments straight from L2 beats both a
// resident copy and a per-warp cp.async ring (8192^2: 10.65 -> 10.37 us at one row, 21.0 ->
// 17.1 us at 16 rows): shared memory is the busiest unit of this kernel (table lookups), and
// x does not have to go through it.
constexpr int kXDirect = 0, kXResident = 1;

template <int BITS, int NB, int WARPS, bool FP16, int EPI, int XM, int NORM, bool TEAM>
__global__ void __launch_bounds__((WARPS + 1) * 32, 1)
    linear_lut_kernel(const __grid_constant__ LinearParams p, const __grid_constant__ InlineLut<BITS> inl) {
  using L = Layout<BITS>;
  constexpr bool WIDE = BITS != 3;
  using T = Table<BITS, WIDE>;
  constexpr int W = WARPS;
  constexpr int kThreads = (WARPS + 1) * 32;
  extern __shared__ __align__(128) uint8_t smem_raw[];

  const uint32_t raw = smem_addr(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  EpilogueSync* esync = reinterpret_cast<EpilogueSync*>(smem_raw);
  float* slots = reinterpret_cast<float*>(smem_raw + p.slots_off);
  const uint32_t table_addr = raw + p.table_off;
  const uint32_t lane_base = table_addr + T::lane_offset(lane);
  const uint32_t xres_addr = raw + p.xres_off;
  if (threadIdx.x == 0) {
    esync->count[0] = esync->count[1] = 0;
    esync->gen[0] = esync->gen[1] = 0;
  }

  // my slab range [c0, c1); compute warp w takes slabs c0 + w, c0 + w + W, ...
  const int cta = blockIdx.x;
  const int c0 = cta_begin(p, cta);
  const int c1 = c0 + p.base + (cta < p.rem ? 1 : 0);
  int it = c0 + warp;  // the slab in the registers
  const uint8_t* wp = p.tiled + (size_t)it * L::kSlabBytes;
  constexpr uint32_t kStep = W * L::kSlabBytes;  // bytes between consecutive slabs of a warp

  // start streaming before anything else: these loads read weights only
  SlabRegs<BITS> s, s2;
  if (warp < W && it < c1) {
    load_slab<BITS>(s, wp, lane);
    if (it + W < c1) prefetch_slab_l2<BITS>(wp + kStep, lane);
  }
  {
    const bool from_params = p.lut == nullptr;
    auto word = [&](int i) {
      return from_params ? inl.w[i] : __ldg(reinterpret_cast<const uint32_t*>(p.lut) + i);
    };
    if constexpr (BITS == 4 || BITS == 2 || BITS == 1) {
      fill_table_unrolled<BITS, WIDE, kThreads>(table_addr, word, (int)threadIdx.x);
    } else {
      fill_table<BITS, WIDE>(table_addr, kThreads, word, (int)threadIdx.x);
    }
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // everything above touched only weights; x, out and the workspace follow stream order
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (WIDE && (table_addr & 0xFFFFu) != 0u) {  // the host planned for another window address (uniform exit)
    if (threadIdx.x == 0) atomicOr(p.counters + kStatusWord, kStatusSmemLayout);
    return;
  }
  const int rt_first = div_k(p, c0);
  const int rt_last = div_k(p, c1 - 1);
  // finisher: the use counts of the two tiles of this CTA that can be split (first and last)
  // and the number of this push, fetched now so that their latency is out of the way
  int uses_first = 0, uses_last = 0;
  uint32_t push_seq = 0;
  if (warp == W) {
    uses_first = ld_relaxed_s32(p.counters + rt_first);
    uses_last = ld_relaxed_s32(p.counters + rt_last);
    // number of this push = reduces completed before this launch (the reduce kernel counts)
    if (EPI == kEpiPush) push_seq = (uint32_t)ld_relaxed_s32(reinterpret_cast<const int*>(p.seq));
  }
  if constexpr (XM == kXResident && NORM == kNormInput) {
    // x = norm_w * round(h * rsqrt(mean(h^2) + eps)), the roundings of the separate RMSNorm
    // kernel; mean(h^2) from the sums of squares the previous projection left per 64 elements.
    // A thread's first two vectors of h and of the norm weight are requested before the
    // factors are computed, so that all of it costs one round trip to L2.
    static_assert(NORM != kNormInput || XM == kXResident, "the norm is applied while x is staged in shared memory");
    const int vecs = p.k >> 3, total = p.m * vecs;
    float* inv_smem = reinterpret_cast<float*>(smem_raw + kSmemInv);
    uint4 hv[2], wv[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = threadIdx.x + u * kThreads;
      if (i < total) {
        hv[u] = ldg_l2(p.norm_h + (size_t)i * 8);
        wv[u] = ldg_l2(p.norm_w + (size_t)(i % vecs) * 8);
      }
    }
    if (warp < p.m) {  // one warp per batch row: partial sums added in a fixed order
      // four loads per lane in flight (128 tiles, i.e. 8192 columns, in one trip to L2)
      float ssum = 0.f;
      const float* ss_row = p.norm_ss + (size_t)warp * p.norm_tiles;
#pragma unroll 1
      for (int j0 = lane; j0 < p.norm_tiles; j0 += 128) {
        float part[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) part[u] = j0 + 32 * u < p.norm_tiles ? __ldcg(ss_row + j0 + 32 * u) : 0.f;
        ssum += (part[0] + part[1]) + (part[2] + part[3]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
      if (lane == 0) inv_smem[warp] = rsqrtf(ssum / (float)p.k + p.norm_eps);
    }
    __syncthreads();
    auto stage = [&](int i, const uint4& h4, const uint4& w4) {
      const int row = i / vecs, c = i - row * vecs;
      const float inv = inv_smem[row];
      const uint32_t* hw = reinterpret_cast<const uint32_t*>(&h4);
      const uint32_t* ww = reinterpret_cast<const uint32_t*>(&w4);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = to_float<FP16>(from_float<FP16>(pair_lo<FP16>(hw[j]) * inv)) * pair_lo<FP16>(ww[j]);
        const float b = to_float<FP16>(from_float<FP16>(pair_hi<FP16>(hw[j]) * inv)) * pair_hi<FP16>(ww[j]);
        o[j] = (uint32_t)from_float<FP16>(a) | ((uint32_t)from_float<FP16>(b) << 16);
      }
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(xres_addr + row * p.xres_row + c * 16), "r"(o[0]),
                   "r"(o[1]), "r"(o[2]), "r"(o[3])
                   : "memory");
    };
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = threadIdx.x + u * kThreads;
      if (i < total) stage(i, hv[u], wv[u]);
    }
    // the rest four vectors per thread at a time: their eight loads are in flight together
#pragma unroll 1
    for (int i0 = threadIdx.x + 2 * kThreads; i0 < total; i0 += 4 * kThreads) {
      uint4 h4[4], w4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kThreads;
        if (i < total) {
          h4[u] = ldg_l2(p.norm_h + (size_t)i * 8);
          w4[u] = ldg_l2(p.norm_w + (size_t)(i % vecs) * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kThreads;
        if (i < total) stage(i, h4[u], w4[u]);
      }
    }
  } else if constexpr (XM == kXResident) {
    // x fits: one copy per CTA.  x is contiguous ([m, k]), so the copy runs over all of its
    // 16-byte vectors at once, eight loads per thread in flight (one trip to L2 per eight
    // vectors instead of one per batch row); a row of the copy is 16 bytes longer than k.
    const int vecs = p.k >> 3, total = p.m * vecs;
    constexpr int kStageBatch = 8;
    int row = 0, c = threadIdx.x;
#pragma unroll 1
    for (int i0 = threadIdx.x; i0 < total; i0 += kStageBatch * kThreads) {
      uint4 xv[kStageBatch];
#pragma unroll
      for (int u = 0; u < kStageBatch; ++u)
        if (i0 + u * kThreads < total) xv[u] = ldg_l2(p.x + (size_t)(i0 + u * kThreads) * 8);
#pragma unroll
      for (int u = 0; u < kStageBatch; ++u) {
        if (i0 + u * kThreads < total) {
          while (c >= vecs) {
            c -= vecs;
            ++row;
          }
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(xres_addr + row * p.xres_row + c * 16), "r"(xv[u].x),
                       "r"(xv[u].y), "r"(xv[u].z), "r"(xv[u].w)
                       : "memory");
          c += kThreads;
        }
      }
    }
  }
  __syncthreads();  // table, x and the epilogue's sync words are in place

  const int tt = p.slot_t, sw = 32 * tt;
  const int E = NB * kSubTiles * sw;  // sums of one row tile
  const uint32_t slot_set_floats = W * E;
  // Team mode (large deposits): the compute warps add their deposits themselves, every warp a
  // slice, into one of two blocks of E sums; the finisher starts from those.  A template
  // parameter: the kernels of small batches carry none of it.
  constexpr bool team = TEAM;
  float* tsum = reinterpret_cast<float*>(smem_raw + p.tsum_off);
  bool timed_out = false;

  if (warp == W) {
    // ---- finisher ----
    float* stash = reinterpret_cast<float*>(smem_raw + p.stash_off);
    // what only this warp's epilogues read is fetched here, after the CTA-wide barrier, so that
    // the compute warps do not wait for these trips to L2
    if constexpr (NORM == kNormOutput) {
      // deferred RMSNorm: factor of every batch row from the per-tile sums of squares (four loads
      // per lane in flight, fixed order), kept in shared memory for this warp's epilogues
      float* inv_smem = reinterpret_cast<float*>(smem_raw + kSmemInv);
#pragma unroll 1
      for (int b0 = 0; b0 < 8 * NB; b0 += 4) {  // four batch rows at a time: sixteen loads per lane in flight
        float ssum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int j0 = lane; j0 < p.scale_tiles; j0 += 128) {
          float part[4][4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int u = 0; u < 4; ++u)
              part[i][u] = (b0 + i < p.m && j0 + 32 * u < p.scale_tiles)
                               ? __ldcg(p.scale_ss + (size_t)(b0 + i) * p.scale_tiles + j0 + 32 * u)
                               : 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) ssum[i] += (part[i][0] + part[i][1]) + (part[i][2] + part[i][3]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ssum[i] += __shfl_xor_sync(0xffffffffu, ssum[i], o);
          if (lane == 0) inv_smem[b0 + i] = b0 + i < p.m ? rsqrtf(ssum[i] / (float)p.k + p.scale_eps) : 0.f;
        }
        if (b0 + 4 >= p.m) {  // the remaining rows are unused: zero factors
          if (lane == 0)
            for (int b = b0 + 4; b < 8 * NB; ++b) inv_smem[b] = 0.f;
          break;
        }
      }
      __syncwarp();
    }
    if constexpr (EPI == kEpiRope) {  // the position and its cos/sin table, kept in shared memory
      uint32_t* table = reinterpret_cast<uint32_t*>(smem_raw + kSmemRope);
      table[lane] = __ldcg(p.rope_table + lane);
      table[lane + 32] = __ldcg(p.rope_table + lane + 32);
      if (lane == 0) *reinterpret_cast<long long*>(smem_raw + kSmemPos) = *reinterpret_cast<const volatile long long*>(p.rope_pos);
    }
    __syncwarp();
    for (int rt = rt_first; rt <= rt_last; ++rt) {
      const int seg = rt - rt_first;
      const int set = p.slot_sets == 2 ? (seg & 1) : 0;
      float* my_slots = team ? tsum + set * E : slots + set * slot_set_floats;
      uint16_t* gathered = reinterpret_cast<uint16_t*>(team ? tsum + 2 * E : my_slots + E);
      const int seg_lo = rt * p.k_slabs, seg_hi = seg_lo + p.k_slabs;
      const bool full = (c0 <= seg_lo) && (c1 >= seg_hi);
      const bool owner = (c0 <= seg_lo);  // holds the tile's first slab
      const int uses = rt == rt_first ? uses_first : uses_last;  // only those two can be split
      const uint32_t tag = ((uint32_t)(uses + 1) << 12) | (uint32_t)rt;
      uint32_t hpre[8 * NB] = {};
      uint32_t wpre = 0;  // the next norm's weights of rows lane and lane + 32 of the tile
      // the tile's part of the residual stream, requested before the other CTAs' sums are polled
      // and the deposits come in
      if constexpr (EPI == kEpiResid) {
        if (full || owner) {
          if (p.resid_w != nullptr) {
            const int row = rt * kTileRows + lane;
            const uint16_t lo = row < p.n ? __ldg(p.resid_w + row) : (uint16_t)0;
            const uint16_t hi = row + 32 < p.n ? __ldg(p.resid_w + row + 32) : (uint16_t)0;
            wpre = (uint32_t)lo | ((uint32_t)hi << 16);
          }
#pragma unroll
          for (int b = 0; b < 8 * NB; ++b) {
            if (b < p.m) {
              const int row = rt * kTileRows + lane;
              const uint16_t lo = row < p.n ? __ldcg(p.resid_h + (size_t)b * p.n + row) : (uint16_t)0;
              const uint16_t hi = row + 32 < p.n ? __ldcg(p.resid_h + (size_t)b * p.n + row + 32) : (uint16_t)0;
              hpre[b] = (uint32_t)lo | ((uint32_t)hi << 16);
            }
          }
        }
      }
      if (!full && owner) {
        if (!fetch_foreign<NB>(p, stash, rt, tag, E)) timed_out = true;
        __syncwarp();
      }
      if (!wait_shared_word(&esync->count[set], W)) timed_out = true;
      __threadfence_block();
      if constexpr (team) {  // one block of sums, made by the compute warps
        tile_finish<NB, 1, FP16, EPI, NORM == kNormOutput>(p, my_slots, gathered, stash, p.partial + (size_t)cta * (512 * NB), !full && owner,
                                      !full && !owner, tag, rt, push_seq, hpre, wpre, smem_raw);
      } else {
        tile_finish<NB, WARPS, FP16, EPI, NORM == kNormOutput>(p, my_slots, gathered, stash, p.partial + (size_t)cta * (512 * NB),
                                          !full && owner, !full && !owner, tag, rt, push_seq, hpre, wpre, smem_raw);
      }
      __syncwarp();
      if (lane == 0) {
        if (!full && owner) p.counters[rt] = (uses + 1) & 0x7FFFF;  // this use of the split tile is done
        esync->count[set] = 0;
        __threadfence_block();
        atomicAdd(&esync->gen[set], 1);
      }
      __syncwarp();
    }
    if (timed_out && lane == 0) atomicOr(p.counters + kStatusWord, kStatusTimeout);
    return;
  }

  // ---- compute warps ----
  float tot[kSubTiles][NB][4];
#pragma unroll
  for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) tot[r][nb][i] = 0.f;

  int rt = div_k(p, it);  // row tile of slab `it` and its position inside the tile
  int ks = it - rt * p.k_slabs;
  int cur_rt = rt_first;

  // Deposits the totals of row tiles cur_rt .. target - 1 (zeros for tiles in which this warp
  // had no slab) and clears them.
  auto flush_until = [&](int target) {
    while (cur_rt < target) {
      const int seg = cur_rt - rt_first;
      const int set = p.slot_sets == 2 ? (seg & 1) : 0, turn = p.slot_sets == 2 ? (seg >> 1) : seg;
      float* my_slots = slots + set * slot_set_floats;
      // the slot set is free once the finisher has summed the tile that used it before
      if (!wait_shared_word(&esync->gen[set], turn)) timed_out = true;
      if constexpr (team) {
        // one block of deposits, filled and added up in `slot_phases` parts of the tile's four
        // sub-tiles (fewer sub-tiles at a time where shared memory is short); the adding follows
        // the finisher's order, so the sums do not depend on the mode
        const int rshift = p.slot_phases == 1 ? 2 : p.slot_phases == 2 ? 1 : 0, rpp = 1 << rshift;
        const int Eph = rpp * NB * sw;
        float* sums = tsum + set * E;
#pragma unroll 1
        for (int ph = 0; ph < (int)p.slot_phases; ++ph) {
#pragma unroll
          for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
              if ((r >> rshift) == ph && t < tt) {
                float4 dv = make_float4(tot[r][nb][0], tot[r][nb][1], tot[r][nb][2], tot[r][nb][3]);
                *reinterpret_cast<float4*>(slots + ((warp * rpp + (r & (rpp - 1))) * NB + nb) * sw + t * 32 + g * 4) = dv;
              }
          asm volatile("bar.sync 1, %0;" ::"r"(W * 32) : "memory");
#pragma unroll 1
          for (int e0 = 4 * (warp * 32 + lane); e0 < Eph; e0 += 4 * W * 32) {
            float4 even = make_float4(0.f, 0.f, 0.f, 0.f), odd = even;
#pragma unroll 5
            for (int w = 0; w + 1 < W; w += 2) {
              const float4 a = *reinterpret_cast<const float4*>(slots + w * Eph + e0);
              const float4 b = *reinterpret_cast<const float4*>(slots + (w + 1) * Eph + e0);
              even.x += a.x; even.y += a.y; even.z += a.z; even.w += a.w;
              odd.x += b.x; odd.y += b.y; odd.z += b.z; odd.w += b.w;
            }
            if (W & 1) {
              const float4 a = *reinterpret_cast<const float4*>(slots + (W - 1) * Eph + e0);
              even.x += a.x; even.y += a.y; even.z += a.z; even.w += a.w;
            }
            *reinterpret_cast<float4*>(sums + ph * Eph + e0) =
                make_float4(even.x + odd.x, even.y + odd.y, even.z + odd.z, even.w + odd.w);
          }
          asm volatile("bar.sync 1, %0;" ::"r"(W * 32) : "memory");
        }
#pragma unroll
        for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) tot[r][nb][0] = tot[r][nb][1] = tot[r][nb][2] = tot[r][nb][3] = 0.f;
      } else {
#pragma unroll
        for (int r = 0; r < kSubTiles; ++r)
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            if (t < tt) {
              float4 dv = make_float4(tot[r][nb][0], tot[r][nb][1], tot[r][nb][2], tot[r][nb][3]);
              *reinterpret_cast<float4*>(my_slots + ((warp * kSubTiles + r) * NB + nb) * sw + t * 32 + g * 4) = dv;
            }
            tot[r][nb][0] = tot[r][nb][1] = tot[r][nb][2] = tot[r][nb][3] = 0.f;
          }
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) atomicAdd(&esync->count[set], 1);
      ++cur_rt;
    }
  };

  // per-lane address of this lane's x fragment of column 0, per batch-column group
  uint32_t x_lane[NB];  // resident x: shared-memory address; otherwise: element offset into x
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int b = min(g + 8 * nb, p.m - 1);  // lanes of unused batch columns read a live row
    x_lane[nb] = XM == kXResident ? xres_addr + b * p.xres_row + t * 32 : (uint32_t)(b * p.k + t * 16);
  }

  // Works on the slab held in `s`, at position `kpos` inside its row tile.
  auto compute = [&](const SlabRegs<BITS>& s, int kpos) {
    auto block = [&](auto jbc) {
      constexpr int JB = decltype(jbc)::value;
      const int col = (kpos * L::KSB + JB) * kBlock;
      if (L::KSB > 1 && col >= p.k) return;  // a padded block holds zero codes and scales
      uint32_t xb[NB][8];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        uint4 lo, hi;
        if constexpr (XM == kXResident) {
          lo = ring128(x_lane[nb] + col * 2);
          hi = ring128(x_lane[nb] + col * 2 + 16);
        } else {
          lo = ldg_l2(p.x + x_lane[nb] + col);
          hi = ldg_l2(p.x + x_lane[nb] + col + 8);
        }
        xb[nb][0] = lo.x; xb[nb][1] = lo.y; xb[nb][2] = lo.z; xb[nb][3] = lo.w;
        xb[nb][4] = hi.x; xb[nb][5] = hi.y; xb[nb][6] = hi.z; xb[nb][7] = hi.w;
      }
      const uint4 sc = s.sc[JB];
      auto sub_tile = [&](auto rc) {
        constexpr int R = decltype(rc)::value;
        uint32_t a[4][4];
        build_fragments<BITS, JB, WIDE>(s.code[R], lane_base, a);
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

  // One step: start loading the warp's next slab into `nxt`, ask L2 for the one after it, work
  // on the slab in `cur`, move on.  Returns false when the warp has no slab left.
  auto step = [&](const SlabRegs<BITS>& cur, SlabRegs<BITS>& nxt) {
    if (it >= c1) return false;
    if (rt != cur_rt) flush_until(rt);
    if (it + W < c1) load_slab<BITS>(nxt, wp + kStep, lane);
    if (it + 2 * W < c1) prefetch_slab_l2<BITS>(wp + 2 * (size_t)kStep, lane);
    compute(cur, ks);
    wp += kStep;
    it += W;
    ks += W;
    while (ks >= p.k_slabs) {
      ks -= p.k_slabs;
      ++rt;
    }
    return true;
  };
  // two register sets, used alternately
  while (step(s, s2) && step(s2, s)) {
  }
  flush_until(rt_last + 1);
  if (timed_out && lane == 0) atomicOr(p.counters + kStatusWord, kStatusTimeout);
}

// ---- host side ----------------------------------------------------------------------

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

// Plans the shared-memory layout of one CTA as offsets from the start of its dynamic shared
// memory, which kernels see at address `base` of the shared window:
//   [sync words] ... [table, at a multiple of 64 KB of the window when it is the wide one] ...
// with the reduction slots, the sums and (for the fused RMSNorm) all of x placed below the table
// where there is room, above it otherwise.  Sets how the kernel finds x (*xmode): resident in
// shared memory for the fused RMSNorm, read from L2 otherwise; -1 if a resident x does not fit.
// Returns the dynamic size needed.
template <int BITS, int NB>
size_t plan_smem(uint32_t base, int warps, size_t limit, bool need_resident, LinearParams& p, int* xmode) {
  constexpr bool WIDE = BITS != 3;
  using T = Table<BITS, WIDE>;
  const uint32_t tt = ((p.m < 8 ? p.m : 8) + 1) / 2;
  const uint32_t e_bytes = NB * kSubTiles * 32 * tt * sizeof(float);  // the sums of one row tile
  // large deposits (batches of five rows and more, or two n-tiles) are added up by the compute
  // warps themselves; small ones by the finisher, from two slot sets used in turn
  const bool team = tt >= 3 || NB == 2;
  const uint32_t xres_row = (uint32_t)p.k * 2 + kXRowPad;
  const uint32_t xres_bytes = align_up((uint32_t)p.m * xres_row, 128);
  p.team = team ? 1 : 0;
  p.slot_sets = 2;
  p.slot_t = tt;
  p.xres_row = xres_row;
  const uint32_t table_off = WIDE ? align_up(base + kSmemHead, 65536) - base : kSmemHead;
  p.table_off = table_off;

  // lays everything out for a number of deposit phases and an x mode; returns the size needed
  auto layout = [&](uint32_t phases, int mode) -> size_t {
    uint32_t low = kSmemHead, high = table_off + T::kBytes;  // cursors below and above the table
    auto place = [&](uint32_t bytes) {
      bytes = align_up(bytes, 128);
      if (low + bytes <= table_off) {
        const uint32_t at = low;
        low += bytes;
        return at;
      }
      const uint32_t at = high;
      high += bytes;
      return at;
    };
    p.slot_phases = phases;
    p.slots_off = place(team ? warps * e_bytes / phases : 2 * warps * e_bytes);
    p.tsum_off = team ? place(3 * e_bytes) : 0;  // two blocks of sums used in turn + the gather block of the push
    p.stash_off = place(e_bytes);
    p.xres_off = mode == kXResident ? place(xres_bytes) : 0;
    return high;
  };
  const int mode = need_resident ? kXResident : kXDirect;
  for (uint32_t phases = 1; phases <= (team ? 4u : 1u); phases *= 2) {
    const size_t need = layout(phases, mode);
    if (need <= limit) {
      *xmode = mode;
      return need;
    }
  }
  *xmode = -1;  // does not fit (the fused RMSNorm on too large an x)
  return layout(1, kXDirect);
}

// Sets the kernel's shared-memory limit once per device and launches it.
template <class Kernel, int BITS>
int launch_kernel(Kernel kernel, std::atomic<size_t> (&configured)[64], const LinearParams& p, const InlineLut<BITS>& inl,
                  int grid, int threads, size_t smem, unsigned flags, cudaStream_t stream) {
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  std::atomic<size_t>& have = configured[dev & 63];
  if (have.load(std::memory_order_acquire) < smem) {
    FDK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    have.store(smem, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
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

template <int BITS, int NB, int WARPS, bool FP16, int EPI, int XM, int NORM, bool TEAM>
int launch_team(const LinearParams& p, const InlineLut<BITS>& inl, int grid, size_t smem, unsigned flags,
                cudaStream_t stream) {
  static std::atomic<size_t> configured[64] = {};
  return launch_kernel(linear_lut_kernel<BITS, NB, WARPS, FP16, EPI, XM, NORM, TEAM>, configured, p, inl, grid,
                       (WARPS + 1) * 32, smem, flags, stream);
}

// Two n-tiles always run in team mode; one n-tile from five batch rows on.
template <int BITS, int NB, int WARPS, bool FP16, int EPI, int XM, int NORM>
int launch_instance(const LinearParams& p, const InlineLut<BITS>& inl, int grid, size_t smem, unsigned flags,
                    cudaStream_t stream) {
  if constexpr (NB == 1) {
    if (!p.team) return launch_team<BITS, NB, WARPS, FP16, EPI, XM, NORM, false>(p, inl, grid, smem, flags, stream);
  }
  return launch_team<BITS, NB, WARPS, FP16, EPI, XM, NORM, true>(p, inl, grid, smem, flags, stream);
}

template <int BITS, int NB, int WARPS, bool FP16>
int launch_width(LinearParams p, const InlineLut<BITS>& inl, int sm_count, unsigned flags, cudaStream_t stream) {
  uint32_t base = 0;
  if (int st = dynamic_smem_base(&base)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  const bool norm = p.norm_h != nullptr;
  int xm = kXDirect;
  const size_t smem = plan_smem<BITS, NB>(base, WARPS, (size_t)di.max_smem_optin, norm, p, &xm);
  FDK_CHECK_ARG(xm >= 0, FDK_ERR_SHAPE, "the fused RMSNorm needs x [%d, %d] to fit in shared memory", p.m, p.k);
  FDK_CHECK_ARG(smem <= (size_t)di.max_smem_optin, FDK_ERR_CUDA, "shared-memory plan of %zu bytes exceeds %d", smem,
                di.max_smem_optin);
  // one CTA per SM, fewer when there are fewer slabs than that
  int grid = sm_count;
  if (grid > p.total) grid = p.total;
  p.base = p.total / grid;
  p.rem = p.total % grid;

  const int epi = p.tp > 0 ? kEpiPush : p.silu ? kEpiSilu : p.resid_h != nullptr ? kEpiResid : p.rope_pos != nullptr ? kEpiRope : kEpiStore;
#define FDK_LAUNCH(EPI_, XM_, NORM_) \
  return launch_instance<BITS, NB, WARPS, FP16, EPI_, XM_, NORM_>(p, inl, grid, smem, flags, stream)
  if constexpr (!FP16) {  // the decode fusions exist for bf16 only
    if (norm) {
      if (epi == kEpiStore) FDK_LAUNCH(kEpiStore, kXResident, kNormInput);
      if (epi == kEpiSilu) FDK_LAUNCH(kEpiSilu, kXResident, kNormInput);
      if (epi == kEpiRope) FDK_LAUNCH(kEpiRope, kXResident, kNormInput);
      FDK_CHECK_ARG(false, FDK_ERR_BAD_ARG, "the fused RMSNorm goes with the plain, SiLU or rotary output only");
    }
    if (p.scale_ss != nullptr) {
      if (epi == kEpiStore) FDK_LAUNCH(kEpiStore, kXDirect, kNormOutput);
      if (epi == kEpiSilu) FDK_LAUNCH(kEpiSilu, kXDirect, kNormOutput);
      if (epi == kEpiRope) FDK_LAUNCH(kEpiRope, kXDirect, kNormOutput);
      if (epi == kEpiResid) FDK_LAUNCH(kEpiResid, kXDirect, kNormOutput);
      FDK_CHECK_ARG(false, FDK_ERR_BAD_ARG, "the deferred RMSNorm does not go with the tensor-parallel push");
    }
    if (epi == kEpiResid) FDK_LAUNCH(kEpiResid, kXDirect, kNormNone);
    if (epi == kEpiRope) FDK_LAUNCH(kEpiRope, kXDirect, kNormNone);
  } else {
    FDK_CHECK_ARG(!norm && p.scale_ss == nullptr && epi != kEpiResid && epi != kEpiRope, FDK_ERR_BAD_ARG,
                  "the decode fusions take bf16 only");
  }
  if (epi == kEpiPush) FDK_LAUNCH(kEpiPush, kXDirect, kNormNone);
  if (epi == kEpiSilu) FDK_LAUNCH(kEpiSilu, kXDirect, kNormNone);
  FDK_LAUNCH(kEpiStore, kXDirect, kNormNone);
#undef FDK_LAUNCH
}

template <int BITS, int NB, bool FP16>
int launch(LinearParams p, const void* lut_host, int sm_count, unsigned flags, cudaStream_t stream) {
  InlineLut<BITS> inl;
  if (lut_host != nullptr) {
    memcpy(inl.w, lut_host, sizeof(inl.w));
    p.lut = nullptr;
  } else {
    memset(inl.w, 0, sizeof(inl.w));
  }
  return launch_width<BITS, NB, kGemvWarps<NB>, FP16>(p, inl, sm_count, flags, stream);
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

// Whether the fused RMSNorm (all of x in shared memory) can take a batch of m rows of k columns.
template <int BITS>
int norm_fits_bits(int m, int k, int* fits) {
  uint32_t base = 0;
  if (int st = dynamic_smem_base(&base)) return st;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  LinearParams p{};
  p.m = m;
  p.k = k;
  int xm = -1;
  if (m > 8) {
    plan_smem<BITS, 2>(base, kGemvWarps<2>, (size_t)di.max_smem_optin, true, p, &xm);
  } else {
    plan_smem<BITS, 1>(base, kGemvWarps<1>, (size_t)di.max_smem_optin, true, p, &xm);
  }
  *fits = xm >= 0 ? 1 : 0;
  return FDK_OK;
}

}  // namespace fdk
