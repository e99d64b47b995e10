// Launch parameters of the fused GEMV kernel and the entry into its per-width instantiations
// (linear_lut_bits*.cu), shared with the C entry points (linear_lut.cu).
#pragma once
#include "fdk_common.cuh"
#include "lut_table.cuh"

namespace fdk {

constexpr int kStatusTimeout = 1;        // a bounded wait ran out
constexpr int kStatusSmemLayout = 2;     // (tensor-core GEMM) shared window base differs from the host's plan

struct LinearParams {
  const uint8_t* tiled;
  const void* lut;  // byte table in device memory, or null when it travels in the parameters
  const uint16_t* x;
  uint16_t* out;
  uint2* partial;  // [grid][512 * NB] {partial sum, tag} words
  int* counters;   // [row_tiles] use counts of the split row tiles + status word
  int m, n, k;
  int k_slabs;     // slabs per row tile
  uint32_t k_magic;  // ceil(2^32 / k_slabs): n / k_slabs == umulhi(n, k_magic) while n * k_slabs < 2^32
  int total;       // row_tiles * k_slabs
  int base, rem;   // CTA c owns `base + (c < rem)` consecutive slabs
  // shared-memory plan, as byte offsets from the start of the dynamic shared memory
  uint32_t table_off;
  uint32_t slots_off;
  uint32_t slot_t;        // fragment column pairs kept per row in the reduction slots: ceil(min(m, 8) / 2)
  uint32_t slot_sets;     // blocks of sums (slot sets, or the team's sums) used in turn by consecutive row tiles
  uint32_t team;          // 1: the compute warps add their deposits themselves into tsum, the finisher starts there
  uint32_t slot_phases;   // team mode: the deposits of a tile are made and added in this many parts (1, 2, 4)
  uint32_t tsum_off;      // team mode: [2][E] sums used in turn + [E] gather block of the tensor-parallel push
  uint32_t xres_off;      // all of x staged once per CTA at this offset (resident x)
  uint32_t xres_row;      // bytes between its rows
  uint32_t stash_off;     // E floats: the other CTAs' sums of a split row tile, fetched ahead by the finisher
  // input side of the decode fusion (norm_h != null): x = norm_w * bf16(h * rsqrt(mean(h^2) + eps)),
  // computed while x is staged; mean(h^2) of row b = sum of norm_ss[b][0 .. norm_tiles) / k
  const uint16_t* norm_h;   // [m, k]
  const uint16_t* norm_w;   // [k]
  const float* norm_ss;     // [m, norm_tiles]
  int norm_tiles;
  float norm_eps;
  // output side of the decode fusion, one of:
  // residual (resid_h != null): h[m, n] += bf16(y) in place, resid_ss[b][row tile] = sum of the squares of
  // the new h over the tile's 64 rows
  uint16_t* resid_h;
  float* resid_ss;          // [m, ceil(n / 64)]
  // deferred RMSNorm, producer side (with the residual output): resid_x[m, n] = bf16(resid_w[row] * h)
  const uint16_t* resid_w;  // [n] or null
  uint16_t* resid_x;
  // deferred RMSNorm, consumer side: the complete sums of batch row b are multiplied by
  // rsqrt(sum of scale_ss[b][0 .. scale_tiles) / k + scale_eps) before they are rounded
  const float* scale_ss;    // [m, scale_tiles] or null
  int scale_tiles;
  float scale_eps;
  // rotary (rope_pos != null): the rows are the fused q|k|v projection with every q and k head's rows
  // ordered [0..31, 64..95, 32..63, 96..127]; q is rotated into q_out, k rotated and v copied into the
  // caches at *rope_pos (nothing is written for a position outside [0, max_len))
  const long long* rope_pos;
  const uint32_t* rope_table;  // [64] {bf16 cos, bf16 sin} of the position's 64 angles
  uint16_t* q_out;
  uint16_t* k_cache;
  uint16_t* v_cache;
  int q_heads, kv_heads, max_len;
  // tensor-parallel push (tp > 0): outputs go to every rank's exchange buffer instead of `out`
  int silu;  // rows come as 32 gate + 32 up per tile; write silu(gate) * up, [m, n / 2]
  int tp, rank;
  uint2* peer_stage[8];     // staging words {two 16-bit outputs, tag} [2][tp][slot / 2] of each rank, as mapped here
  const uint32_t* seq;      // local count of reduces done so far = number of this push
  long long stage_slot;     // elements of one (half, rank) slot
};

// Plans shared memory and launches; one explicit instantiation per code width, each in a
// translation unit of its own so that they compile in parallel.
template <int BITS>
int launch_bits(const LinearParams& p, const void* lut_host, int grid, int dtype, unsigned flags, cudaStream_t stream);

// Whether the kernel's fused RMSNorm, which needs all of x in shared memory, can take x [m, k].
template <int BITS>
int norm_fits_bits(int m, int k, int* fits);

}  // namespace fdk
