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
  uint32_t slot_sets;     // slot sets used in turn by consecutive row tiles: 2, or 1 where they are large
  uint32_t xres_off;      // all of x staged once per CTA at this offset (kernels instantiated with XRES)
  uint32_t xres_row;      // bytes between its rows
  uint32_t stash_off;     // E floats: the other CTAs' sums of a split row tile, fetched ahead by the finisher
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

}  // namespace fdk
