// Launch parameters of the fused GEMV kernel and the entry into its per-width instantiations
// (linear_lut_bits*.cu), shared with the C entry points (linear_lut.cu).
#pragma once
#include "fdk_common.cuh"
#include "lut_table.cuh"

namespace fdk {

constexpr int kMaxStages = 4;

constexpr int kStatusTimeout = 1;        // a bounded wait on a copy barrier ran out
constexpr int kStatusSmemLayout = 2;     // shared window base differs from what the host planned for

struct LinearParams {
  const uint8_t* tiled;
  const void* lut;  // byte table in device memory, or null when it travels in the parameters
  const uint16_t* x;
  uint16_t* out;
  uint2* partial;  // [grid][512 * NB] {partial sum, tag} words
  int* counters;   // [row_tiles] use counts of the split row tiles + status word
  int m, n, k;
  int k_slabs;     // slabs per row tile
  int total;       // row_tiles * k_slabs
  int base, rem;   // CTA c owns `base + (c < rem)` consecutive slabs
  // shared-memory plan, as addresses in the shared window
  uint32_t smem_base;     // expected address of the dynamic shared memory
  uint32_t table_addr;
  uint32_t slots_addr;
  uint32_t mbar_addr;
  uint32_t stage_a_addr;  // first stages live below the table ...
  uint32_t stage_a_count;
  uint32_t stage_b_addr;  // ... the others above it
  uint32_t stage_bytes;   // slab + this launch's x rows, rounded to 128
  uint32_t stages;        // ring stages per warp
  uint32_t slot_t;        // fragment column pairs kept per row in the reduction slots: ceil(min(m, 8) / 2)
  uint32_t slot_sets;     // slot sets used in turn by consecutive row tiles: 2, or 1 where they are large
  uint32_t xres_addr;     // all of x staged once per CTA at this address (0: x rows come with each slab)
  uint32_t xres_row;      // bytes between its rows
  uint32_t xres_bar;      // barrier of that one copy
  // tensor-parallel push (tp > 0): outputs go to every rank's exchange buffer instead of `out`
  int silu;  // rows come as 32 gate + 32 up per tile; write silu(gate) * up, [m, n / 2]
  int tp, rank;
  uint2* peer_stage[8];     // staging words {two 16-bit outputs, tag} [2][tp][slot / 2] of each rank, as mapped here
  const uint32_t* seq;      // local count of reduces done so far = number of this push
  long long stage_slot;     // elements of one (half, rank) slot
#ifdef FDK_TRACE
  unsigned long long* trace;  // [grid][warps][8] cycle counts (development builds only)
#endif
};

// Plans shared memory, picks the CTA shape and launches; one explicit instantiation per code
// width, each in a translation unit of its own so that they compile in parallel.
template <int BITS>
int launch_bits(const LinearParams& p, const void* lut_host, int grid, int dtype, unsigned flags, cudaStream_t stream);

}  // namespace fdk
