// Tile layout of the repacked ("tiled") weight buffer, shared by the repacker,
// the dequantiser and the fused GEMV / skinny-GEMM kernels.
//
// Source format (the reference's, src/fdk/models.py:94-104): codes row-major
// [N, K*bits/8] uint8 with element 0 of a byte in the high bits, one 16-bit
// scale per (row, 64-run of K), a per-byte value table [256, 8/bits].
//
// Tiled format: the matrix is cut into SLABS of 64 rows x (64*KSB) columns,
// stored row-tile major ([ceil(N/64)][ceil(K/(64*KSB))] slabs).  One slab is
// what one warp consumes per pipeline step, as V+... 16-byte vector loads per
// lane that are contiguous across the warp (512 B per load instruction):
//
//   codes   [r = 0..3][v = 0..V-1][lane = 0..31][16 bytes]
//   scales  [jb = 0..KSB-1][g = 0..7][r = 0..3][half = 0..1]  16-bit each
//
// r is a 16-row sub-tile (one m16n8k16 A operand), lane = 4*g + t with g the
// fragment row (rows 16r+g and 16r+g+8) and t the fragment column group.
// The V*16 bytes of a lane are, for each 64-block jb of the slab, the 2*bits
// bytes of row 16r+g that hold block elements [16t, 16t+16), followed by the
// same bytes of row 16r+g+8.  Bytes keep their source order, so the per-byte
// value table of the source format still applies to every byte of the tiled
// buffer.  (3-bit codes, which have no byte table, are re-encoded: see
// Layout<3>.)  Rows >= N and blocks >= K/64 are stored as code 0 / scale 0.
#pragma once
#include <cstddef>
#include <cstdint>

namespace fdk {

constexpr int kBlock = 64;      // elements per scale block (the tiled format always has one scale per 64)
constexpr int kTileRows = 64;   // rows per slab
constexpr int kSubTiles = 4;    // 16-row sub-tiles per slab

template <int BITS>
struct Layout {
  static_assert(BITS == 1 || BITS == 2 || BITS == 3 || BITS == 4 || BITS == 8, "unsupported bit width");
  // 64-blocks per slab, chosen so that a lane's share is a whole number of 16-byte vectors
  static constexpr int KSB = (BITS == 1 || BITS == 3) ? 4 : (BITS == 2 ? 2 : 1);
  static constexpr int kRowChunk = 2 * BITS;              // bytes holding 16 elements of one row
  static constexpr int kLaneBytes = KSB * 2 * kRowChunk;  // per lane, per sub-tile, per slab
  static constexpr int V = kLaneBytes / 16;
  static_assert(kLaneBytes % 16 == 0, "lane share must be whole 16-byte vectors");
  static constexpr int kCodeBytes = kSubTiles * V * 512;
  static constexpr int kScaleBytes = KSB * 128;
  static constexpr int kSlabBytes = kCodeBytes + kScaleBytes;
  static constexpr int kSlabK = KSB * kBlock;             // columns covered by one slab
};

struct TiledDims {
  int row_tiles;   // ceil(N / 64)
  int k_slabs;     // ceil(K / slab columns)
  int slab_bytes;
  int ksb;
  int v;
};

inline __host__ __device__ TiledDims tiled_dims(int n, int k, int bits) {
  TiledDims d{};
  int ksb = (bits == 1 || bits == 3) ? 4 : (bits == 2 ? 2 : 1);
  int lane_bytes = ksb * 4 * bits;
  d.ksb = ksb;
  d.v = lane_bytes / 16;
  d.slab_bytes = kSubTiles * d.v * 512 + ksb * 128;
  d.row_tiles = (n + kTileRows - 1) / kTileRows;
  d.k_slabs = (k + ksb * kBlock - 1) / (ksb * kBlock);
  return d;
}

inline __host__ __device__ size_t tiled_bytes(int n, int k, int bits) {
  TiledDims d = tiled_dims(n, k, bits);
  return (size_t)d.row_tiles * d.k_slabs * d.slab_bytes;
}

// Byte offset, inside the tiled buffer, of byte `i` (0 <= i < 8*bits) of the
// 64-block `blk` of row `n`.  Valid for the byte-preserving widths 1/2/4/8.
inline __host__ __device__ size_t tiled_code_offset(int n, int blk, int i, int bits, const TiledDims& d) {
  int rt = n >> 6, r = (n >> 4) & 3, rr = n & 15, g = rr & 7, half = rr >> 3;
  int ks = blk / d.ksb, jb = blk % d.ksb;
  int cb = 2 * bits;
  int t = i / cb, ib = i % cb;
  int lane = 4 * g + t;
  int q = jb * 2 * cb + half * cb + ib;
  int v = q >> 4, qq = q & 15;
  size_t slab = ((size_t)rt * d.k_slabs + ks) * d.slab_bytes;
  return slab + (size_t)(((r * d.v + v) * 32 + lane) * 16 + qq);
}

// Byte offset of the 16-bit scale of (row n, 64-block blk).
inline __host__ __device__ size_t tiled_scale_offset(int n, int blk, const TiledDims& d) {
  int rt = n >> 6, r = (n >> 4) & 3, rr = n & 15, g = rr & 7, half = rr >> 3;
  int ks = blk / d.ksb, jb = blk % d.ksb;
  size_t slab = ((size_t)rt * d.k_slabs + ks) * d.slab_bytes;
  return slab + (size_t)(kSubTiles * d.v * 512) + (size_t)(jb * 128 + g * 16 + r * 4 + half * 2);
}

}  // namespace fdk
