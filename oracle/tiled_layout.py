"""Host model (numpy) of libfdk_b200's tiled weight layout.  TEST INFRASTRUCTURE ONLY.

The tiled layout is this library's own (the reference's kernels read the packed
tensors of src/fdk/models.py:94-104 as they are), so there is nothing in the
reference to pin it against; tests pin the CUDA repacker against this
independent restatement of the layout rules instead, byte for byte.

Layout rules (see csrc/fdk_layout.cuh for the rationale):
  slab        = 64 rows x (64 * KSB) columns, slabs stored row-tile major
  KSB         = 4 for 1 and 3 bits, 2 for 2 bits, 1 for 4 and 8 bits
  slab codes  = [r 0..3][v 0..V-1][lane 0..31][16 B]
  slab scales = [jb 0..KSB-1][g 0..7][r 0..3][half 0..1] 16-bit
  lane bytes  = for each 64-block jb: the 2*bits bytes of row 16r+g holding block
                elements [16t, 16t+16) (lane = 4g + t), then those of row 16r+g+8
  3 bits      = each 6-byte group re-encoded as a little-endian 48-bit integer whose
                bits [6p, 6p+6) are (code[2p] << 3) | code[2p+1]
"""

from __future__ import annotations

import numpy as np


def dims(n: int, k: int, bits: int) -> dict:
    ksb = 4 if bits in (1, 3) else (2 if bits == 2 else 1)
    lane_bytes = ksb * 4 * bits
    v = lane_bytes // 16
    return dict(
        ksb=ksb,
        v=v,
        slab_bytes=4 * v * 512 + ksb * 128,
        code_bytes=4 * v * 512,
        row_tiles=-(-n // 64),
        k_slabs=-(-k // (64 * ksb)),
    )


def tiled_size(n: int, k: int, bits: int) -> int:
    d = dims(n, k, bits)
    return d["row_tiles"] * d["k_slabs"] * d["slab_bytes"]


def _encode3(group6: np.ndarray) -> np.ndarray:
    """[..., 6] uint8 (MSB-first stream of 16 3-bit codes) -> [..., 6] uint8 re-encoded."""
    g = group6.astype(np.uint64)
    be = np.zeros(g.shape[:-1], dtype=np.uint64)
    for i in range(6):
        be = (be << np.uint64(8)) | g[..., i]
    out = np.zeros_like(be)
    for p in range(8):
        pair = (be >> np.uint64(42 - 6 * p)) & np.uint64(0x3F)
        out |= pair << np.uint64(6 * p)
    res = np.zeros(group6.shape, dtype=np.uint8)
    for i in range(6):
        res[..., i] = ((out >> np.uint64(8 * i)) & np.uint64(0xFF)).astype(np.uint8)
    return res


def repack(codes: np.ndarray, scale_bits: np.ndarray, bits: int) -> np.ndarray:
    """codes [N, K*bits/8] uint8, scale [N, K/g] uint16 (g a multiple of 64) -> tiled uint8."""
    codes = np.asarray(codes, dtype=np.uint8)
    scale_bits = np.asarray(scale_bits, dtype=np.uint16)
    n = codes.shape[0]
    k = codes.shape[1] * 8 // bits
    g_size = k // scale_bits.shape[1]
    assert g_size % 64 == 0 and k % 64 == 0
    d = dims(n, k, bits)
    out = np.zeros(tiled_size(n, k, bits), dtype=np.uint8)
    cb = 2 * bits
    blocks = k // 64

    src = codes.reshape(n, blocks, 4, cb)  # [row, block, t, byte]
    if bits == 3:
        src = _encode3(src)
    row = np.arange(n)[:, None, None, None]
    blk = np.arange(blocks)[None, :, None, None]
    t = np.arange(4)[None, None, :, None]
    ib = np.arange(cb)[None, None, None, :]
    rt, r, g, half = row >> 6, (row >> 4) & 3, row & 7, (row & 15) >> 3
    ks, jb = blk // d["ksb"], blk % d["ksb"]
    lane = 4 * g + t
    q = jb * 2 * cb + half * cb + ib
    v, qq = q >> 4, q & 15
    off = (rt * d["k_slabs"] + ks) * d["slab_bytes"] + ((r * d["v"] + v) * 32 + lane) * 16 + qq
    out[np.broadcast_to(off, src.shape).ravel()] = src.ravel()

    sc = np.repeat(scale_bits, g_size // 64, axis=1)  # one per 64-block
    row2 = np.arange(n)[:, None]
    blk2 = np.arange(blocks)[None, :]
    rt, r, g, half = row2 >> 6, (row2 >> 4) & 3, row2 & 7, (row2 & 15) >> 3
    ks, jb = blk2 // d["ksb"], blk2 % d["ksb"]
    soff = (rt * d["k_slabs"] + ks) * d["slab_bytes"] + d["code_bytes"] + jb * 128 + g * 16 + r * 4 + half * 2
    soff = np.broadcast_to(soff, sc.shape).ravel()
    out[soff] = (sc.ravel() & 0xFF).astype(np.uint8)
    out[soff + 1] = (sc.ravel() >> 8).astype(np.uint8)
    return out
