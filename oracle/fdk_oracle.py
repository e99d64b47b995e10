"""CPU oracle for the fused-dequantisation hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain numpy (integer / byte work, bit-level bf16
arithmetic) and eager CPU torch (the quantiser, which is torch arithmetic in
the reference too), the algorithm of the reference project
graphcore-research/fused-dequantisation-kernels for:

  * the packed weight format and the quantiser    src/fdk/models.py:63-104
  * the torch "dequantise then matmul" reference  src/fdk/kernels.py:19-25
  * the relative-RMS error measure                 src/fdk/kernels.py:9-13
  * the byte / op accounting                       src/fdk/models.py:283-310,
                                                   src/fdk/bench.py:224-231,298-307

Only tests, the smoke check and the benchmark's CPU-baseline leg may import it.
The shipped package never does; its CUDA path fails loudly when the native
library is missing instead of falling back to anything in here.

Parity status: PINNED for bits 1/2/4/8 -- tests/golden/ holds vectors made by
importing the reference itself (tests/golden/make_golden.py) and
tests/test_oracle.py checks every function below against them bit-for-bit.
The 3-bit format has no counterpart in the reference (8 % 3 != 0 there), so
for 3 bits parity is unpinned: it is defined here at the index level only.

bf16 values travel as numpy uint16 bit patterns so that "bit-exact" is a plain
integer comparison.
"""

from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------
# bf16 <-> fp32 at the bit level
# --------------------------------------------------------------------------


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 values (exact)."""
    bits = np.asarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round-to-nearest-even (what torch's
    float->bfloat16 conversion does; NaN is kept quiet)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    r = ((u + bias) >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, np.uint16(0x7FC0), r)
    return r


def f16_to_f32(bits: np.ndarray) -> np.ndarray:
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


# --------------------------------------------------------------------------
# format helpers
# --------------------------------------------------------------------------

SUPPORTED_BITS = (1, 2, 3, 4, 8)


def elements_per_byte(bits: int) -> int:
    """E in the reference (models.py:68).  Not defined for 3 bits."""
    assert bits in (1, 2, 4, 8)
    return 8 // bits


def packed_row_bytes(k: int, bits: int) -> int:
    assert (k * bits) % 8 == 0
    return k * bits // 8


def unpack_indices(weight_data: np.ndarray, bits: int, k: int) -> np.ndarray:
    """[N, K*bits/8] uint8 -> [N, K] code indices.

    Element 0 of every byte sits in the HIGH bits (models.py:94-102: the
    multipliers are 2**arange(0, 8, bits) flipped).  For 3 bits (an extension)
    the row is one MSB-first bit stream, element j at stream bits [3j, 3j+3).
    """
    wd = np.asarray(weight_data, dtype=np.uint8)
    n = wd.shape[0]
    assert wd.shape[1] == packed_row_bytes(k, bits)
    stream = np.unpackbits(wd, axis=1, bitorder="big")  # [N, K*bits], MSB first
    fields = stream.reshape(n, k, bits).astype(np.uint16)
    weights = (1 << np.arange(bits - 1, -1, -1)).astype(np.uint16)
    return (fields * weights).sum(axis=2).astype(np.uint8)


def pack_indices(idx: np.ndarray, bits: int) -> np.ndarray:
    """Inverse of unpack_indices: [N, K] codes -> [N, K*bits/8] uint8."""
    idx = np.asarray(idx, dtype=np.uint8)
    n, k = idx.shape
    shifts = np.arange(bits - 1, -1, -1).astype(np.uint8)
    stream = ((idx[:, :, None] >> shifts) & 1).astype(np.uint8).reshape(n, k * bits)
    return np.packbits(stream, axis=1, bitorder="big")


def byte_lut(base_lut_bits: np.ndarray, bits: int) -> np.ndarray:
    """[2^bits] bf16 -> [256, E] byte table = cartesian_prod(lut x E)
    (models.py:103): row b holds the E values byte b decodes to, first
    element (high bits) first."""
    e = elements_per_byte(bits)
    base = np.asarray(base_lut_bits, dtype=np.uint16)
    assert base.shape == (1 << bits,)
    b = np.arange(256, dtype=np.uint16)
    cols = []
    for j in range(e):
        shift = (e - 1 - j) * bits
        cols.append(base[(b >> shift) & ((1 << bits) - 1)])
    return np.stack(cols, axis=1)


def base_lut_from_byte_lut(lut8_bits: np.ndarray) -> np.ndarray:
    """Recover the 2^bits codebook: it is the last column of the first 2^bits
    rows of the byte table."""
    lut8 = np.asarray(lut8_bits, dtype=np.uint16)
    bits = 8 // lut8.shape[1]
    return lut8[: 1 << bits, -1].copy()


# --------------------------------------------------------------------------
# the reference operator: dequantise, then matmul   (kernels.py:19-25)
# --------------------------------------------------------------------------


def dequantise(
    weight_data: np.ndarray,
    lut8_bits: np.ndarray,
    scale_bits: np.ndarray,
    dtype: str = "bf16",
) -> np.ndarray:
    """W[n, k] = dtype( float(lut8[byte][j]) * float(scale[n, k // g]) ).

    This is `lut8[bq.long()].flatten(1).view(n, k/g, g).mul(bs[:, :, None])`
    of the reference: one multiply in the storage dtype, i.e. the exact fp32
    product rounded once.  Returns bit patterns [N, K] uint16.
    """
    wd = np.asarray(weight_data, dtype=np.uint8)
    lut8 = np.asarray(lut8_bits, dtype=np.uint16)
    sc = np.asarray(scale_bits, dtype=np.uint16)
    n = wd.shape[0]
    e = lut8.shape[1]
    k = wd.shape[1] * e
    groups = sc.shape[1]
    assert sc.shape[0] == n and k % groups == 0
    to_f32, from_f32 = (bf16_to_f32, f32_to_bf16) if dtype == "bf16" else (f16_to_f32, f32_to_f16)
    vals = to_f32(lut8[wd.astype(np.int64)].reshape(n, k))  # gather
    g = k // groups
    prod = vals.reshape(n, groups, g) * to_f32(sc)[:, :, None]
    return from_f32(prod.reshape(n, k))


def dequantise_indices(
    idx: np.ndarray, base_lut_bits: np.ndarray, scale_bits: np.ndarray, dtype: str = "bf16"
) -> np.ndarray:
    """Index-level form of `dequantise` (needed for 3 bits, where no byte
    table exists): W = dtype(base_lut[idx] * scale)."""
    idx = np.asarray(idx)
    n, k = idx.shape
    sc = np.asarray(scale_bits, dtype=np.uint16)
    groups = sc.shape[1]
    to_f32, from_f32 = (bf16_to_f32, f32_to_bf16) if dtype == "bf16" else (f16_to_f32, f32_to_f16)
    vals = to_f32(np.asarray(base_lut_bits, dtype=np.uint16)[idx.astype(np.int64)])
    prod = vals.reshape(n, groups, k // groups) * to_f32(sc)[:, :, None]
    return from_f32(prod.reshape(n, k))


def mm_lut(
    x_bits: np.ndarray,
    weight_data: np.ndarray,
    lut8_bits: np.ndarray,
    scale_bits: np.ndarray,
    dtype: str = "bf16",
) -> np.ndarray:
    """y = x @ W.T with W from `dequantise`; products of storage-dtype values
    accumulated in fp32 (float64 here, which only tightens it) and rounded once
    to the storage dtype.  x: [m, K] or [K].  Returns bit patterns."""
    to_f32, from_f32 = (bf16_to_f32, f32_to_bf16) if dtype == "bf16" else (f16_to_f32, f32_to_f16)
    w = to_f32(dequantise(weight_data, lut8_bits, scale_bits, dtype)).astype(np.float64)
    x = to_f32(np.asarray(x_bits, dtype=np.uint16)).astype(np.float64)
    y = x @ w.T
    return from_f32(y.astype(np.float32))


def mm_dense(x_bits: np.ndarray, w_bits: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """y = x @ W.T for an already dequantised W (bit patterns in, bit patterns out)."""
    to_f32, from_f32 = (bf16_to_f32, f32_to_bf16) if dtype == "bf16" else (f16_to_f32, f32_to_f16)
    x = to_f32(np.asarray(x_bits, dtype=np.uint16)).astype(np.float64)
    w = to_f32(np.asarray(w_bits, dtype=np.uint16)).astype(np.float64)
    return from_f32((x @ w.T).astype(np.float32))


def rmsen(expected: np.ndarray, actual: np.ndarray) -> float:
    """sqrt(sum((a-e)^2) / sum(e^2)) on float values (kernels.py:9-13)."""
    e = np.asarray(expected, dtype=np.float64)
    a = np.asarray(actual, dtype=np.float64)
    assert e.shape == a.shape
    return float(np.sqrt(((a - e) ** 2).sum() / (e**2).sum()))


# --------------------------------------------------------------------------
# accounting   (bench.py:224-231, 298-307; models.py:283-310)
# --------------------------------------------------------------------------


def bench_bytes_rw(m: int, k: int, n: int, g: int, bits: int, itemsize: int = 2) -> int:
    return n * (k * bits) // 8 + (m * k + n * (k // g) + m * n) * itemsize


def bench_ops(m: int, k: int, n: int) -> int:
    return 2 * m * k * n


def packed_weight_bytes(n: int, k: int, bits: int, g: int = 64, itemsize: int = 2) -> int:
    """Codes + block scales of one quantised matrix: the "packed-weight bytes"
    that the GEMV bandwidth figure is quoted on."""
    return n * k * bits // 8 + n * (k // g) * itemsize
