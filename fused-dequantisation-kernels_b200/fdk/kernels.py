"""Operator API of the LUT hot path -- same names, argument meaning and assertions as the
reference's src/fdk/kernels.py, backed by libfdk_b200.so instead of Triton.

  run_mv_lut(a, b, lut, bs, out)   fused dequantise + GEMV        (kernels.py:158-182)
  run_mm_lut(a, b, lut, bs, out)   fused dequantise + GEMM        (kernels.py:460-489)
  mm_lut_ref(a, bq, lut8, bs)      torch "dequantise then matmul"  (kernels.py:19-25)
  run_mv / run_mm                  plain bf16 products: cuBLAS baselines here
  dequantise(b, lut, bs)           bit-exact dense W (first two lines of mm_lut_ref)

The reference's operators read the packed tensors directly.  The native kernels read a
tiled copy of them; for callers that pass packed tensors it is built on first use and
cached per tensor object and version (modules hold their tiled buffer themselves).
"""

from __future__ import annotations

import weakref

import torch
from torch import Tensor

from . import native


def _assert_rmsen(expected: Tensor, actual: Tensor, tol: float) -> None:
    assert expected.shape == actual.shape
    expected_sse = expected.float().pow(2).sum()
    rmsen = (actual - expected).float().pow(2).sum().div(expected_sse).sqrt()
    assert rmsen < tol, f"rmsen={rmsen}"


def bits_of_lut(lut: Tensor) -> int:
    """Bit width from the table shape: [256, E] -> 8 // E; the 3-bit extension carries
    its plain [8, 1] codebook."""
    if lut.shape[0] == 8:
        return 3
    return 8 // lut.shape[1]


### torch reference (runs wherever its tensors live; the reference wraps it in torch.compile)


def mm_lut_ref(a: Tensor, bq: Tensor, lut8: Tensor, bs: Tensor, out: Tensor | None = None) -> Tensor:
    bv = lut8[bq.long()].flatten(start_dim=1)
    b = bv.view(*bs.shape, -1).mul(bs[:, :, None]).flatten(start_dim=1)
    return torch.matmul(a, b.T, out=out)


### tiled-buffer cache for the operator-level API
# Keyed on the weight tensor OBJECT (id, checked against a weak reference, which also evicts the
# entry when the tensor is collected) and on the versions of both tensors: a new tensor that the
# allocator happens to place at the address of a freed one is never mistaken for it.

_tiled_cache: dict[int, tuple] = {}


def clear_tiled_cache() -> None:
    _tiled_cache.clear()


def tiled_for(b: Tensor, bs: Tensor, n: int, k: int, bits: int) -> Tensor:
    key = id(b)
    stamp = (b._version, id(bs), bs._version, n, k, bits)
    hit = _tiled_cache.get(key)
    if hit is not None and hit[0]() is b and hit[1]() is bs and hit[2] == stamp:
        return hit[3]
    tiled = native.repack(b, bs, n, k, bits, k // bs.shape[1])
    _tiled_cache[key] = (weakref.ref(b, lambda _, k_=key: _tiled_cache.pop(k_, None)), weakref.ref(bs), stamp, tiled)
    return tiled


### native operators

# Programmatic dependent launch for the two operators below: the kernel may be scheduled while
# the previous kernel of the stream is still running, reads its weights and its table right
# away and waits for that kernel only before it reads x or writes out.  Off by default: it is
# for callers whose weights do not change between launches (a decode loop, a benchmark).
programmatic_launch = False



def run_mv_lut(a: Tensor, b: Tensor, lut: Tensor, bs: Tensor, out: Tensor) -> None:
    # shape inference
    (k,) = a.shape
    (n,) = out.shape
    bits = bits_of_lut(lut)
    group_size = k // bs.shape[1]
    # assertions (as the reference's, kernels.py:165-170)
    assert a.dtype == lut.dtype == bs.dtype == out.dtype
    assert b.dtype == torch.uint8
    assert b.shape == (n, k * bits // 8)
    assert bs.shape == (n, k // group_size)
    assert lut.shape == ((8, 1) if bits == 3 else (256, 8 // bits))
    assert all([t.is_contiguous() for t in [a, b, lut, bs, out]])
    native.linear_lut(a[None], tiled_for(b, bs, n, k, bits), lut, out[None], n, k, bits, pdl=programmatic_launch)


def run_mm_lut(a: Tensor, b: Tensor, lut: Tensor, bs: Tensor, out: Tensor) -> None:
    # shape inference
    m, k = a.shape
    _, n = out.shape
    bits = bits_of_lut(lut)
    group_size = k // bs.shape[1]
    # assertions (as the reference's, kernels.py:467-473)
    assert a.dtype == lut.dtype == bs.dtype == out.dtype
    assert b.dtype == torch.uint8
    assert b.shape == (n, k * bits // 8)
    assert bs.shape == (n, k // group_size)
    assert lut.shape == ((8, 1) if bits == 3 else (256, 8 // bits))
    assert out.shape == (m, n)
    assert all([t.is_contiguous() for t in [a, b, lut, out]])
    native.linear_lut(a, tiled_for(b, bs, n, k, bits), lut, out, n, k, bits, pdl=programmatic_launch)


def dequantise(b: Tensor, lut: Tensor, bs: Tensor) -> Tensor:
    """Dense W [n, k], bit-identical to the torch reference's intermediate."""
    return native.dequantise(b, lut, bs, bits_of_lut(lut))


### 16-bit baselines (the reference has Triton kernels here; cuBLAS is the bar on B200)


def run_mv(a: Tensor, b: Tensor, out: Tensor) -> None:
    n, k = b.shape
    assert a.shape == (k,)
    assert out.shape == (n,)
    torch.matmul(a[None], b.T, out=out[None])


def run_mm(a: Tensor, b: Tensor, out: Tensor) -> None:
    m, k = a.shape
    n, _ = b.shape
    assert b.shape == (n, k)
    assert out.shape == (m, n)
    assert a.dtype == b.dtype == out.dtype
    assert all([t.is_contiguous() for t in [a, b, out]])
    torch.matmul(a, b.T, out=out)
