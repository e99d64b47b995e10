"""Eager CPU-torch half of the oracle.  TEST INFRASTRUCTURE ONLY (see
fdk_oracle.py for who may import it).

The reference's quantiser and its "torch reference" operator are themselves
sequences of torch ops evaluated in bf16, so the faithful CPU restatement of
those two is eager torch on CPU tensors:

  * quantise_weight  follows QuantisedLinear.create   src/fdk/models.py:63-104
  * mm_lut_ref       follows kernels.mm_lut_ref        src/fdk/kernels.py:19-25
                     (without the torch.compile decorator: the paper notebook
                     does the same with torch.compiler.disable)

Both are pinned against vectors produced by the reference (tests/golden/).
mm_lut_ref is also the timed CPU baseline ("port") of the benchmark.
"""

from __future__ import annotations

import torch
from torch import Tensor


def quantise_weight(
    weight: Tensor, bits: int, block_size: int, lut: Tensor | None = None
) -> tuple[Tensor, Tensor, Tensor]:
    """weight [N, K] -> (weight_data uint8 [N, K*bits/8], scale [N, K/g],
    byte table [256, 8/bits]) in weight's dtype.

    Steps, as in the reference: per-block scale (abs-mean when bits <= 2,
    abs-max otherwise, floored at 1e-12); nearest-codebook index found by
    bucketising w/scale at the codebook midpoints; indices packed E per byte,
    first element in the high bits; codebook expanded to a per-byte table.
    For bits == 3 (no reference counterpart) the indices are packed as one
    MSB-first bit stream per row and the returned table is the plain
    [8, 1] codebook.
    """
    n_codes = 1 << bits
    if lut is None:
        lut = torch.linspace(-1, 1, steps=n_codes, device=weight.device, dtype=weight.dtype)
    else:
        assert lut.ndim == 1 and lut.shape[0] <= n_codes
        lut = torch.nn.functional.pad(lut, (0, n_codes - lut.shape[0]), value=lut[-1])

    blocks = weight.unflatten(-1, (-1, block_size))
    if bits <= 2:
        scale = blocks.abs().mean(dim=-1)
    else:
        scale = blocks.abs().amax(dim=-1)
    scale.clamp_min_(1e-12)
    scaled = (blocks / scale[..., None]).flatten(-2)

    boundaries = (lut[1:] + lut[:-1]) / 2
    idx = torch.bucketize(scaled, boundaries).clamp_(0, n_codes - 1)

    if bits == 3:
        import numpy as np

        from fdk_oracle import pack_indices

        data = torch.from_numpy(pack_indices(idx.to(torch.uint8).numpy(), 3))
        return data, scale, lut.reshape(n_codes, 1)

    per_byte = 8 // bits
    place = 2 ** torch.arange(0, 8, bits, device=weight.device, dtype=torch.uint8).flip(0)
    data = (
        idx.to(torch.uint8).unflatten(-1, (-1, per_byte)).mul(place).sum(-1, dtype=torch.uint8)
    )
    table = torch.cartesian_prod(*([lut] * per_byte)).view(256, -1)
    return data, scale, table


def dequantise_ref(bq: Tensor, lut8: Tensor, bs: Tensor) -> Tensor:
    """Dense W [N, K]: gather the byte table, multiply each block by its scale."""
    values = lut8[bq.long()].flatten(start_dim=1)
    return values.view(*bs.shape, -1).mul(bs[:, :, None]).flatten(start_dim=1)


def mm_lut_ref(a: Tensor, bq: Tensor, lut8: Tensor, bs: Tensor) -> Tensor:
    """a @ W.T with W materialised by dequantise_ref (same dtype throughout)."""
    return torch.matmul(a, dequantise_ref(bq, lut8, bs).T)


def rmsen(expected: Tensor, actual: Tensor) -> float:
    sse = expected.float().pow(2).sum()
    return float((actual.float() - expected.float()).pow(2).sum().div(sse).sqrt())
