"""The reference's Marlin selector (src/fdk/marlin/__init__.py: `Layer`, `Layer.pack`, `mul`,
`replace_linear`) on the native sm_100a kernels.

The reference JIT-builds Marlin's own CUDA extension here (fp16 x int4 `mma.sync` kernel,
src/fdk/marlin/marlin_cuda_kernel.cu).  This module keeps its Python surface and its packed
tensor format -- `B` int32 [K/16, 2N], `s` fp16 [K/groupsize, N], `centroids` fp16 [256, 2],
so that Marlin-format state dicts load and save unchanged -- and runs the product on
libfdk_b200's fused kernel in its fp16 instantiation: the Marlin tensors are converted once
(`import_marlin`) into packed codes + block scales, repacked into the kernels' tiled layout and
cached per `B` tensor.

Marlin format, restated (src/fdk/marlin/__init__.py:57-87, 152-189).  Quantised values
q[k][n] in 0..15 (weight = (q - 8) * s[k // groupsize][n]) are cut into 16 x 16 tiles; a row of
`B` holds one 16-row band of K, tile after tile, and inside every run of four tiles (1024
values = 128 int32) the values are shuffled so that one int32 holds what one thread of an
m16n8k16 B fragment needs: value (ki, ni) of tile t of the run goes to position
32 * (4 * (ni % 8) + (ki // 2) % 4) + 8 * t + e of the run, where e enumerates
{column half ni // 8} x {row group ki // 8} x {ki % 2} in an order that differs between the
linear variant (even/odd split for the magic-number conversion) and the lookup-table variant
(consecutive K elements in one byte).  Eight consecutive positions make one int32, position
8 j + i in nibble i.  Scales are shuffled in runs of 64 (grouped) or 32 (one group).
"""

from __future__ import annotations

import weakref

import torch
from torch import Tensor, nn

from . import native

# order of the eight values of one thread within an int32 (position e of the run -> which of the
# eight it is), src/fdk/marlin/__init__.py:73-78
_NIBBLE_ORDER = {True: (0, 2, 4, 6, 1, 3, 5, 7), False: (0, 1, 4, 5, 2, 3, 6, 7)}


def _run_position(ki: Tensor, ni: Tensor, tile_in_run: Tensor, is_linear: bool) -> Tensor:
    """Position (0..1023) inside a run of four tiles of value (ki, ni) of tile `tile_in_run`."""
    order = torch.tensor(_NIBBLE_ORDER[is_linear])
    which = 4 * (ni // 8) + 2 * (ki // 8) + ki % 2           # which of the thread's eight values
    slot = torch.empty(8, dtype=torch.long)
    slot[order] = torch.arange(8)                            # value `which` sits in nibble slot[which]
    thread = 4 * (ni % 8) + (ki // 2) % 4
    return 32 * thread + 8 * tile_in_run + slot[which]


def _positions(k: int, n: int, is_linear: bool) -> tuple[Tensor, Tensor]:
    """For every (k, n): the flat index into B viewed as nibbles [K/16, 16 N] -- (row, nibble column)."""
    kk, nn_ = torch.meshgrid(torch.arange(k), torch.arange(n), indexing="ij")
    tile = nn_ // 16
    pos = _run_position(kk % 16, nn_ % 16, tile % 4, is_linear)
    return kk // 16, (tile // 4) * 1024 + pos


def _scale_order(groups: int, n: int, single: bool) -> Tensor:
    """index[j] = which element of the row-major [groups, n] scales sits at flat position j of `s`."""
    flat = torch.arange(groups * n)
    if single:
        within = torch.tensor([2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)])
        return (flat.view(-1, 32)[:, within]).reshape(-1)
    within = torch.tensor([i + 8 * j for i in range(8) for j in range(8)])
    return (flat.view(-1, 64)[:, within]).reshape(-1)


def pack_marlin(q: Tensor, scales: Tensor, groupsize: int, is_linear: bool) -> tuple[Tensor, Tensor]:
    """q [K, N] integers 0..15 and scales [K/groupsize, N] fp16 -> (B int32 [K/16, 2N], s fp16 [K/groupsize, N])."""
    k, n = q.shape
    row, col = _positions(k, n, is_linear)
    nibbles = torch.zeros((k // 16, 16 * n), dtype=torch.int64)
    nibbles[row, col] = q.to(torch.int64).cpu()
    words = (nibbles.view(k // 16, 2 * n, 8) << (4 * torch.arange(8))).sum(-1)
    words = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
    order = _scale_order(scales.shape[0], n, single=groupsize == k)
    s = scales.reshape(-1).cpu()[order].view(scales.shape[0], n).contiguous()
    return words, s


def import_marlin(B: Tensor, s: Tensor, is_linear: bool = True) -> tuple[Tensor, Tensor]:
    """Marlin tensors -> the packed format of `QuantisedLinear`: codes uint8 [N, K/2] (first of two
    consecutive K elements in the high nibble) and scales fp16 [N, K/groupsize].  With the linear
    grid `arange(-8, 8)` as codebook (or the layer's own [256, 2] table, see `byte_table`), the
    dequantised weight equals Marlin's (q - 8) * s bit for bit."""
    k, n = B.shape[0] * 16, B.shape[1] // 2
    device = B.device
    words = B.to(torch.int64).cpu() & 0xFFFFFFFF
    nibbles = ((words[:, :, None] >> (4 * torch.arange(8))) & 15).view(k // 16, 16 * n)
    row, col = _positions(k, n, is_linear)
    q = nibbles[row, col]                                    # [K, N]
    codes = (q[0::2] * 16 + q[1::2]).T.contiguous().to(torch.uint8)
    groups = s.shape[0]
    order = _scale_order(groups, n, single=groups == 1)
    scales = torch.empty(groups * n, dtype=s.dtype)
    scales[order] = s.reshape(-1).cpu()
    return codes.to(device), scales.view(groups, n).T.contiguous().to(device)


def byte_table(centroids: Tensor | None, device, dtype=torch.half) -> Tensor:
    """The [256, 2] table of `QuantisedLinear` for a Marlin layer: row (e0 << 4 | e1) = values of the
    two elements.  Marlin's own table is indexed with the second element in the high nibble
    (src/fdk/marlin/marlin_cuda_kernel.cu:156-167); None stands for the linear grid -8 .. 7."""
    if centroids is None:
        values = torch.arange(-8, 8, dtype=dtype, device=device)
        return torch.cartesian_prod(values, values).view(256, 2)
    swapped = (torch.arange(256, device=centroids.device) % 16) * 16 + torch.arange(256, device=centroids.device) // 16
    return centroids[swapped].contiguous()


_converted: dict[int, tuple] = {}


def _native_form(B: Tensor, s: Tensor, centroids: Tensor | None):
    """(tiled buffer, byte table, n, k), converted once per `B` tensor object and version."""
    key = id(B)
    stamp = (B._version, id(s), s._version, None if centroids is None else (id(centroids), centroids._version))
    hit = _converted.get(key)
    if hit is not None and hit[0]() is B and hit[1] == stamp:
        return hit[2]
    codes, scales = import_marlin(B, s, is_linear=centroids is None)
    n, k = codes.shape[0], codes.shape[1] * 2
    tiled = native.repack(codes, scales, n, k, 4, k // scales.shape[1])
    form = (tiled, byte_table(centroids, B.device, s.dtype), n, k)
    _converted[key] = (weakref.ref(B, lambda _, k_=key: _converted.pop(k_, None)), stamp, form)
    return form


def mul(A, B, C, s, centroids, workspace, thread_k=-1, thread_n=-1, sms=-1, max_par=16):
    """FP16 x INT4 multiply with the reference's signature (src/fdk/marlin/__init__.py:37-51).
    @A: `torch.half` input matrix of shape `(m, k)`
    @B: `torch.int` weight matrix of original shape `(k, n)` in Marlin format; see `Layer.pack()`
    @C: `torch.half` out matrix of shape `(m, n)`
    @s: `torch.half` scales of shape `(k / groupsize, n)` in Marlin order
    @centroids: `torch.half` table of shape `(256, 2)`, or `None` for the linear grid
    @workspace, @thread_k, @thread_n, @sms, @max_par: accepted for compatibility; the native
        kernels plan for themselves and keep their own scratch
    """
    if A.dtype != torch.half or C.dtype != torch.half or s.dtype != torch.half:
        raise RuntimeError("marlin.mul takes torch.half tensors")
    tiled, table, n, k = _native_form(B, s, centroids)
    if A.shape[-1] != k or C.shape[-1] != n or A.shape[0] != C.shape[0]:
        raise RuntimeError(f"Problem (m={A.shape[0]}, n={C.shape[-1]}, k={A.shape[-1]}) does not match the weight ({n} x {k}).")
    native.linear_lut(A.contiguous(), tiled, table, C, n, k, 4)


class Layer(nn.Module):
    """Marlin layer of the reference: 4-bit (symmetric grouped) linear layer without bias."""

    def __init__(self, infeatures, outfeatures, groupsize=-1, is_linear=False):
        """Create an empty Marlin layer.
        @infeatures: number of input features (must be divisible by 128)
        @outfeatures: number of output features (must be divisible by 256)
        @groupsize: quantization groupsize (must be -1, 128 or 64)
        """
        super().__init__()
        if groupsize not in [-1, 128, 64]:
            raise ValueError("Only groupsize -1, 128 and 64 are supported.")
        if infeatures % 128 != 0 or outfeatures % 256 != 0:
            raise ValueError("`infeatures` must be divisible by 128 and `outfeatures` by 256.")
        if groupsize == -1:
            groupsize = infeatures
        if infeatures % groupsize != 0:
            raise ValueError("`infeatures` must be divisible by `groupsize`.")
        self.k = infeatures
        self.n = outfeatures
        self.groupsize = groupsize
        self.is_linear = is_linear
        self.register_buffer("B", torch.empty((self.k // 16, self.n * 16 // 8), dtype=torch.int))
        self.register_buffer("s", torch.empty((self.k // groupsize, self.n), dtype=torch.half))
        self.register_buffer("workspace", torch.zeros(self.n // 128 * 16, dtype=torch.int), persistent=False)
        if is_linear:
            self.centroids = None
        else:
            self.register_buffer("centroids", torch.randn((256, 2), dtype=torch.half))

    def forward(self, A):
        C = torch.empty(A.shape[:-1] + (self.s.shape[1],), dtype=A.dtype, device=A.device)
        mul(A.view((-1, A.shape[-1])), self.B, C.view((-1, C.shape[-1])), self.s, self.centroids, self.workspace)
        return C

    def pack(self, linear, scales):
        """Pack a fake-quantized linear layer into the Marlin representation.
        @linear: fake-quantized `torch.nn.Linear` layer to convert (must be of type `torch.half`)
        @scales: corresponding quantization scales of shape `(outfeatures, groups)`
        """
        if linear.weight.dtype != torch.half:
            raise ValueError("Only `torch.half` weights are supported.")
        w = linear.weight.data.T                                    # [K, N]
        per_element = scales.T.repeat_interleave(self.groupsize, dim=0)   # the scale of every (k, n)
        q = torch.round(w / per_element).int().add_(8).clamp_(0, 15)
        B, s = pack_marlin(q, scales.T.contiguous(), self.groupsize, self.is_linear)
        self.B[:, :] = B.to(self.B.device)
        self.s[:, :] = s.to(self.s.device)


def replace_linear(module, name_filter=lambda n: True, groupsize=-1, name=""):
    """Recursively replace all `torch.nn.Linear` layers by empty Marlin layers.
    @module: top-level module in which to perform the replacement
    @name_filter: lambda indicating if a layer should be replaced
    @groupsize: marlin groupsize
    @name: root-level name
    """
    if isinstance(module, Layer):
        return
    for attr in dir(module):
        child = getattr(module, attr)
        path = f"{name}.{attr}" if name else attr
        if isinstance(child, nn.Linear) and name_filter(path):
            setattr(module, attr, Layer(child.in_features, child.out_features, groupsize=groupsize))
    for child_name, child in module.named_children():
        replace_linear(child, name_filter, groupsize=groupsize, name=f"{name}.{child_name}" if name else child_name)
