"""ctypes binding of libfdk_b200.so: the only way the package reaches the GPU kernels.

There is no fallback: if the library is missing or a call returns a non-zero
status, an exception is raised (the reference turns its native error codes into
exceptions in the same way, src/fdk/marlin/marlin_cuda.cpp:63-66,84-93).
"""

from __future__ import annotations

import ctypes
import os
import weakref
from pathlib import Path

import torch
from torch import Tensor

_LIB_PATH = Path(__file__).resolve().parent / "libfdk_b200.so"

OK = 0
DTYPE_BF16 = 0
DTYPE_F16 = 1
FLAG_PDL = 1
FLAG_SILU_PAIRS = 2
FLAG_NO_SYNC = 4


class FdkError(RuntimeError):
    def __init__(self, status: int, text: str, detail: str):
        super().__init__(f"libfdk_b200: {text} (status {status}): {detail}")
        self.status = status


_lib: ctypes.CDLL | None = None

TP_MAX_RANKS = 8


class TpExchange(ctypes.Structure):
    """`fdk_tp_exchange` of the C header."""

    _fields_ = [
        ("tp", ctypes.c_int),
        ("rank", ctypes.c_int),
        ("buffers", ctypes.c_void_p * TP_MAX_RANKS),
        ("slot_elems", ctypes.c_longlong),
    ]


class LinearFusion(ctypes.Structure):
    """`fdk_linear_fusion` of the C header: what the projection kernel does besides the product."""

    _fields_ = [
        ("norm_h", ctypes.c_void_p),
        ("norm_weight", ctypes.c_void_p),
        ("norm_sumsq", ctypes.c_void_p),
        ("norm_tiles", ctypes.c_int),
        ("norm_eps", ctypes.c_float),
        ("resid_h", ctypes.c_void_p),
        ("resid_sumsq", ctypes.c_void_p),
        ("rope_pos", ctypes.c_void_p),
        ("rope_table", ctypes.c_void_p),
        ("q_out", ctypes.c_void_p),
        ("k_cache", ctypes.c_void_p),
        ("v_cache", ctypes.c_void_p),
        ("q_heads", ctypes.c_int),
        ("kv_heads", ctypes.c_int),
        ("max_len", ctypes.c_int),
        ("resid_norm_weight", ctypes.c_void_p),
        ("resid_x", ctypes.c_void_p),
        ("scale_sumsq", ctypes.c_void_p),
        ("scale_tiles", ctypes.c_int),
        ("scale_eps", ctypes.c_float),
    ]


_SIGNATURES = {
    "fdk_linear_lut_fused": (
        ctypes.c_int,
        [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5
        + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.POINTER(LinearFusion), ctypes.c_void_p],
    ),
    "fdk_rope_table": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p]),
    "fdk_sumsq_tiles": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "fdk_norm_prepare": (ctypes.c_int, [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "fdk_tp_exchange_bytes": (ctypes.c_size_t, [ctypes.c_int, ctypes.c_longlong]),
    "fdk_tp_buffer_create": (ctypes.c_int, [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]),
    "fdk_tp_buffer_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "fdk_tp_buffer_close": (ctypes.c_int, [ctypes.c_void_p]),
    "fdk_tp_buffer_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "fdk_tp_exchange_status": (ctypes.c_int, [ctypes.POINTER(TpExchange), ctypes.POINTER(ctypes.c_int)]),
    "fdk_linear_lut_push": (
        ctypes.c_int,
        [ctypes.c_void_p] * 4 + [ctypes.c_int] * 5
        + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.POINTER(TpExchange), ctypes.c_void_p],
    ),
    "fdk_rmsnorm_reduce": (
        ctypes.c_int,
        [ctypes.c_void_p, ctypes.POINTER(TpExchange), ctypes.c_void_p, ctypes.c_void_p]
        + [ctypes.c_int] * 2 + [ctypes.c_float, ctypes.c_void_p],
    ),
    "fdk_version": (ctypes.c_int, []),
    "fdk_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "fdk_last_error_detail": (ctypes.c_char_p, []),
    "fdk_tiled_size": (ctypes.c_int, [ctypes.c_int] * 3 + [ctypes.POINTER(ctypes.c_size_t)]),
    "fdk_repack": (ctypes.c_int, [ctypes.c_void_p] * 2 + [ctypes.c_int] * 4 + [ctypes.c_void_p] * 2),
    "fdk_unpack": (ctypes.c_int, [ctypes.c_void_p] + [ctypes.c_int] * 4 + [ctypes.c_void_p] * 3),
    "fdk_dequantise": (ctypes.c_int, [ctypes.c_void_p] * 3 + [ctypes.c_int] * 5 + [ctypes.c_void_p] * 2),
    "fdk_dequantise_tiled": (ctypes.c_int, [ctypes.c_void_p] * 2 + [ctypes.c_int] * 4 + [ctypes.c_void_p] * 2),
    "fdk_workspace_size": (ctypes.c_int, [ctypes.POINTER(ctypes.c_size_t)]),
    "fdk_workspace_init": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "fdk_linear_lut_static": (
        ctypes.c_int,
        [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_uint, ctypes.c_void_p],
    ),
    "fdk_static_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "fdk_linear_norm_fits": (ctypes.c_int, [ctypes.c_int] * 3 + [ctypes.POINTER(ctypes.c_int)]),
    "fdk_rmsnorm": (ctypes.c_int, [ctypes.c_void_p] * 4 + [ctypes.c_int] * 2 + [ctypes.c_float, ctypes.c_void_p]),
    "fdk_rope_append": (ctypes.c_int, [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_void_p]),
    "fdk_rope_append_paired": (ctypes.c_int, [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_void_p]),
    "fdk_silu_mul": (ctypes.c_int, [ctypes.c_void_p] * 2 + [ctypes.c_int] * 3 + [ctypes.c_void_p]),
    "fdk_decode_attention_scratch": (ctypes.c_int, [ctypes.c_int] * 4 + [ctypes.POINTER(ctypes.c_size_t)] * 2),
    "fdk_decode_attention": (ctypes.c_int, [ctypes.c_void_p] * 7 + [ctypes.c_int] * 6 + [ctypes.c_void_p]),
    "fdk_argmax": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "fdk_decode_attention_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]),
    "fdk_workspace_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]),
    "fdk_linear_lut": (
        ctypes.c_int,
        [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p],
    ),
    "fdk_linear_lut_host": (
        ctypes.c_int,
        [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5
        + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p],
    ),
}


def library_path() -> Path:
    return Path(os.environ.get("FDK_B200_LIBRARY", _LIB_PATH))


def lib() -> ctypes.CDLL:
    """Loads the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not path.exists():
            raise FdkError(
                -1,
                "native library not built",
                f"{path} is missing; run `python fused-dequantisation-kernels_b200/build.py` "
                "(there is no CPU or PyTorch fallback for the kernels)",
            )
        handle = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue  # optional entry points are bound where they are used
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != OK:
        handle = lib()
        raise FdkError(
            status,
            handle.fdk_status_string(status).decode(),
            handle.fdk_last_error_detail().decode(),
        )


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return DTYPE_BF16
    if dtype == torch.float16:
        return DTYPE_F16
    raise TypeError(f"fdk kernels take bfloat16 or float16, got {dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise FdkError(-2, "tensor not on a CUDA device", "the fdk kernels have no CPU path")


def tiled_size(n: int, k: int, bits: int) -> int:
    out = ctypes.c_size_t(0)
    check(lib().fdk_tiled_size(n, k, bits, ctypes.byref(out)))
    return out.value


def repack(codes: Tensor, scale: Tensor, n: int, k: int, bits: int, block_size: int) -> Tensor:
    """Packed codes + scales (reference layout) -> tiled uint8 buffer on the same device."""
    _require_cuda(codes, scale)
    assert codes.dtype == torch.uint8 and codes.is_contiguous() and scale.is_contiguous()
    tiled = torch.empty(tiled_size(n, k, bits), dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        check(lib().fdk_repack(codes.data_ptr(), scale.data_ptr(), n, k, bits, block_size, tiled.data_ptr(), _stream()))
    return tiled


def unpack(tiled: Tensor, n: int, k: int, bits: int, block_size: int, dtype: torch.dtype) -> tuple[Tensor, Tensor]:
    _require_cuda(tiled)
    codes = torch.empty((n, k * bits // 8), dtype=torch.uint8, device=tiled.device)
    scale = torch.empty((n, k // block_size), dtype=dtype, device=tiled.device)
    with torch.cuda.device(tiled.device):
        check(lib().fdk_unpack(tiled.data_ptr(), n, k, bits, block_size, codes.data_ptr(), scale.data_ptr(), _stream()))
    return codes, scale


def dequantise(codes: Tensor, lut: Tensor, scale: Tensor, bits: int) -> Tensor:
    _require_cuda(codes, lut, scale)
    n = codes.shape[0]
    k = codes.shape[1] * 8 // bits
    block_size = k // scale.shape[1]
    assert lut.dtype == scale.dtype and all(t.is_contiguous() for t in (codes, lut, scale))
    w = torch.empty((n, k), dtype=scale.dtype, device=codes.device)
    with torch.cuda.device(codes.device):
        check(
            lib().fdk_dequantise(
                codes.data_ptr(), lut.data_ptr(), scale.data_ptr(), n, k, bits, block_size,
                dtype_code(scale.dtype), w.data_ptr(), _stream(),
            )
        )
    return w


def dequantise_tiled(tiled: Tensor, lut: Tensor, n: int, k: int, bits: int) -> Tensor:
    _require_cuda(tiled, lut)
    w = torch.empty((n, k), dtype=lut.dtype, device=tiled.device)
    with torch.cuda.device(tiled.device):
        check(lib().fdk_dequantise_tiled(tiled.data_ptr(), lut.data_ptr(), n, k, bits, dtype_code(lut.dtype), w.data_ptr(), _stream()))
    return w


_workspaces: dict[tuple[int, int], Tensor] = {}


def workspace(device: torch.device) -> Tensor:
    """One zero-initialised scratch buffer per (device, stream).  Allocated on first use,
    so the first call on a stream must happen before that stream is captured in a graph."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, _stream())
    ws = _workspaces.get(key)
    if ws is None:
        with torch.cuda.device(index):
            size = ctypes.c_size_t(0)
            check(lib().fdk_workspace_size(ctypes.byref(size)))
            ws = torch.empty(size.value, dtype=torch.uint8, device=f"cuda:{index}")
            check(lib().fdk_workspace_init(ws.data_ptr(), size.value, _stream()))
        _workspaces[key] = ws
    return ws


def device_status(device: torch.device | None = None) -> int:
    """Device-side status word of the current stream's workspace (synchronises)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    out = ctypes.c_int(0)
    check(lib().fdk_workspace_status(workspace(device).data_ptr(), ctypes.byref(out)))
    return out.value


def static_status() -> int:
    """Device-side status word of the scratch built into fdk_linear_lut_static (synchronises)."""
    out = ctypes.c_int(0)
    check(lib().fdk_static_status(ctypes.byref(out)))
    return out.value


def linear_norm_fits(m: int, k: int, bits: int) -> bool:
    """Whether `linear_lut_fused` can apply its RMSNorm to a batch of m rows of k columns."""
    out = ctypes.c_int(0)
    check(lib().fdk_linear_norm_fits(m, k, bits, ctypes.byref(out)))
    return bool(out.value)


_host_luts: dict[int, tuple[weakref.ref, int, bytes]] = {}


def host_lut(lut: Tensor) -> bytes:
    """Host copy of a lookup table, made once per tensor object and version: it rides along
    with the launch parameters so that the kernel need not fetch the table from memory.
    The first call for a table synchronises (device -> host copy)."""
    key = id(lut)
    hit = _host_luts.get(key)
    if hit is not None and hit[0]() is lut and hit[1] == lut._version:
        return hit[2]
    data = lut.detach().contiguous().view(torch.int16).cpu().numpy().tobytes()
    _host_luts[key] = (weakref.ref(lut, lambda _, k=key: _host_luts.pop(k, None)), lut._version, data)
    return data


def linear_lut(
    x: Tensor, tiled: Tensor, lut: Tensor, out: Tensor, n: int, k: int, bits: int,
    pdl: bool = False, lut_bytes: bytes | None = None, silu_pairs: bool = False,
) -> None:
    """out[m, n] = x[m, k] @ W.T, W never materialised.  Writes `out` in place.  silu_pairs: W's
    rows alternate 32 gate rows and their 32 up rows, out[m, n / 2] = silu(gate) * up (m <= 16)."""
    _require_cuda(x, tiled, lut, out)
    m = x.shape[0]
    ws = workspace(x.device)
    if lut_bytes is None:
        lut_bytes = host_lut(lut)
    with torch.cuda.device(x.device):
        check(
            lib().fdk_linear_lut(
                x.data_ptr(), tiled.data_ptr(), lut.data_ptr(), lut_bytes, out.data_ptr(), m, n, k, bits,
                dtype_code(x.dtype), ws.data_ptr(), ws.numel(),
                (FLAG_PDL if pdl else 0) | (FLAG_SILU_PAIRS if silu_pairs else 0), _stream(),
            )
        )


def linear_lut_host(
    x_host: Tensor, tiled: Tensor, lut: Tensor, out_host: Tensor, x_dev: Tensor, out_dev: Tensor, n: int, k: int,
    bits: int, lut_bytes: bytes | None = None,
) -> None:
    """out_host[m, n] = x_host[m, k] @ W.T for activations in host memory: copy in, projection, copy
    out and a stream synchronisation in one library call.  x_dev / out_dev: device staging buffers."""
    _require_cuda(tiled, lut, x_dev, out_dev)
    assert not x_host.is_cuda and not out_host.is_cuda and x_host.is_contiguous() and out_host.is_contiguous()
    m = x_host.shape[0]
    assert x_dev.numel() >= m * k and out_dev.numel() >= m * n and out_host.numel() == m * n and x_host.shape[1] == k
    ws = workspace(tiled.device)
    if lut_bytes is None:
        lut_bytes = host_lut(lut)
    with torch.cuda.device(tiled.device):
        check(
            lib().fdk_linear_lut_host(
                x_host.data_ptr(), tiled.data_ptr(), lut.data_ptr(), lut_bytes, out_host.data_ptr(), m, n, k, bits,
                dtype_code(x_host.dtype), x_dev.data_ptr(), out_dev.data_ptr(), ws.data_ptr(), ws.numel(), 0, _stream(),
            )
        )


def prepare_linear_lut_host(tiled: Tensor, lut: Tensor, lut_bytes: bytes, x_dev: Tensor, out_dev: Tensor, m: int,
                            n: int, k: int, bits: int, dtype: torch.dtype, synchronise: bool = True):
    """`linear_lut_host` with everything but the two host pointers bound once (current stream and
    workspace included): returns call(x_host_ptr, out_host_ptr).  For callers that make the same call
    many times -- the argument marshalling is a visible part of a 40 us round trip."""
    _require_cuda(tiled, lut, x_dev, out_dev)
    assert x_dev.numel() >= m * k and out_dev.numel() >= m * n
    fn = lib().fdk_linear_lut_host
    ws = workspace(tiled.device)
    index = tiled.device.index
    fixed_a = (tiled.data_ptr(), lut.data_ptr(), lut_bytes)
    fixed_b = (m, n, k, bits, dtype_code(dtype), x_dev.data_ptr(), out_dev.data_ptr(), ws.data_ptr(), ws.numel(),
               0 if synchronise else FLAG_NO_SYNC, _stream())
    keep = (tiled, lut, x_dev, out_dev, ws)  # the buffers live as long as the call does

    def call(x_host_ptr: int, out_host_ptr: int, _keep=keep) -> None:
        if torch.cuda.current_device() == index:
            status = fn(x_host_ptr, *fixed_a, out_host_ptr, *fixed_b)
        else:
            with torch.cuda.device(index):
                status = fn(x_host_ptr, *fixed_a, out_host_ptr, *fixed_b)
        if status != OK:
            check(status)

    return call


def linear_lut_fused(
    x: Tensor | None, tiled: Tensor, lut: Tensor, out: Tensor | None, m: int, n: int, k: int, bits: int,
    fusion: LinearFusion, pdl: bool = False, lut_bytes: bytes | None = None, silu_pairs: bool = False,
) -> None:
    """fdk_linear_lut with the decode-step fusions of `fusion` (see the C header): RMSNorm on the
    input side; residual add + sums of squares, or rotary embedding + KV append, on the output side."""
    _require_cuda(tiled, lut)
    ws = workspace(tiled.device)
    if lut_bytes is None:
        lut_bytes = host_lut(lut)
    with torch.cuda.device(tiled.device):
        check(
            lib().fdk_linear_lut_fused(
                None if x is None else x.data_ptr(), tiled.data_ptr(), lut.data_ptr(), lut_bytes,
                None if out is None else out.data_ptr(), m, n, k, bits, DTYPE_BF16, ws.data_ptr(), ws.numel(),
                (FLAG_PDL if pdl else 0) | (FLAG_SILU_PAIRS if silu_pairs else 0), ctypes.byref(fusion), _stream(),
            )
        )


def rope_table(pos: Tensor, table: Tensor, theta: float) -> None:
    """table[64] int32 = {bf16 cos, bf16 sin} of the rotary angles at position `pos` (device int64)."""
    _require_cuda(pos, table)
    assert pos.dtype == torch.int64 and table.dtype == torch.int32 and table.numel() == 64
    with torch.cuda.device(pos.device):
        check(lib().fdk_rope_table(pos.data_ptr(), table.data_ptr(), theta, _stream()))


def norm_prepare(h: Tensor, weight: Tensor, x: Tensor, sumsq: Tensor) -> None:
    """x = bf16(weight * h) and sumsq[rows, ceil(width / 64)] = sums of squares of h per 64 elements:
    the producer side of the deferred RMSNorm of `linear_lut_fused`."""
    _require_cuda(h, weight, x, sumsq)
    rows, width = h.shape
    assert h.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
    assert h.is_contiguous() and x.is_contiguous() and x.shape == h.shape and weight.numel() == width
    assert sumsq.dtype == torch.float32 and sumsq.shape == (rows, (width + 63) // 64)
    with torch.cuda.device(h.device):
        check(lib().fdk_norm_prepare(h.data_ptr(), weight.data_ptr(), x.data_ptr(), sumsq.data_ptr(), rows, width, _stream()))


def sumsq_tiles(h: Tensor, sumsq: Tensor) -> None:
    """sumsq[rows, ceil(width / 64)] float32 = sums of squares of h per 64 elements."""
    _require_cuda(h, sumsq)
    rows, width = h.shape
    assert sumsq.dtype == torch.float32 and sumsq.shape == (rows, (width + 63) // 64)
    with torch.cuda.device(h.device):
        check(lib().fdk_sumsq_tiles(h.data_ptr(), sumsq.data_ptr(), rows, width, _stream()))


def rmsnorm(h: Tensor, delta: Tensor | None, weight: Tensor, out: Tensor, eps: float) -> None:
    """h += delta (when given, in place), out = RMSNorm(h) * weight.  bf16 [rows, width]."""
    _require_cuda(h, weight, out)
    rows, width = h.shape
    with torch.cuda.device(h.device):
        check(
            lib().fdk_rmsnorm(
                h.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(), out.data_ptr(),
                rows, width, eps, _stream(),
            )
        )


# ---- tensor-parallel exchange -------------------------------------------------------------


def tp_exchange_bytes(tp: int, slot_elems: int) -> int:
    size = lib().fdk_tp_exchange_bytes(tp, slot_elems)
    if size == 0:
        raise FdkError(1, "bad argument", f"tp={tp}, slot_elems={slot_elems}")
    return size


def tp_buffer_create(nbytes: int, device: torch.device) -> tuple[int, bytes]:
    """Zeroed device buffer that other processes can map -> (device pointer, 64-byte handle)."""
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    with torch.cuda.device(device):
        check(lib().fdk_tp_buffer_create(nbytes, ctypes.byref(ptr), handle))
    return ptr.value, handle.raw


def tp_buffer_open(handle: bytes, device: torch.device) -> int:
    ptr = ctypes.c_void_p()
    with torch.cuda.device(device):
        check(lib().fdk_tp_buffer_open(handle, ctypes.byref(ptr)))
    return ptr.value


def tp_buffer_close(ptr: int) -> None:
    check(lib().fdk_tp_buffer_close(ptr))


def tp_buffer_destroy(ptr: int) -> None:
    check(lib().fdk_tp_buffer_destroy(ptr))


def make_exchange(tp: int, rank: int, buffers: list[int], slot_elems: int) -> TpExchange:
    ex = TpExchange()
    ex.tp, ex.rank, ex.slot_elems = tp, rank, slot_elems
    for j, ptr in enumerate(buffers):
        ex.buffers[j] = ptr
    return ex


def tp_exchange_status(ex: TpExchange) -> int:
    out = ctypes.c_int(0)
    check(lib().fdk_tp_exchange_status(ctypes.byref(ex), ctypes.byref(out)))
    return out.value


def linear_lut_push(
    x: Tensor, tiled: Tensor, lut: Tensor, ex: TpExchange, n: int, k: int, bits: int,
    pdl: bool = False, lut_bytes: bytes | None = None,
) -> None:
    """x[m, k] @ W.T stored into slot `ex.rank` of every rank's exchange buffer (m <= 16)."""
    _require_cuda(x, tiled, lut)
    m = x.shape[0]
    ws = workspace(x.device)
    if lut_bytes is None:
        lut_bytes = host_lut(lut)
    with torch.cuda.device(x.device):
        check(
            lib().fdk_linear_lut_push(
                x.data_ptr(), tiled.data_ptr(), lut.data_ptr(), lut_bytes, m, n, k, bits,
                dtype_code(x.dtype), ws.data_ptr(), ws.numel(), FLAG_PDL if pdl else 0, ctypes.byref(ex), _stream(),
            )
        )


def rmsnorm_reduce(h: Tensor, ex: TpExchange, weight: Tensor, out: Tensor, eps: float) -> None:
    """h += sum over ranks of the latest push (in place), out = RMSNorm(h) * weight."""
    _require_cuda(h, weight, out)
    rows, width = h.shape
    with torch.cuda.device(h.device):
        check(
            lib().fdk_rmsnorm_reduce(
                h.data_ptr(), ctypes.byref(ex), weight.data_ptr(), out.data_ptr(), rows, width, eps, _stream(),
            )
        )


def rope_append(
    qkv: Tensor, pos: Tensor, q_out: Tensor, k_cache: Tensor, v_cache: Tensor,
    q_heads: int, kv_heads: int, theta: float, paired: bool = False,
) -> None:
    """Rotary embedding of the fused q|k|v projection at position `pos` (device int64 scalar),
    k and v appended to the caches [rows, kv_heads, max_len, 128].  paired: the q and k heads come
    in the row order of the projection kernel's rotary output ([0..31, 64..95, 32..63, 96..127])."""
    _require_cuda(qkv, pos, q_out, k_cache, v_cache)
    assert pos.dtype == torch.int64
    with torch.cuda.device(qkv.device):
        check(
            (lib().fdk_rope_append_paired if paired else lib().fdk_rope_append)(
                qkv.data_ptr(), pos.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                qkv.shape[0], q_heads, kv_heads, 128, k_cache.shape[2], theta, _stream(),
            )
        )


def silu_mul(gate_up: Tensor, out: Tensor, group: int | None = None) -> None:
    """out = silu(gate) * up; gate_up's columns alternate `group` gates and `group` ups
    (default: all gates, then all ups)."""
    _require_cuda(gate_up, out)
    rows, width = out.shape
    with torch.cuda.device(out.device):
        check(lib().fdk_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, width, width if group is None else group, _stream()))


def attention_slices(batch: int, q_heads: int, kv_heads: int, max_len: int, ctas: int | None = None) -> int:
    """Context slices per (batch row, KV head) for `decode_attention`: 96 keys or more each (a
    CTA's eight warps then have all their keys in flight at once), as long as the grid
    stays within `ctas` CTAs (default: two per SM, which is what the tensor-core kernel that
    serves grids larger than the GPU runs at); more slices than that only add merge work.
    Measured on a B200, 24 query / 8 KV heads, context 1024: 16 rows 15.5 us unsliced (128 CTAs),
    12.9 us in two slices (256 CTAs); 8 rows 11.0 us in two, 9.4 us in four."""
    if ctas is None:
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count if torch.cuda.is_available() else 148
        ctas = 2 * sms
    return max(1, min(max_len // 96, ctas // (batch * kv_heads), 16))


def attention_scratch(batch: int, q_heads: int, kv_heads: int, splits: int, device: torch.device) -> tuple[Tensor, Tensor]:
    a, b = ctypes.c_size_t(0), ctypes.c_size_t(0)
    check(lib().fdk_decode_attention_scratch(batch, q_heads, kv_heads, splits, ctypes.byref(a), ctypes.byref(b)))
    # both zero-filled once: the slices' words are tagged with the use count kept in the counters
    return (torch.zeros(a.value // 4, dtype=torch.float32, device=device), torch.zeros(b.value // 4, dtype=torch.int32, device=device))


def argmax(x: Tensor, out: Tensor) -> None:
    """out[r] = argmax of row r of x [rows, n] (bf16 or fp16; lowest index among equals)."""
    _require_cuda(x, out)
    assert x.dim() == 2 and x.is_contiguous() and out.dtype == torch.int64 and out.is_contiguous() and out.numel() == x.shape[0]
    with torch.cuda.device(x.device):
        check(lib().fdk_argmax(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], dtype_code(x.dtype), _stream()))


def attention_status(counters: Tensor, batch: int, kv_heads: int) -> int:
    """Status word of a decode-attention scratch (synchronises): 0, or 1 after a wait ran out."""
    out = ctypes.c_int(0)
    with torch.cuda.device(counters.device):
        check(lib().fdk_decode_attention_status(counters.data_ptr(), batch, kv_heads, ctypes.byref(out)))
    return out.value


def decode_attention(q: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor, out: Tensor,
                     scratch: Tensor, counters: Tensor, q_heads: int, kv_heads: int, splits: int) -> None:
    """One query token per batch row against the KV cache [batch, kv_heads, max_len, 128], keys 0..pos."""
    _require_cuda(q, k_cache, v_cache, pos, out)
    with torch.cuda.device(q.device):
        check(
            lib().fdk_decode_attention(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), out.data_ptr(),
                scratch.data_ptr(), counters.data_ptr(), q.shape[0], q_heads, kv_heads, 128, k_cache.shape[2],
                splits, _stream(),
            )
        )
