"""CPU-side checks of the C-ABI library: it loads, exports every symbol the public header
declares, and its host-only entry points and argument validation behave.  No kernel runs."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

import tiled_layout as TL

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from fdk import native

    return native.lib()


def declared_symbols() -> list[str]:
    text = (ROOT / "include" / "fdk_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fdk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert "fdk_linear_lut" in names and "fdk_repack" in names and len(names) >= 11
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/fdk_b200.h but not exported"


def test_version_and_status_strings(lib):
    assert lib.fdk_version() >= 100
    assert lib.fdk_status_string(0) == b"ok"
    assert lib.fdk_status_string(2) == b"unsupported shape"
    assert b"unknown" in lib.fdk_status_string(1234)


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("n,k", [(64, 64), (100, 384), (4096, 4096), (128256, 3072)])
def test_tiled_size_matches_host_model(lib, bits, n, k):
    out = ctypes.c_size_t(0)
    assert lib.fdk_tiled_size(n, k, bits, ctypes.byref(out)) == 0
    assert out.value == TL.tiled_size(n, k, bits)
    if n % 64 == 0 and k % 256 == 0:
        # no padding: exactly the packed-weight bytes (codes + one 16-bit scale per 64)
        assert out.value == n * k * bits // 8 + n * (k // 64) * 2


def test_argument_validation_needs_no_gpu(lib):
    from fdk import native

    out = ctypes.c_size_t(0)
    assert lib.fdk_tiled_size(64, 100, 4, ctypes.byref(out)) == 2  # k not a multiple of 64
    assert lib.fdk_tiled_size(64, 128, 5, ctypes.byref(out)) == 2  # bits
    assert lib.fdk_tiled_size(0, 128, 4, ctypes.byref(out)) == 1
    assert lib.fdk_tiled_size(64, 128, 4, None) == 1
    assert lib.fdk_repack(None, None, 64, 128, 4, 64, None, None) == 1
    assert lib.fdk_repack(None, None, 64, 128, 4, 32, None, None) == 2  # block size
    assert lib.fdk_linear_lut(None, None, None, None, None, 1, 64, 128, 4, 0, None, 0, 0, None) == 1
    assert lib.fdk_linear_lut(None, None, None, None, None, 1, 64, 128, 4, 0, None, 0, 8, None) == 1
    assert lib.fdk_workspace_init(None, 0, None) == 6
    with pytest.raises(native.FdkError) as e:
        native.check(lib.fdk_tiled_size(64, 100, 4, ctypes.byref(out)))
    assert "multiple of 64" in str(e.value)


def test_python_ops_refuse_cpu_tensors():
    import torch

    from fdk import kernels, native

    a = torch.zeros(128, dtype=torch.bfloat16)
    b = torch.zeros((64, 64), dtype=torch.uint8)
    lut = torch.zeros((256, 2), dtype=torch.bfloat16)
    bs = torch.zeros((64, 2), dtype=torch.bfloat16)
    out = torch.zeros(64, dtype=torch.bfloat16)
    with pytest.raises(native.FdkError):
        kernels.run_mv_lut(a, b, lut, bs, out)


def test_host_layout_model_is_a_permutation():
    rng = np.random.default_rng(0)
    for bits in (1, 2, 4, 8):
        n, k = 128, 512
        codes = rng.integers(0, 256, size=(n, k * bits // 8), dtype=np.uint8)
        scale = rng.integers(1, 65535, size=(n, k // 64), dtype=np.uint16)
        tiled = TL.repack(codes, scale, bits)
        # no padding at this shape: the tiled buffer is a permutation of the source bytes
        src = np.concatenate([codes.ravel(), scale.view(np.uint8).ravel()])
        assert np.array_equal(np.sort(tiled), np.sort(src))


def test_exchange_entry_points_validate_without_a_gpu(lib):
    from fdk import native

    assert lib.fdk_tp_exchange_bytes(2, 1024) == 256 + 2 * 2 * 1024 * 4
    assert lib.fdk_tp_exchange_bytes(0, 1024) == 0 and lib.fdk_tp_exchange_bytes(9, 1024) == 0
    assert lib.fdk_tp_exchange_bytes(2, 0) == 0
    assert lib.fdk_linear_lut_push(None, None, None, None, 1, 64, 64, 4, 0, None, 0, 0, None, None) == 1
    assert lib.fdk_rmsnorm_reduce(None, None, None, None, 1, 64, 1e-5, None) == 1
    assert lib.fdk_tp_buffer_open(None, None) == 1
    assert lib.fdk_tp_buffer_close(None) == 1 and lib.fdk_tp_buffer_destroy(None) == 1
    ex = native.make_exchange(2, 1, [4096, 8192], 512)
    assert (ex.tp, ex.rank, ex.slot_elems, ex.buffers[1]) == (2, 1, 512, 8192)
    assert ctypes.sizeof(native.TpExchange) == 8 + 8 * 8 + 8


def test_attention_slice_plan():
    """`attention_slices`: about 96 keys or more per slice, at most 16 slices, the grid within the
    given number of CTAs (two per SM of a B200 here)."""
    from fdk import native

    plan = lambda batch, kv, max_len: native.attention_slices(batch, 3 * kv, kv, max_len, ctas=296)
    assert plan(1, 8, 1153) == 12      # context 1024 of the 4B model: 12 slices of 97 keys
    assert plan(1, 8, 2177) == 16      # capped
    assert plan(4, 8, 1153) == 9       # 296 // 32
    assert plan(16, 8, 1153) == 2
    assert plan(64, 8, 1153) == 1      # larger than the GPU already: one slice
    assert plan(1, 8, 64) == 1         # fewer than 96 keys: one slice
    for batch in (1, 2, 3, 5, 8, 13, 40):
        for kv in (1, 2, 8):
            s = plan(batch, kv, 4096)
            assert 1 <= s <= 16 and (s == 1 or s * batch * kv <= 296)
