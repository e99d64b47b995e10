"""Pins the CPU oracle against vectors produced by the reference itself
(tests/golden/make_golden.py).  Everything here is bit-exact."""

import numpy as np
import pytest
import torch

import fdk_oracle as O
import fdk_oracle_torch as OT


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("bits", [8, 4, 2, 1])
def test_quantiser_matches_reference(golden_dir, bits):
    z = np.load(golden_dir / "quantise_linspace.npz")
    p = f"b{bits}_"
    data, scale, table = OT.quantise_weight(_bf16(z[p + "w"]), bits, 64)
    assert np.array_equal(data.numpy(), z[p + "weight_data"])
    assert np.array_equal(_bits(scale), z[p + "scale"])
    assert np.array_equal(_bits(table), z[p + "lut"])


@pytest.mark.parametrize("bits", [4, 2])
def test_quantiser_custom_codebook(golden_dir, bits):
    z = np.load(golden_dir / "quantise_codebook.npz")
    p = f"b{bits}_"
    data, scale, table = OT.quantise_weight(_bf16(z[p + "w"]), bits, 128, lut=_bf16(z[p + "codebook"]))
    assert np.array_equal(data.numpy(), z[p + "weight_data"])
    assert np.array_equal(_bits(scale), z[p + "scale"])
    assert np.array_equal(_bits(table), z[p + "lut"])
    # numpy byte table from the recovered codebook reproduces the reference's table
    assert np.array_equal(O.byte_lut(O.base_lut_from_byte_lut(z[p + "lut"]), bits), z[p + "lut"])


@pytest.mark.parametrize("name,bit_list", [("quantise_linspace.npz", [8, 4, 2, 1]), ("quantise_codebook.npz", [4, 2])])
def test_dequantise_bit_exact(golden_dir, name, bit_list):
    z = np.load(golden_dir / name)
    for bits in bit_list:
        p = f"b{bits}_"
        w = O.dequantise(z[p + "weight_data"], z[p + "lut"], z[p + "scale"])
        assert np.array_equal(w, z[p + "w_deq"]), f"bits={bits}"
        # index-level form agrees with the byte-table form
        k = w.shape[1]
        idx = O.unpack_indices(z[p + "weight_data"], bits, k)
        w2 = O.dequantise_indices(idx, O.base_lut_from_byte_lut(z[p + "lut"]), z[p + "scale"])
        assert np.array_equal(w2, w)
        assert np.array_equal(O.pack_indices(idx, bits), z[p + "weight_data"])
        # torch restatement too
        wt = OT.dequantise_ref(torch.from_numpy(z[p + "weight_data"]), _bf16(z[p + "lut"]), _bf16(z[p + "scale"]))
        assert np.array_equal(_bits(wt), z[p + "w_deq"])


@pytest.mark.parametrize("bits", [8, 4, 2, 1])
def test_matmul_matches_reference(golden_dir, bits):
    z = np.load(golden_dir / "quantise_linspace.npz")
    p = f"b{bits}_"
    y = O.mm_lut(z[p + "x"], z[p + "weight_data"], z[p + "lut"], z[p + "scale"])
    ref = O.bf16_to_f32(z[p + "y"])
    # fp32-vs-float64 accumulation may flip a last bf16 bit; the measure the
    # reference uses (rel-RMS error) must be far inside its 1e-2 tolerance.
    assert O.rmsen(ref, O.bf16_to_f32(y)) < 2e-3
    yt = OT.mm_lut_ref(_bf16(z[p + "x"]), torch.from_numpy(z[p + "weight_data"]), _bf16(z[p + "lut"]), _bf16(z[p + "scale"]))
    assert np.array_equal(_bits(yt), z[p + "y"])
    yv = OT.mm_lut_ref(_bf16(z[p + "x"])[0], torch.from_numpy(z[p + "weight_data"]), _bf16(z[p + "lut"]), _bf16(z[p + "scale"]))
    assert np.array_equal(_bits(yv), z[p + "y_vec"])


def test_reference_kernel_test_inputs(golden_dir):
    z = np.load(golden_dir / "kernel_test_4b.npz")
    y = O.mm_lut(z["a"], z["bq"], z["lut8"], z["bs"])
    assert O.rmsen(O.bf16_to_f32(z["y"]), O.bf16_to_f32(y)) < 2e-3


def test_bf16_rounding_matches_torch():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(100000).astype(np.float32) * np.float32(10.0) ** rng.integers(-20, 20, 100000).astype(np.float32)
    x[:4] = [0.0, -0.0, np.inf, -np.inf]
    ours = O.f32_to_bf16(x)
    theirs = _bits(torch.from_numpy(x).bfloat16())
    assert np.array_equal(ours, theirs)
    assert np.array_equal(O.bf16_to_f32(ours), torch.from_numpy(x).bfloat16().float().numpy())


def test_three_bit_index_format_round_trip():
    rng = np.random.default_rng(3)
    idx = rng.integers(0, 8, size=(16, 128), dtype=np.uint8)
    packed = O.pack_indices(idx, 3)
    assert packed.shape == (16, 48)
    assert np.array_equal(O.unpack_indices(packed, 3, 128), idx)
    # element 0 sits in the top three bits of byte 0
    assert packed[0, 0] >> 5 == idx[0, 0]


def test_accounting_formulas(golden_dir):
    z = np.load(golden_dir / "module_quantise.npz")
    for bits in (8, 4, 2, 1):
        assert int(z[f"b{bits}_count_ops"]) == O.bench_ops(1, 384, 256)
        assert int(z[f"b{bits}_count_bytes"]) == O.packed_weight_bytes(256, 384, bits, 64)
    assert O.packed_weight_bytes(4096, 4096, 4) == 8_912_896
    assert O.bench_bytes_rw(1, 8192, 8192, 64, 4) == 8192 * 8192 // 2 + (8192 + 8192 * 128 + 8192) * 2
