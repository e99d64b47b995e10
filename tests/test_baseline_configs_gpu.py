"""The benchmark configurations themselves as parity cases (seeded synthetic inputs):

  1. one nn.Linear, K = N = 4096, bf16 weights ~ N(0, 1/4096) from seed 100, quantise() with
     4 bits and block 64, batch 1 and 200: packed tensors and dequantised W bit for bit against
     the CPU oracle (the reference's quantiser restated), outputs against the CPU torch
     reference operator within the reference's own tolerance (src/fdk/kernels.py:196,502);
  2. the kernel sweep: K = N in {3072, 4096, 6144, 8192} x bits {1, 2, 3, 4} x batch
     {1, 2, 4, 8, 16}, block 64, a sorted k-means-like codebook of N(0,1), weights ~ N(0, 1/K);
  5. the projection shapes of the largest model: 20480 x 6144 and 6144 x 20480.

The dense oracle W comes from the numpy oracle on the packed tensors; products are checked with
rel-RMS error <= 1e-2 (reference tolerance) and <= 4e-3 (fp32 accumulation + one bf16 rounding).
"""

import numpy as np
import pytest
import torch

import fdk_oracle as O
import fdk_oracle_torch as OT
from gpu_util import kmeans_like_codebook, from_bits, to_bits

pytestmark = pytest.mark.gpu

TOL = 1e-2  # src/fdk/kernels.py:196,502


def _oracle_dense(layer, bits: int, k: int) -> np.ndarray:
    """bf16 bit patterns of W from the module's packed tensors, on the CPU."""
    codes = layer.weight_data.cpu().numpy()
    scale = to_bits(layer.scale)
    lut = to_bits(layer.lut)
    if bits == 3:
        return O.dequantise_indices(O.unpack_indices(codes, 3, k), lut.reshape(-1), scale)
    return O.dequantise(codes, lut, scale)


def _expected(x: torch.Tensor, w_bits: np.ndarray) -> torch.Tensor:
    """x @ W.T on the CPU: products of bf16 values are exact in fp32, fp32 accumulation."""
    w = torch.from_numpy(O.bf16_to_f32(w_bits))
    return x.float().cpu() @ w.T


def _rmsen(expected: torch.Tensor, got: torch.Tensor) -> float:
    return (got.float().cpu() - expected).pow(2).sum().div(expected.pow(2).sum()).sqrt().item()


def test_config1_single_linear_4096():
    from fdk import models, native

    torch.manual_seed(100)
    linear = torch.nn.Linear(4096, 4096, bias=False)
    linear.weight.data = (torch.randn(4096, 4096) * 4096**-0.5).bfloat16().float()
    config = models.QuantisationConfig(bits=4, block_size=64)
    layer = models.quantise(linear, config, torch.device("cuda"), torch.bfloat16)
    assert isinstance(layer, models.QuantisedLinear)

    # the quantiser on the GPU gives what the CPU restatement of the reference's quantiser gives
    data, scale, table = OT.quantise_weight(linear.weight.data.bfloat16(), 4, 64)
    assert torch.equal(layer.weight_data.cpu(), data)
    assert np.array_equal(to_bits(layer.scale), to_bits(scale))
    assert np.array_equal(to_bits(layer.lut), to_bits(table))

    # dequantised W, bit for bit
    w_ref = O.dequantise(data.numpy(), to_bits(table), to_bits(scale))
    w = native.dequantise(layer.weight_data.data, layer.lut, layer.scale.data, 4)
    assert np.array_equal(to_bits(w), w_ref)
    assert np.array_equal(to_bits(native.dequantise_tiled(layer.tiled(), layer.lut, 4096, 4096, 4)), w_ref)

    for m in (1, 200):
        x = torch.randn((m, 4096), generator=torch.Generator().manual_seed(m)).bfloat16()
        expected = OT.mm_lut_ref(x, data, table, scale).float()  # the reference operator, on the CPU
        got = layer(x.cuda())
        torch.cuda.synchronize()
        assert got.shape == (m, 4096) and got.dtype == torch.bfloat16
        err = _rmsen(expected, got)
        assert err < TOL, f"m={m}: rmsen={err}"
    assert native.device_status() == 0


@pytest.mark.parametrize("bits", [1, 2, 3, 4])
@pytest.mark.parametrize("size", [3072, 4096, 6144, 8192])
def test_config2_kernel_sweep(size, bits):
    from fdk import models, native

    k = n = size
    gen = torch.Generator(device="cuda").manual_seed(size + bits)
    w = (torch.randn((n, k), generator=gen, device="cuda") * k**-0.5).bfloat16()
    codebook = from_bits(kmeans_like_codebook(bits, seed=bits))
    layer = models.QuantisedLinear.create(w, models.QuantisationConfig(bits, 64), lut=codebook)
    del w
    w_bits = _oracle_dense(layer, bits, k)
    assert np.array_equal(to_bits(native.dequantise_tiled(layer.tiled(), layer.lut, n, k, bits)), w_bits)
    x = torch.randn((16, k), generator=gen, device="cuda").bfloat16()
    expected = _expected(x, w_bits)
    for m in (1, 2, 4, 8, 16):
        got = layer(x[:m].contiguous())
        torch.cuda.synchronize()
        err = _rmsen(expected[:m], got)
        assert err < TOL, f"m={m}: rmsen={err}"
        assert err < 4e-3, f"m={m}: rmsen={err}"
    assert native.device_status() == 0


@pytest.mark.parametrize("n,k", [(20480, 6144), (6144, 20480)])
def test_config5_projection_shapes(n, k):
    from fdk import models, native

    bits = 4
    gen = torch.Generator(device="cuda").manual_seed(n)
    w = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).bfloat16()
    layer = models.QuantisedLinear.create(w, models.QuantisationConfig(bits, 64), lut=from_bits(kmeans_like_codebook(bits, 0)))
    del w
    w_bits = _oracle_dense(layer, bits, k)
    x = torch.randn((16, k), generator=gen, device="cuda").bfloat16()
    expected = _expected(x, w_bits)
    for m in (1, 4, 16):
        got = layer(x[:m].contiguous())
        torch.cuda.synchronize()
        err = _rmsen(expected[:m], got)
        assert err < 4e-3, f"m={m}: rmsen={err}"
    assert native.device_status() == 0
