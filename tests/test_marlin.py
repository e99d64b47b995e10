"""The Marlin selector surface (fdk.marlin: Layer, pack, mul, import_marlin) against the reference's
own packing, run on CPU when tests/golden/marlin_pack.npz was generated
(src/fdk/marlin/__init__.py:57-87, 152-189): `pack` reproduces B and s bit for bit, and
`import_marlin` turns them into codes and scales whose dequantised weight is Marlin's
(q - 8) * s exactly.  The product itself (GPU) is checked against an fp16 torch matmul."""

import numpy as np
import pytest
import torch

import fdk_oracle as O
from fdk import marlin, models

CASES = {"g64_linear": (256, 256, 64, True), "g128_lut": (256, 512, 128, False), "single_linear": (128, 256, -1, True)}


def _half(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.half)


@pytest.mark.parametrize("name", list(CASES))
def test_pack_reproduces_the_reference_format(golden_dir, name):
    k, n, groupsize, is_linear = CASES[name]
    z = np.load(golden_dir / "marlin_pack.npz")
    linear = torch.nn.Linear(k, n, bias=False, dtype=torch.half)
    linear.weight.data = _half(z[name + "_weight"])
    layer = marlin.Layer(k, n, groupsize=groupsize, is_linear=is_linear)
    layer.pack(linear, _half(z[name + "_scale"]))
    assert np.array_equal(layer.B.numpy(), z[name + "_B"])
    assert np.array_equal(layer.s.view(torch.int16).numpy().view(np.uint16), z[name + "_s"])
    assert sorted(layer.state_dict()) == (["B", "s"] if is_linear else ["B", "centroids", "s"])


@pytest.mark.parametrize("name", list(CASES))
def test_import_gives_marlins_weights_bit_for_bit(golden_dir, name):
    k, n, groupsize, is_linear = CASES[name]
    g = k if groupsize == -1 else groupsize
    z = np.load(golden_dir / "marlin_pack.npz")
    codes, scales = marlin.import_marlin(torch.from_numpy(z[name + "_B"]), _half(z[name + "_s"]), is_linear=is_linear)
    assert codes.shape == (n, k // 2) and scales.shape == (n, k // g)
    # the scales come back in their own order
    assert np.array_equal(scales.view(torch.int16).numpy().view(np.uint16), z[name + "_scale"])
    # codes: q = round(w / s) + 8 clamped, two consecutive K elements per byte, the first in the high nibble
    w, s = _half(z[name + "_weight"]), _half(z[name + "_scale"])
    q = torch.round(w / s.repeat_interleave(g, dim=1)).int().add(8).clamp(0, 15)
    assert torch.equal(codes, (q[:, 0::2] * 16 + q[:, 1::2]).to(torch.uint8))
    # dequantised through the byte table = (q - 8) * s in fp16
    table = marlin.byte_table(None, "cpu")
    dense = O.dequantise(codes.numpy(), table.view(torch.int16).numpy().view(np.uint16),
                         scales.view(torch.int16).numpy().view(np.uint16), dtype="f16")
    want = ((q - 8).half() * s.repeat_interleave(g, dim=1))
    assert np.array_equal(dense, want.view(torch.int16).numpy().view(np.uint16))


def test_lookup_table_of_the_lut_variant_is_reindexed():
    """Marlin indexes its [256, 2] table with the second element in the high nibble."""
    values = torch.arange(-8, 8, dtype=torch.half)
    reference_table = torch.cartesian_prod(values, values).flip(1)  # what the reference stores (models.py:117-119)
    assert torch.equal(marlin.byte_table(reference_table, "cpu"), marlin.byte_table(None, "cpu"))


def test_layer_rejects_what_the_reference_rejects():
    with pytest.raises(ValueError):
        marlin.Layer(256, 256, groupsize=32)
    with pytest.raises(ValueError):
        marlin.Layer(192, 256)
    with pytest.raises(ValueError):
        marlin.Layer(256, 128)
    layer = marlin.Layer(256, 256, groupsize=64)
    with pytest.raises(ValueError):
        layer.pack(torch.nn.Linear(256, 256, bias=False), torch.ones(256, 4))  # fp32 weights


def test_load_kmeans_state_dict_fills_quantised_layers():
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(128, 64, bias=False), torch.nn.LayerNorm(64))
    cfg = models.QuantisationConfig(2, 64, kernel="torch.compile")
    target = models.quantise(net, cfg, torch.device("cpu"), torch.bfloat16)
    codebook = torch.tensor([-1.5, -0.4, 0.3, 1.6], dtype=torch.bfloat16)
    trained = models.QuantisedLinear.create(torch.randn(64, 128).bfloat16(), cfg, lut=codebook)
    state = {"0.weight_data": trained.weight_data.data, "0.scale": trained.scale.data, "0.lut": codebook,
             "1.weight": torch.full((64,), 2.0), "1.bias": torch.zeros(64)}
    assert models.load_kmeans_state_dict(target, state) == ["0"]
    assert torch.equal(target[0].weight_data, trained.weight_data) and torch.equal(target[0].lut, trained.lut)
    assert torch.equal(target[1].weight, torch.full((64,), 2.0, dtype=torch.bfloat16))
    x = torch.randn(3, 128).bfloat16()
    assert torch.equal(target[0](x), trained(x))


@pytest.mark.gpu
@pytest.mark.parametrize("kernel,m", [("marlin", 1), ("marlin", 24), ("marlin-lut", 3), ("marlin-lut", 200)])
def test_quantise_returns_a_marlin_layer_and_its_product_is_right(kernel, m):
    torch.manual_seed(1)
    linear = torch.nn.Linear(512, 768, bias=False)
    cfg = models.QuantisationConfig(4, 64, kernel=kernel)
    layer = models.quantise(linear, cfg, torch.device("cuda"), torch.half)
    assert isinstance(layer, marlin.Layer) and layer.is_linear == (kernel == "marlin")
    assert models.count_ops(layer) == 2 * 512 * 768
    assert models.count_parameter_read_bytes(layer) == 768 * 512 // 2 + 768 * 8 * 2
    w = linear.weight.data.half().cuda()
    s = (w.unflatten(-1, (-1, 64)).abs().amax(-1) / 7).clamp_min(1e-12)
    q = torch.round(w / s.repeat_interleave(64, dim=1)).add(8).clamp(0, 15)
    dense = (q - 8) * s.repeat_interleave(64, dim=1)  # fp16, Marlin's dequantised weight
    x = torch.randn((m, 512), device="cuda").half()
    want = x.float() @ dense.float().T
    got = layer(x).float()
    err = (got - want).pow(2).sum().div(want.pow(2).sum()).sqrt().item()
    assert err < 2e-3, f"rel-RMS error {err}"
    # a table of the lookup variant that is not the linear grid is honoured too
    if kernel == "marlin-lut":
        table = torch.randn((256, 2), device="cuda").half()
        layer.centroids.copy_(table)
        codes = (q[:, 0::2] * 16 + q[:, 1::2]).long()          # first element in the high nibble
        swapped = (codes % 16) * 16 + codes // 16                 # Marlin's index: second element high
        dense2 = (table[swapped].flatten(1) * s.repeat_interleave(64, dim=1)).float()
        got2 = layer(x).float()
        want2 = x.float() @ dense2.T
        assert (got2 - want2).pow(2).sum().div(want2.pow(2).sum()).sqrt().item() < 2e-3
