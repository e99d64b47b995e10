"""CPU tests of the drop-in model API (fdk.models): the quantiser reproduces the reference's
packed tensors bit for bit, the torch.compile selector reproduces its outputs, the module
walker follows the reference's rules, and the accounting matches its formulas."""

import numpy as np
import pytest
import torch
from torch import nn

from fdk import models
from fdk.models import QuantisationConfig, QuantisedLinear, quantise


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16)


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


@pytest.mark.parametrize("bits", [8, 4, 2, 1])
def test_quantise_module_matches_reference(golden_dir, bits):
    z = np.load(golden_dir / "module_quantise.npz")
    ref_module = nn.Sequential(nn.Linear(384, 256, bias=False))
    with torch.no_grad():
        ref_module[0].weight.copy_(torch.from_numpy(z["weight_fp32"]))
    module = quantise(
        ref_module, QuantisationConfig(bits=bits, block_size=64, kernel="torch.compile"),
        device=torch.device("cpu"), dtype=torch.bfloat16,
    )
    q = module[0]
    p = f"b{bits}_"
    assert isinstance(q, QuantisedLinear)
    assert np.array_equal(q.weight_data.numpy(), z[p + "weight_data"])
    assert np.array_equal(_bits(q.scale.data), z[p + "scale"])
    assert np.array_equal(_bits(q.lut), z[p + "lut"])
    assert sorted(q.state_dict().keys()) == list(z[p + "state_keys"])
    y = module(torch.from_numpy(z["x_fp32"]).bfloat16())
    assert np.array_equal(_bits(y), z[p + "y"])
    assert models.count_ops(module) == int(z[p + "count_ops"])
    assert models.count_parameter_read_bytes(module) == int(z[p + "count_bytes"])
    assert q.bits == bits and q.block_size == 64
    # the source module is left untouched
    assert ref_module[0].weight.dtype == torch.float32


@pytest.mark.parametrize("bits", [4, 2])
def test_create_with_codebook_matches_reference(golden_dir, bits):
    z = np.load(golden_dir / "quantise_codebook.npz")
    p = f"b{bits}_"
    q = QuantisedLinear.create(_bf16(z[p + "w"]), QuantisationConfig(bits, 128, kernel="torch.compile"), lut=_bf16(z[p + "codebook"]))
    assert np.array_equal(q.weight_data.numpy(), z[p + "weight_data"])
    assert np.array_equal(_bits(q.scale.data), z[p + "scale"])
    assert np.array_equal(_bits(q.lut), z[p + "lut"])
    assert np.array_equal(_bits(q(_bf16(z[p + "x"]))), z[p + "y"])


def test_module_walker_rules():
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = nn.Linear(128, 64, bias=False)
            self.norm = nn.LayerNorm(64)
            self.lm_head = nn.Linear(64, 32, bias=False)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.body = Block()
            self.lm_head = nn.Linear(64, 32, bias=False)

    torch.manual_seed(0)
    src = Model()
    cfg = QuantisationConfig(4, 64, kernel="torch.compile")
    out = quantise(src, cfg, torch.device("cpu"), torch.bfloat16)
    assert isinstance(out.body.proj, QuantisedLinear)
    assert isinstance(out.lm_head, nn.Linear) and out.lm_head.weight.dtype == torch.bfloat16  # "^lm_head$" skipped
    assert isinstance(out.body.lm_head, QuantisedLinear)  # dotted key "body.lm_head" does not match
    assert out.body.norm.weight.dtype == torch.bfloat16
    # config None copies and casts only
    plain = quantise(src, None, torch.device("cpu"), torch.bfloat16)
    assert isinstance(plain.body.proj, nn.Linear)
    # a custom codebook reaches the top-level module only, as in the reference
    cb = torch.tensor([-1.0, -0.2, 0.3, 1.0]).bfloat16()
    top = quantise(nn.Linear(64, 16, bias=False), QuantisationConfig(2, 64, kernel="torch.compile"), torch.device("cpu"), torch.bfloat16, lut=cb)
    assert torch.equal(top.lut[:4, -1], cb)
    nested = quantise(nn.Sequential(nn.Linear(64, 16, bias=False)), QuantisationConfig(2, 64, kernel="torch.compile"), torch.device("cpu"), torch.bfloat16, lut=cb)
    assert torch.equal(nested[0].lut[:4, -1], torch.linspace(-1, 1, 4, dtype=torch.bfloat16))


def test_quantise_rejections():
    cfg = QuantisationConfig(4, 64)
    with pytest.raises(AssertionError, match="Bias"):
        quantise(nn.Linear(64, 8, bias=True), cfg, torch.device("cpu"), torch.bfloat16)
    with pytest.raises(AssertionError, match="multiple of 64"):
        quantise(nn.Linear(96, 8, bias=False), cfg, torch.device("cpu"), torch.bfloat16)

    class MyLinear(nn.Linear):
        pass

    with pytest.raises(AssertionError, match="subclasses"):
        quantise(MyLinear(64, 8, bias=False), cfg, torch.device("cpu"), torch.bfloat16)
    with pytest.raises(AssertionError, match="at most"):
        QuantisedLinear.create(torch.zeros(8, 64).bfloat16(), cfg, lut=torch.zeros(17).bfloat16())


def test_three_bit_extension_packs_as_the_oracle_defines():
    import fdk_oracle as O

    torch.manual_seed(3)
    w = (torch.randn(32, 128) * 0.1).bfloat16()
    q = QuantisedLinear.create(w, QuantisationConfig(3, 64, kernel="torch.compile"))
    assert q.weight_data.shape == (32, 48) and q.lut.shape == (8, 1) and q.bits == 3
    idx = O.unpack_indices(q.weight_data.numpy(), 3, 128)
    assert idx.max() <= 7
    # nearest-codebook assignment: dequantised weights sit within half a codebook step (x scale)
    w_hat = O.bf16_to_f32(O.dequantise_indices(idx, _bits(q.lut).reshape(-1), _bits(q.scale.data)))
    step = 2.0 / 7
    err = np.abs(w_hat - w.float().numpy()) / np.repeat(q.scale.float().numpy(), 64, axis=1)
    assert err.max() <= step / 2 + 0.02


def test_marlin_selector_numbers():
    torch.manual_seed(1)
    w = (torch.randn(64, 128) * 0.05).half()
    q = QuantisedLinear.create_marlin(w, QuantisationConfig(4, 64, kernel="marlin"))
    assert q.lut.dtype == torch.half and q.scale.dtype == torch.half
    assert torch.equal(q.lut[:16, -1], torch.arange(-8, 8).half())
    blocks = w.unflatten(-1, (-1, 64))
    assert torch.equal(q.scale.data, (blocks.abs().amax(-1) / 7).clamp_min(1e-12))


def test_llama_dims_match_reference(golden_dir):
    z = np.load(golden_dir / "llama_configs.npz")
    for key in ("4B", "12B", "31B"):
        d = models.get_custom_llama_dims(key)
        got = [d.hidden_size, d.num_hidden_layers, d.num_attention_heads, d.num_key_value_heads, d.intermediate_size, d.vocab_size, d.head_dim]
        assert got == list(z[key])
    d = models.get_custom_llama_dims("b200-31B")
    assert (d.hidden_size, d.num_hidden_layers, d.intermediate_size) == (6144, 64, 20480)


def test_quantisation_config_selector():
    cfgs = list(models._quantisation_configs([16, 4, 1], [64], ["triton", "marlin-lut"], "^lm_head$"))
    assert cfgs[0] is None
    assert [(c.bits, c.kernel) for c in cfgs[1:]] == [(4, "triton"), (4, "marlin-lut"), (1, "triton")]
