"""Regenerates tests/golden/*.npz by running the REFERENCE project on CPU.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/fused-dequantisation-kernels

The reference's Marlin extension is JIT-compiled at import and needs a GPU, so
a stub `fdk.marlin` module is registered first; nothing on the LUT path uses
it.  `mm_lut_ref` is evaluated eagerly (TORCHDYNAMO_DISABLE=1), as the paper
notebook of the reference does.  bf16 tensors are stored as uint16 bit
patterns so that tests can compare bit-for-bit.
"""

from __future__ import annotations

import os
import sys
import types
from pathlib import Path

os.environ["TORCHDYNAMO_DISABLE"] = "1"
sys.dont_write_bytecode = True

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bits_of(t: torch.Tensor) -> np.ndarray:
    assert t.dtype in (torch.bfloat16, torch.float16)
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main(ref_root: str) -> None:
    stub = types.ModuleType("fdk.marlin")

    class Layer(torch.nn.Module):
        pass

    stub.Layer = Layer
    sys.modules["fdk.marlin"] = stub
    sys.path.insert(0, str(Path(ref_root) / "src"))
    import fdk.kernels as K  # type: ignore
    import fdk.models as M  # type: ignore

    # ---- 1. quantiser + dequantise + matmul, default (linspace) codebook ----
    out: dict[str, np.ndarray] = {}
    n, k, g = 48, 256, 64
    for bits in (8, 4, 2, 1):
        torch.manual_seed(100 + bits)
        w = (torch.randn(n, k) * k**-0.5).bfloat16()
        q = M.QuantisedLinear.create(w, M.QuantisationConfig(bits, g, kernel="torch.compile"))
        x = torch.randn(5, k).bfloat16()
        wref = q.lut[q.weight_data.long()].flatten(1).view(n, k // g, g).mul(q.scale[:, :, None]).flatten(1)
        y = K.mm_lut_ref(x, q.weight_data, q.lut, q.scale)
        y1 = K.mm_lut_ref(x[0], q.weight_data, q.lut, q.scale)
        p = f"b{bits}_"
        out[p + "w"] = bits_of(w)
        out[p + "weight_data"] = q.weight_data.numpy().copy()
        out[p + "scale"] = bits_of(q.scale.data)
        out[p + "lut"] = bits_of(q.lut)
        out[p + "x"] = bits_of(x)
        out[p + "w_deq"] = bits_of(wref)
        out[p + "y"] = bits_of(y)
        out[p + "y_vec"] = bits_of(y1)
    np.savez_compressed(HERE / "quantise_linspace.npz", **out)

    # ---- 2. custom codebook (sorted, shorter than 2^bits -> right-padded), block 128 ----
    out = {}
    n, k, g = 32, 256, 128
    for bits in (4, 2):
        torch.manual_seed(7 + bits)
        w = (torch.randn(n, k) * 0.05).bfloat16()
        cb = torch.sort(torch.randn((1 << bits) - 1)).values.bfloat16()
        q = M.QuantisedLinear.create(w, M.QuantisationConfig(bits, g, kernel="torch.compile"), lut=cb)
        x = torch.randn(2, k).bfloat16()
        wref = q.lut[q.weight_data.long()].flatten(1).view(n, k // g, g).mul(q.scale[:, :, None]).flatten(1)
        p = f"b{bits}_"
        out[p + "w"] = bits_of(w)
        out[p + "codebook"] = bits_of(cb)
        out[p + "weight_data"] = q.weight_data.numpy().copy()
        out[p + "scale"] = bits_of(q.scale.data)
        out[p + "lut"] = bits_of(q.lut)
        out[p + "x"] = bits_of(x)
        out[p + "w_deq"] = bits_of(wref)
        out[p + "y"] = bits_of(K.mm_lut_ref(x, q.weight_data, q.lut, q.scale))
    np.savez_compressed(HERE / "quantise_codebook.npz", **out)

    # ---- 3. the reference's own kernel-test inputs (random bytes, rand scales) ----
    # kernels.py:185-196 builds these on the GPU; the same recipe on CPU, smaller n.
    out = {}
    n, k, g = 64, 4096, 64
    torch.manual_seed(42)
    a = torch.randn((3, k), dtype=torch.bfloat16)
    bq = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8)
    lut4 = torch.linspace(-1, 1, 16, dtype=torch.bfloat16)
    lut8 = torch.cartesian_prod(lut4, lut4)
    bs = torch.rand((n, k // g), dtype=torch.bfloat16)
    out["a"] = bits_of(a)
    out["bq"] = bq.numpy().copy()
    out["lut8"] = bits_of(lut8)
    out["bs"] = bits_of(bs)
    out["y"] = bits_of(K.mm_lut_ref(a, bq, lut8, bs))
    np.savez_compressed(HERE / "kernel_test_4b.npz", **out)

    # ---- 4. module-level: quantise(nn.Sequential(Linear(384, 256))) as test_quantise does ----
    out = {}
    for bits in (8, 4, 2, 1):
        torch.manual_seed(100)
        x = torch.randn((100, 384))
        ref_module = torch.nn.Sequential(torch.nn.Linear(384, 256, bias=False))
        module = M.quantise(
            ref_module,
            M.QuantisationConfig(bits=bits, block_size=64, kernel="torch.compile"),
            device=torch.device("cpu"),
            dtype=torch.bfloat16,
        )
        y = module(x.bfloat16())
        p = f"b{bits}_"
        if bits == 8:  # same seed for every bit width -> store the shared inputs once
            out["weight_fp32"] = ref_module[0].weight.detach().numpy().copy()
            out["x_fp32"] = x.numpy().copy()
            out["expected_fp32"] = ref_module(x).detach().numpy().copy()
        else:
            assert np.array_equal(out["weight_fp32"], ref_module[0].weight.detach().numpy())
        out[p + "weight_data"] = module[0].weight_data.numpy().copy()
        out[p + "scale"] = bits_of(module[0].scale.data)
        out[p + "lut"] = bits_of(module[0].lut)
        out[p + "y"] = bits_of(y)
        out[p + "count_ops"] = np.int64(M.count_ops(module))
        out[p + "count_bytes"] = np.int64(M.count_parameter_read_bytes(module))
        out[p + "state_keys"] = np.array(sorted(module[0].state_dict().keys()))
    np.savez_compressed(HERE / "module_quantise.npz", **out)

    # ---- 5. custom-llama configs resolved by the reference ----
    out = {}
    for key in M.custom_llama_configs:
        c = M.get_custom_llama_config(key)
        out[key] = np.array(
            [
                c.hidden_size,
                c.num_hidden_layers,
                c.num_attention_heads,
                c.num_key_value_heads,
                c.intermediate_size,
                c.vocab_size,
                c.head_dim,
            ],
            dtype=np.int64,
        )
    np.savez_compressed(HERE / "llama_configs.npz", **out)

    # ---- 6. Marlin packing: the reference's own Layer.pack on CPU ----
    # The reference module builds its CUDA extension when it is imported; the build is replaced
    # by a dummy so that the pure-Python packing code can run here.
    import importlib.util

    import torch.utils.cpp_extension as cpp_extension

    real_load = cpp_extension.load
    cpp_extension.load = lambda *a, **kw: types.SimpleNamespace()
    try:
        spec = importlib.util.spec_from_file_location("ref_marlin", Path(ref_root) / "src" / "fdk" / "marlin" / "__init__.py")
        ref_marlin = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref_marlin)
    finally:
        cpp_extension.load = real_load
    out = {}
    for name, (k, n, groupsize, is_linear) in {
        "g64_linear": (256, 256, 64, True), "g128_lut": (256, 512, 128, False), "single_linear": (128, 256, -1, True),
    }.items():
        torch.manual_seed(len(name))
        linear = torch.nn.Linear(k, n, bias=False, dtype=torch.half)
        g = k if groupsize == -1 else groupsize
        scale = (linear.weight.data.unflatten(-1, (-1, g)).abs().amax(dim=-1) / 7).clamp_min_(1e-12)
        layer = ref_marlin.Layer(k, n, groupsize=groupsize, is_linear=is_linear)
        layer.pack(linear, scale)
        out[name + "_weight"] = bits_of(linear.weight.data)
        out[name + "_scale"] = bits_of(scale)
        out[name + "_B"] = layer.B.numpy().copy()
        out[name + "_s"] = bits_of(layer.s)
    np.savez_compressed(HERE / "marlin_pack.npz", **out)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
