"""Model-level quantisation -- drop-in for the reference's src/fdk/models.py on the LUT path.

Same surface: QuantisationConfig, QuantisedLinear (create / forward / state_dict keys
weight_data, scale, lut), quantise(), Generator, count_ops, count_parameter_read_bytes,
the custom-llama configs and the `python -m fdk.models` selector.  What differs is below
the operator boundary: the `triton` kernel selector runs the native sm_100a kernels of
libfdk_b200 on a tiled copy of the packed weights built once per module.

Kernel selectors (QuantisationConfig.kernel):
  "triton"         native fused kernel (name kept so existing configs keep working); bf16
  "torch.compile"  the torch reference, dequantise then matmul (eager here)
  "marlin", "marlin-lut"  the reference's fp16 4-bit selectors (models.py:107-125): same
                   numbers (scale = absmax / 7, codes = round(w / s) + 8 clamped, values
                   arange(-8, 8)), run by the same native kernel in its fp16 instantiation.
"""

from __future__ import annotations

import copy
import re
import sys
from dataclasses import dataclass
from typing import Iterable, Literal

import torch
from torch import Tensor, nn

from . import kernels, native

# Quantised models


@dataclass
class QuantisationConfig:
    bits: int
    block_size: int
    kernel: Literal["triton", "torch.compile", "marlin", "marlin-lut"] = "triton"
    skip: str | None = "^lm_head$"


def _pack_codes(indices: Tensor, bits: int) -> Tensor:
    """[N, K] integer codes -> packed uint8 rows, first element of a byte in the high bits."""
    n, k = indices.shape
    idx = indices.to(torch.uint8)
    if 8 % bits == 0:
        per_byte = 8 // bits
        place = 2 ** torch.arange(0, 8, bits, device=idx.device, dtype=torch.uint8).flip(0)
        return idx.unflatten(-1, (-1, per_byte)).mul(place).sum(-1, dtype=torch.uint8)
    # 3 bits: one MSB-first bit stream per row
    shifts = torch.arange(bits - 1, -1, -1, device=idx.device, dtype=torch.uint8)
    stream = ((idx[..., None] >> shifts) & 1).reshape(n, k * bits // 8, 8)
    place = 2 ** torch.arange(7, -1, -1, device=idx.device, dtype=torch.uint8)
    return stream.mul(place).sum(-1, dtype=torch.uint8)


class QuantisedLinear(nn.Module):
    def __init__(
        self,
        in_features: int,
        out_features: int,
        weight_data: Tensor,
        scale: Tensor,
        lut: Tensor,
        kernel: Literal["triton", "torch.compile", "marlin", "marlin-lut"],
    ):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight_data = nn.Parameter(weight_data, requires_grad=False)
        self.scale = nn.Parameter(scale, requires_grad=False)
        self.lut = nn.Buffer(lut)
        self.kernel = kernel
        self._tiled: Tensor | None = None  # derived from the three tensors above, never saved
        self._tiled_key: tuple | None = None

    @property
    def bits(self) -> int:
        return kernels.bits_of_lut(self.lut)

    @property
    def block_size(self) -> int:
        return self.in_features // self.scale.shape[1]

    def tiled(self) -> Tensor:
        """The kernels' tiled copy of (weight_data, scale); rebuilt when they change or move."""
        key = (
            self.weight_data.data_ptr(), self.scale.data_ptr(),
            self.weight_data._version, self.scale._version, str(self.weight_data.device),
        )
        if self._tiled is None or self._tiled_key != key:
            self._tiled = native.repack(
                self.weight_data.data, self.scale.data, self.out_features, self.in_features,
                self.bits, self.block_size,
            )
            self._tiled_key = key
        return self._tiled

    def lut_bytes(self) -> bytes:
        """Host copy of the table (made once): it travels with the kernel's launch parameters."""
        key = (self.lut.data_ptr(), self.lut._version)
        if getattr(self, "_lut_host_key", None) != key:
            self._lut_host = native.host_lut(self.lut)
            self._lut_host_key = key
        return self._lut_host

    def forward(self, x: Tensor) -> Tensor:
        if x.ndim > 2:
            return self.forward(x.flatten(end_dim=-2)).unflatten(0, x.shape[:-1])
        if self.kernel == "torch.compile":
            return kernels.mm_lut_ref(x, self.weight_data, self.lut, self.scale)
        assert self.kernel in ("triton", "marlin", "marlin-lut")
        out = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=x.dtype)
        assert x.dtype == self.lut.dtype == self.scale.dtype
        native.linear_lut(
            x.contiguous(), self.tiled(), self.lut, out, self.out_features, self.in_features, self.bits,
            pdl=True, lut_bytes=self.lut_bytes(),
        )
        return out

    def forward_silu_pairs(self, x: Tensor, out: Tensor) -> None:
        """For a fused gate|up projection whose rows alternate 32 gate rows and their 32 up rows:
        out[m, n / 2] = silu(gate) * up, in the projection kernel itself up to 16 rows."""
        assert x.ndim == 2 and self.out_features % 64 == 0
        if self.kernel != "torch.compile" and x.shape[0] <= 16:
            native.linear_lut(
                x.contiguous(), self.tiled(), self.lut, out, self.out_features, self.in_features, self.bits,
                pdl=True, lut_bytes=self.lut_bytes(), silu_pairs=True,
            )
        else:
            native.silu_mul(self.forward(x), out, group=32)

    def fused(self, x: Tensor | None, out: Tensor | None, rows: int, fusion: "native.LinearFusion",
              silu_pairs: bool = False) -> None:
        """The projection with the decode-step fusions of `fusion` (RMSNorm on the input side;
        residual add or rotary embedding + KV append on the output side): bf16, up to 16 rows."""
        assert self.kernel != "torch.compile" and rows <= 16
        native.linear_lut_fused(
            x, self.tiled(), self.lut, out, rows, self.out_features, self.in_features, self.bits, fusion,
            pdl=True, lut_bytes=self.lut_bytes(), silu_pairs=silu_pairs,
        )

    def push(self, x: Tensor, exchange: "native.TpExchange") -> None:
        """Row-parallel use in tensor-parallel decode: this rank's partial product goes straight
        into every rank's exchange buffer (no output tensor); native.rmsnorm_reduce sums them."""
        assert x.ndim == 2 and self.kernel != "torch.compile"
        native.linear_lut_push(
            x.contiguous(), self.tiled(), self.lut, exchange, self.out_features, self.in_features, self.bits,
            pdl=True, lut_bytes=self.lut_bytes(),
        )

    @classmethod
    def create(cls, weight: Tensor, c: QuantisationConfig, lut: Tensor | None = None) -> "QuantisedLinear":
        device = weight.device
        n_codes = 2**c.bits
        if lut is not None:
            assert lut.ndim == 1 and lut.shape[0] <= n_codes, f"lut must have at most {n_codes} entries, got {lut.shape[0]}"
            lut = nn.functional.pad(lut, (0, n_codes - lut.shape[0]), value=lut[-1])
        else:
            lut = torch.linspace(-1, 1, steps=n_codes, device=device, dtype=weight.dtype)  # uniform [-1, 1]

        # one scale per block_size run of the input dimension
        blocks = weight.unflatten(-1, (-1, c.block_size))
        scale = blocks.abs().mean(dim=-1) if c.bits <= 2 else blocks.abs().amax(dim=-1)
        scale.clamp_min_(1e-12)
        scaled = (blocks / scale[..., None]).flatten(-2)

        # nearest codebook entry = bucket between codebook midpoints
        indices = torch.bucketize(scaled, (lut[1:] + lut[:-1]) / 2).clamp_(0, n_codes - 1)
        weight_data = _pack_codes(indices, c.bits)
        if 8 % c.bits == 0:
            table = torch.cartesian_prod(*([lut] * (8 // c.bits))).view(256, -1)
        else:
            table = lut.reshape(n_codes, 1)
        return cls(*weight.T.shape, weight_data, scale, table, kernel=c.kernel)

    @classmethod
    def create_marlin(cls, weight: Tensor, c: QuantisationConfig) -> "QuantisedLinear":
        """The reference's Marlin selectors as numbers (models.py:107-125, marlin/__init__.py:152-189):
        fp16, 4 bits, scale = absmax / 7, code = round(w / scale) + 8 clamped to [0, 15],
        value = code - 8."""
        assert c.bits == 4, "Marlin backend only supports 4-bit quantisation"
        assert c.block_size in (64, 128), "Marlin backend requires block_size 64 or 128"
        assert weight.dtype == torch.half, "Marlin backend requires float16 weights"
        blocks = weight.unflatten(-1, (-1, c.block_size))
        scale = blocks.abs().amax(dim=-1) / 7
        scale.clamp_min_(1e-12)
        codes = torch.round(blocks / scale[..., None]).add_(8).clamp_(0, 15).flatten(-2)
        values = torch.arange(-8, 8, dtype=torch.half, device=weight.device)
        table = torch.cartesian_prod(values, values).view(256, -1)
        return cls(*weight.T.shape, _pack_codes(codes, 4), scale, table, kernel=c.kernel)


def quantise(
    source: nn.Module,
    config: QuantisationConfig | None,
    device: torch.device,
    dtype: torch.dtype,
    key: tuple[str, ...] = (),
    lut: Tensor | None = None,
) -> nn.Module:
    """Quantise all nn.Linear layers in a module according to config, returning a new
    quantised module.  The original module is left untouched; parameter sharing is lost.
    As in the reference, `lut` applies to `source` itself only, not to its children."""
    should_quantise = (
        isinstance(source, nn.Linear)
        and config is not None
        and (config.skip is None or not re.search(config.skip, ".".join(key)))
    )
    if should_quantise:
        assert type(source) == nn.Linear, f"nn.Linear subclasses are not supported: {type(source)}"
        assert source.bias is None, "Bias is unsupported"
        assert source.in_features % 64 == 0, f"in_features must be multiple of 64, got {source.in_features}"
        weight = source.weight.data.to(device, dtype)
        if config.kernel.startswith("marlin"):
            module: nn.Module = QuantisedLinear.create_marlin(weight, config)
        else:
            module = QuantisedLinear.create(weight, config, lut=lut)
    else:
        # shallow copy of the module object, fresh containers, own tensors moved
        module = copy.copy(source)
        module._modules = {}
        module._parameters = {}
        module._buffers = {}
        for name, p in source._parameters.items():
            module._parameters[name] = (
                None if p is None else nn.Parameter(p.to(device=device, dtype=dtype), requires_grad=p.requires_grad)
            )
        for name, b in source._buffers.items():
            module._buffers[name] = None if b is None else b.to(device=device, dtype=dtype)

    for name, m in source._modules.items():
        module._modules[name] = None if m is None else quantise(m, config, device, dtype, key + (name,))
    return module


# Benchmarking helpers


def count_ops(model: nn.Module) -> int:
    """Approximate ops per token, respecting quantised layers (ignoring attention)."""
    ops = 0
    for module in model.modules():
        if isinstance(module, QuantisedLinear):
            ops += 2 * module.in_features * module.out_features
        else:
            ops += sum(2 * p.numel() for p in module.parameters(recurse=False))
    return ops


def count_parameter_read_bytes(model: nn.Module) -> int:
    """Approximate bytes read per token: every parameter except embeddings; the lookup
    table is a buffer and is not counted."""
    bytes_r = 0
    for module in model.modules():
        if isinstance(module, nn.Embedding):
            continue
        bytes_r += sum(p.numel() * p.element_size() for p in module.parameters(recurse=False))
    return bytes_r


@dataclass
class Result:
    batch_size: int
    bytes_rw: int
    ops: int
    avg_time: float
    avg_time_stderr: float
    output: list[str]

    def __str__(self) -> str:
        bandwidth = self.bytes_rw / self.avg_time / 1e9
        ops_per_s = self.ops / self.avg_time / 1e12
        return "  ".join(
            [
                f"{self.batch_size / self.avg_time:>6.1f} tokens/s",
                f"{bandwidth:>6.1f} GB/s",
                f"{ops_per_s:>6.1f} TFLOPS",
            ]
        )


# Custom model configs (the reference's own shapes, models.py:345-379, plus the
# shapes the B200 measurements are quoted on)

custom_llama_configs = {
    "4B": dict(dim=3072, n_layers=24, n_heads=24, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024, rope_theta=500000),
    "12B": dict(dim=4096, n_layers=48, n_heads=32, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024, rope_theta=500000),
    "31B": dict(dim=6144, n_layers=60, n_heads=48, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024, rope_theta=500000),
}

# explicit FFN widths: 32 x 3072 / 8192, 40 x 5120 / 13824, 64 x 6144 / 20480
b200_llama_configs = {
    "b200-4B": dict(dim=3072, n_layers=32, n_heads=24, n_kv_heads=8, intermediate_size=8192, rope_theta=500000),
    "b200-12B": dict(dim=5120, n_layers=40, n_heads=40, n_kv_heads=8, intermediate_size=13824, rope_theta=500000),
    "b200-31B": dict(dim=6144, n_layers=64, n_heads=48, n_kv_heads=8, intermediate_size=20480, rope_theta=500000),
}


@dataclass
class LlamaDims:
    """Plain description of a Llama-style decoder (what get_custom_llama_config resolves to)."""

    name: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int = 128256
    head_dim: int = 128
    rope_theta: float = 500000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False


def get_custom_llama_dims(key: str) -> LlamaDims:
    if key in b200_llama_configs:
        c = b200_llama_configs[key]
        inter = c["intermediate_size"]
    else:
        c = custom_llama_configs[key]
        multiple_of = c["multiple_of"]
        inter = multiple_of * ((int(4 * 2 / 3 * c["dim"] * c["ffn_dim_multiplier"]) + multiple_of - 1) // multiple_of)
    return LlamaDims(
        name=f"custom-llama-{key}",
        hidden_size=c["dim"],
        num_hidden_layers=c["n_layers"],
        num_attention_heads=c["n_heads"],
        num_key_value_heads=c["n_kv_heads"],
        intermediate_size=inter,
        rope_theta=c["rope_theta"],
    )


def get_custom_llama_config(key: str):
    """transformers LlamaConfig for a custom-llama size (needs `transformers`)."""
    import transformers

    d = get_custom_llama_dims(key)
    return transformers.models.llama.modeling_llama.LlamaConfig(
        _name_or_path=d.name,
        vocab_size=d.vocab_size,
        hidden_size=d.hidden_size,
        num_hidden_layers=d.num_hidden_layers,
        num_attention_heads=d.num_attention_heads,
        num_key_value_heads=d.num_key_value_heads,
        intermediate_size=d.intermediate_size,
        rope_theta=d.rope_theta,
        dtype=torch.bfloat16,
        tie_word_embeddings=d.tie_word_embeddings,
    )


def _quantisation_configs(
    bits: list[int], block_sizes: list[int], kernels_: list[str], skip: str
) -> Iterable[QuantisationConfig | None]:
    if 16 in bits:
        yield None  # 16-bit (no quantisation)
    for b in bits:
        if b < 16:
            for block_size in block_sizes:
                for kernel in kernels_:
                    if not (kernel.startswith("marlin") and b != 4):
                        yield QuantisationConfig(bits=b, block_size=block_size, kernel=kernel, skip=skip)


# Decode benchmark (the reference's `benchmark` / `run_benchmark` / `_main`, models.py:313-605,
# on the native decode loop of fdk.llama; random token ids stand in for the tokenizer, which
# needs a gated download)


@dataclass
class BenchmarkSettings:
    model: str
    batch_size: int
    quantisation: QuantisationConfig | None
    reps: int
    context: int = 2
    tp: int = 1

    def __str__(self) -> str:
        q = (
            f"b={self.quantisation.block_size} {self.quantisation.bits}-bit {self.quantisation.kernel}"
            if self.quantisation is not None
            else "16-bit"
        )
        return f"{self.model} batch={self.batch_size} ctx={self.context} tp={self.tp} {q}"


def benchmark(model: nn.Module, batch_size: int, reps: int, context: int = 2, seed: int = 0) -> Result:
    """Seconds per decode step of `model` (an fdk.llama.LlamaDecoder): one step per CUDA-graph
    replay, `reps` replays, as the reference does; `context` tokens of synthetic KV cache."""
    from . import bench, llama

    device = model.final_norm.device
    gen = torch.Generator(device=device).manual_seed(seed)
    prompt_ids = torch.randint(0, model.dims.vocab_size, (batch_size, 1), generator=gen, device=device)
    with torch.no_grad():
        generator = llama.Generator(model, prompt_ids, reps + 4, synthetic_context=max(context, 1))
        avg_time, avg_time_stderr = bench.measure_time(lambda _: generator.step(), inner_reps=1, outer_reps=reps)
    return Result(
        batch_size=batch_size,
        bytes_rw=count_parameter_read_bytes(model),
        ops=batch_size * count_ops(model),
        avg_time=avg_time,
        avg_time_stderr=avg_time_stderr,
        output=[],
    )


def resolve_model_dims(name: str) -> LlamaDims:
    """'custom-llama-4B' (reference shapes) or 'custom-llama-b200-4B' (the B200 measurement shapes)."""
    assert name.startswith("custom-llama-"), f"only custom-llama-* models are built offline, got {name}"
    return get_custom_llama_dims(name.replace("custom-llama-", ""))


def _main() -> None:
    import argparse
    import os

    import torch.distributed as dist

    from . import bench, llama

    parser = argparse.ArgumentParser()
    parser.add_argument("--model", default=["custom-llama-4B"], nargs="+",
                        help=f"custom-llama-<size>, sizes {list(custom_llama_configs) + list(b200_llama_configs)}")
    parser.add_argument("--batch-size", default=[1], type=int, nargs="+", help="Generation batch sizes")
    parser.add_argument("--bits", default=[16, 4, 1], type=int, nargs="+", help="Quantisation bit widths")
    parser.add_argument("--skip", default="^lm_head$", help="Regex of parameters to skip during quantisation")
    parser.add_argument("--block-size", default=[64], type=int, nargs="+", help="Quantisation block sizes")
    parser.add_argument("--kernel", default=["triton"], choices=["triton", "torch.compile", "marlin", "marlin-lut"],
                        nargs="+", help="Kernel implementation(s) (ignored for 16-bit)")
    parser.add_argument("--reps", type=int, default=100, help="Number of generation steps to measure")
    parser.add_argument("--context", type=int, default=2, help="Tokens already in the KV cache")
    parser.add_argument("--tp-reduce", default="fused", choices=["fused", "nccl"],
                        help="Under torchrun: how the row-parallel projections' partial sums are added "
                             "(fused = pushed from the kernel over NVLink, batches up to 16; else NCCL)")
    args = parser.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    tp = llama.TensorParallel(rank, world, None, fused=args.tp_reduce == "fused")

    log = bench.Log("models") if rank == 0 else None
    for name in args.model:
        dims = resolve_model_dims(name)
        for batch_size in args.batch_size:
            for config in _quantisation_configs(args.bits, args.block_size, args.kernel, args.skip):
                if config is not None and config.kernel.startswith("marlin"):
                    continue  # fp16 selectors are exercised at layer level, the decode loop is bf16
                settings = BenchmarkSettings(name, batch_size, config, args.reps, args.context, world)
                out = dict(**settings.__dict__)
                if config is not None:
                    out.update(config.__dict__)
                del out["quantisation"]
                try:
                    model = llama.LlamaDecoder.random_init(dims, config, device, tp)
                    result = benchmark(model, batch_size, args.reps, args.context)
                    out.update(result.__dict__)
                    if rank == 0:
                        print(f"{str(settings):>60}:  {result}", file=sys.stderr)
                    if getattr(model, "exchange", None) is not None:
                        out.update(tp_reduce="fused", exchange_status=native.tp_exchange_status(model.exchange))
                    model.close()
                    del model
                except Exception as e:  # as the reference: log and carry on
                    out.update(error=repr(e))
                    if rank == 0:
                        print(f"{str(settings):>60}:  ERROR {e}", file=sys.stderr)
                torch.cuda.empty_cache()
                if log is not None:
                    log(out)
    if world > 1:
        # captured graphs that hold collectives must be gone before the communicator is
        import gc

        gc.collect()
        torch.cuda.synchronize()
        dist.destroy_process_group()


if __name__ == "__main__":
    _main()
