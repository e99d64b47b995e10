"""Model-level quantisation -- drop-in for the reference's src/fdk/models.py on the LUT path.

Same surface: QuantisationConfig, QuantisedLinear (create / forward / state_dict keys
weight_data, scale, lut), quantise(), Generator, count_ops, count_parameter_read_bytes,
the custom-llama configs and the `python -m fdk.models` selector.  What differs is below
the operator boundary: the `triton` kernel selector runs the native sm_100a kernels of
libfdk_b200 on a tiled copy of the packed weights built once per module.

Kernel selectors (QuantisationConfig.kernel):
  "triton"         native fused kernel (name kept so existing configs keep working); bf16
  "torch.compile"  the torch reference, dequantise then matmul (eager here)
  "marlin", "marlin-lut"  the reference's fp16 4-bit selectors (models.py:107-125): quantise()
                   returns an `fdk.marlin.Layer` holding Marlin-format tensors (scale = absmax / 7,
                   codes = round(w / s) + 8 clamped, values arange(-8, 8)); its product runs on
                   the same native kernel in its fp16 instantiation.
"""

from __future__ import annotations

import copy
import re
import sys
from dataclasses import dataclass
from typing import Iterable, Literal

import torch
from torch import Tensor, nn

from . import kernels, marlin, native

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

    def forward_host(self, x_host: Tensor, out_host: Tensor | None = None, synchronise: bool = True) -> Tensor:
        """The forward for activations that live in host memory: x_host [m, in_features] (page-locked
        for asynchronous copies) -> out_host [m, out_features], valid on return.  One library call
        does the copy in, the projection, the copy out and the stream synchronisation, instead of
        `layer(x_host.to(device)).cpu()` (three framework calls and their bookkeeping around an
        11 us kernel).  synchronise=False returns at once: out_host is valid after the caller has
        synchronised the current stream, x_host must stay untouched until then, and further calls
        may be queued meanwhile (their copies and kernels then overlap the host's work)."""
        assert self.kernel != "torch.compile" and x_host.ndim == 2 and not x_host.is_cuda
        m = x_host.shape[0]
        if out_host is None:
            out_host = torch.empty((m, self.out_features), dtype=x_host.dtype).pin_memory()
        assert x_host.shape[1] == self.in_features and x_host.is_contiguous() and x_host.dtype == self.lut.dtype
        assert out_host.shape == (m, self.out_features) and out_host.is_contiguous() and out_host.dtype == x_host.dtype
        tiled = self.tiled()
        key = (m, id(tiled), torch.cuda.current_stream(tiled.device).cuda_stream, synchronise)
        calls = self.__dict__.setdefault("_host_calls", {})
        call = calls.get(key)
        if call is None:  # staging buffers and the bound library call, once per batch size and stream
            x_dev = torch.empty(m * self.in_features, dtype=x_host.dtype, device=tiled.device)
            out_dev = torch.empty(m * self.out_features, dtype=x_host.dtype, device=tiled.device)
            call = native.prepare_linear_lut_host(tiled, self.lut, self.lut_bytes(), x_dev, out_dev, m, self.out_features,
                                                  self.in_features, self.bits, x_host.dtype, synchronise)
            if len(calls) >= 4:  # a changed weight or stream leaves stale entries behind
                calls.clear()
            calls[key] = call
        call(x_host.data_ptr(), out_host.data_ptr())
        return out_host

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


def _create_marlin_layer(weight: Tensor, c: QuantisationConfig) -> nn.Module:
    """The reference's Marlin selectors (models.py:107-125): an `fdk.marlin.Layer` packed from the
    fp16 weight, with the linear grid as lookup table for the "marlin-lut" variant too."""
    assert c.bits == 4, "Marlin backend only supports 4-bit quantisation"
    assert c.block_size in (64, 128), "Marlin backend requires block_size 64 or 128"
    assert weight.dtype == torch.half, "Marlin backend requires float16 weights"
    out_features, in_features = weight.shape
    layer = marlin.Layer(in_features, out_features, groupsize=c.block_size,
                         is_linear={"marlin": True, "marlin-lut": False}[c.kernel]).to(weight.device)
    if not layer.is_linear:
        centroids = torch.arange(-8, 8, dtype=torch.half, device=weight.device)
        layer.centroids[...] = torch.cartesian_prod(centroids, centroids).flip(1)
    scale = weight.unflatten(-1, (-1, c.block_size)).abs().amax(dim=-1) / 7
    scale.clamp_min_(1e-12)
    source = nn.Linear(in_features, out_features, bias=False, device="meta")
    source.weight = nn.Parameter(weight, requires_grad=False)
    layer.pack(source, scale)
    return layer


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
            module: nn.Module = _create_marlin_layer(weight, config)
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
        elif isinstance(module, marlin.Layer):
            ops += 2 * module.k * module.n
        else:
            ops += sum(2 * p.numel() for p in module.parameters(recurse=False))
    return ops


def count_parameter_read_bytes(model: nn.Module) -> int:
    """Approximate bytes read per token: every parameter except embeddings; the lookup
    table is a buffer and is not counted."""
    bytes_r = 0
    for module in model.modules():
        if isinstance(module, marlin.Layer):  # elements and scales only, like QuantisedLinear
            bytes_r += sum(b.numel() * b.element_size() for b in (module.B, module.s))
        elif isinstance(module, nn.Embedding):
            continue
        else:
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
    model.check_status()  # a timed-out wait inside the timed steps would make the number meaningless
    return Result(
        batch_size=batch_size,
        bytes_rw=count_parameter_read_bytes(model),
        ops=batch_size * count_ops(model),
        avg_time=avg_time,
        avg_time_stderr=avg_time_stderr,
        output=[],
    )


def _estimate_fits_on_device(settings: BenchmarkSettings, device: torch.device, dtype: torch.dtype) -> bool:
    """The reference's pre-check (models.py:438-453): parameters from the model name's size
    suffix times bytes per parameter against 80 % of the device memory."""
    _, total_mem_bytes = torch.cuda.mem_get_info(device.index)
    if m := re.search(r"(\d[0-9.]*)[bB]$", settings.model):
        bytes_per_param = (
            dtype.itemsize
            if settings.quantisation is None
            else settings.quantisation.bits / 8 + dtype.itemsize / settings.quantisation.block_size
        )
        if settings.quantisation is not None and settings.quantisation.kernel != "torch.compile":
            bytes_per_param *= 2  # the packed tensors and their tiled copy
        return float(m[1]) * 1e9 * bytes_per_param / max(settings.tp, 1) < total_mem_bytes * 0.8
    print(f"No size for model {settings.model} - assuming it fits", file=sys.stderr)
    return True


def load_host_model(model_name: str):
    """transformers model in fp32 on the host, as the reference loads it (models.py:461-473):
    custom-llama-* from its config (random weights), anything else from a local Hugging Face
    checkpoint.  The tokenizer is attached when it can be had without a download."""
    import transformers

    if model_name.startswith("custom-llama-"):
        model = transformers.AutoModelForCausalLM.from_config(
            get_custom_llama_config(model_name.replace("custom-llama-", "")), dtype=torch.float32
        )
        tokenizer_name = "meta-llama/Llama-3.2-3B"
    else:
        model = transformers.AutoModelForCausalLM.from_pretrained(model_name, dtype=torch.float32)
        tokenizer_name = model_name
    try:
        model.tokenizer = transformers.AutoTokenizer.from_pretrained(tokenizer_name, local_files_only=True)
    except Exception:
        model.tokenizer = None  # gated or absent: the benchmark then uses random token ids
    return model


def build_decoder(model_name: str, config: QuantisationConfig | None, device: torch.device, tp, lut: Tensor | None = None):
    """The native decode loop for `model_name`: custom-llama-* shapes are created shard by shard on
    the device (a 31B fp32 host model would need 125 GB of host memory); any other name is loaded
    with load_host_model and its weights handed to the decoder."""
    from . import llama

    if model_name.startswith("custom-llama-"):
        return llama.LlamaDecoder.random_init(resolve_model_dims(model_name), config, device, tp, lut=lut)
    host = load_host_model(model_name)
    assert type(host).__name__ == "LlamaForCausalLM", f"the native decode loop takes Llama models, got {type(host).__name__}"
    return llama.LlamaDecoder.from_hf(host, config, device, tp, lut=lut)


def kmeans_like_codebook(bits: int, seed: int = 0) -> Tensor:
    """Sorted 2^bits centroids of N(0,1) samples (a few Lloyd iterations): stands in for the trained
    codebooks of the paper's checkpoints (`--lut kmeans`)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(20000, generator=g).sort().values
    c = torch.quantile(x, (torch.arange(2**bits) + 0.5) / 2**bits)
    for _ in range(8):
        idx = torch.bucketize(x, (c[1:] + c[:-1]) / 2)
        c = torch.stack([x[idx == i].mean() if (idx == i).any() else c[i] for i in range(2**bits)])
    return c.sort().values.bfloat16()


def load_kmeans_state_dict(module: nn.Module, state: dict, prefix: str = "") -> list[str]:
    """Loads externally trained quantised layers -- per layer a triple `weight_data` (packed codes
    as QuantisedLinear stores them), `scale` and `lut` (either the [256, 8 / bits] byte table or the
    plain 2^bits codebook, which is expanded) -- into the QuantisedLinear layers of `module`
    (e.g. the result of quantise() on the architecture), and everything else as load_state_dict
    would.  Returns the names of the quantised layers that were filled."""
    filled = []
    for name, layer in module.named_modules():
        if not isinstance(layer, QuantisedLinear):
            continue
        key = f"{prefix}{name}." if name else prefix
        if key + "weight_data" not in state:
            continue
        lut = state[key + "lut"]
        bits = layer.bits
        if lut.ndim == 1:  # plain codebook -> byte table
            assert lut.shape[0] == 2**bits, f"{name}: codebook of {lut.shape[0]} entries for {bits}-bit codes"
            lut = torch.cartesian_prod(*([lut] * (8 // bits))).view(256, -1) if 8 % bits == 0 else lut.reshape(-1, 1)
        data, scale = state[key + "weight_data"], state[key + "scale"]
        assert data.shape == layer.weight_data.shape and data.dtype == torch.uint8, f"{name}: weight_data {tuple(data.shape)}"
        assert scale.shape == layer.scale.shape, f"{name}: scale {tuple(scale.shape)}"
        with torch.no_grad():
            layer.weight_data.copy_(data)
            layer.scale.copy_(scale.to(layer.scale.dtype))
            layer.lut.copy_(lut.to(layer.lut.dtype))
        filled.append(name)
    rest = {k: v for k, v in state.items() if not any(k.startswith(f"{prefix}{n}.") for n in filled)}
    module.load_state_dict(rest, strict=False)
    return filled


def resolve_model_dims(name: str) -> LlamaDims:
    """'custom-llama-4B' (reference shapes) or 'custom-llama-b200-4B' (the B200 measurement shapes)."""
    assert name.startswith("custom-llama-"), f"only custom-llama-* models are built offline, got {name}"
    return get_custom_llama_dims(name.replace("custom-llama-", ""))


def run_benchmark(settings: BenchmarkSettings, device: torch.device, tp, log, lut_kind: str = "linear") -> None:
    """One model x batch x quantisation setting, as the reference's run_benchmark (models.py:476-516):
    memory released first, a pre-check that the model fits, the result (or the error) logged."""
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    config = settings.quantisation
    dtype = torch.float16 if config is not None and config.kernel.startswith("marlin") else torch.bfloat16
    out = dict(**settings.__dict__)
    if config is not None:
        out.update(config.__dict__)
    del out["quantisation"]
    model = None
    try:
        if not _estimate_fits_on_device(settings, device, dtype):
            raise RuntimeError(f"Model {settings.model} is too large for device")
        if dtype == torch.float16:
            raise RuntimeError("the decode loop is bf16; the fp16 Marlin selectors run at layer level (fdk.bench, quantise())")
        lut = None
        if config is not None and lut_kind == "kmeans":
            lut = kmeans_like_codebook(config.bits).to(device)
        model = build_decoder(settings.model, config, device, tp, lut=lut)
        result = benchmark(model, settings.batch_size, settings.reps, settings.context)
        out.update(result.__dict__)
        if tp.rank == 0:
            print(f"{str(settings):>60}:  {result}", file=sys.stderr)
        if getattr(model, "exchange", None) is not None:
            out.update(tp_reduce="fused", exchange_status=native.tp_exchange_status(model.exchange))
    except Exception as e:  # as the reference: log and carry on
        out.update(error=repr(e))
        if tp.rank == 0:
            print(f"{str(settings):>60}:  ERROR {e}", file=sys.stderr)
    finally:
        if model is not None:
            model.close()
            del model
    torch.cuda.empty_cache()
    if log is not None:
        log(out)


def _main() -> None:
    import argparse
    import os

    import torch.distributed as dist

    from . import bench, llama

    parser = argparse.ArgumentParser()
    parser.add_argument("--model", default=["custom-llama-4B"], nargs="+",
                        help=f"custom-llama-<size> (sizes {list(custom_llama_configs) + list(b200_llama_configs)}) "
                             "or a local Hugging Face Llama checkpoint")
    parser.add_argument("--batch-size", default=[1], type=int, nargs="+", help="Generation batch sizes")
    parser.add_argument("--bits", default=[16, 4, 1], type=int, nargs="+", help="Quantisation bit widths")
    parser.add_argument("--skip", default="^lm_head$", help="Regex of parameters to skip during quantisation")
    parser.add_argument("--block-size", default=[64], type=int, nargs="+", help="Quantisation block sizes")
    parser.add_argument("--kernel", default=["triton"], choices=["triton", "torch.compile", "marlin", "marlin-lut"],
                        nargs="+", help="Kernel implementation(s) (ignored for 16-bit)")
    parser.add_argument("--reps", "--gen-tokens", dest="reps", type=int, default=100,
                        help="Number of generation steps (generated tokens) to measure")
    parser.add_argument("--context", type=int, default=2, help="Tokens already in the KV cache")
    parser.add_argument("--lut", default="linear", choices=["linear", "kmeans"],
                        help="Codebook: the reference's default linspace grid, or sorted k-means-like centroids of N(0,1)")
    parser.add_argument("--tp", type=int, default=None,
                        help="Tensor-parallel ranks; must equal the number of processes torchrun started")
    parser.add_argument("--tp-reduce", default="fused", choices=["fused", "nccl"],
                        help="Under torchrun: how the row-parallel projections' partial sums are added "
                             "(fused = pushed from the kernel over NVLink, batches up to 16; else NCCL)")
    args = parser.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.tp is not None and args.tp != world:
        raise SystemExit(f"--tp {args.tp}: start {args.tp} processes, e.g. python -m torch.distributed.run "
                         f"--nproc-per-node {args.tp} --master-addr 127.0.0.1 -m fdk.models ... (found {world})")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    tp = llama.TensorParallel(rank, world, None, fused=args.tp_reduce == "fused")

    log = bench.Log("models") if rank == 0 else None
    for name in args.model:
        for batch_size in args.batch_size:
            for config in _quantisation_configs(args.bits, args.block_size, args.kernel, args.skip):
                run_benchmark(BenchmarkSettings(name, batch_size, config, args.reps, args.context, world), device, tp, log,
                              lut_kind=args.lut)
    if world > 1:
        # captured graphs that hold collectives must be gone before the communicator is
        import gc

        gc.collect()
        torch.cuda.synchronize()
        dist.destroy_process_group()


if __name__ == "__main__":
    _main()
