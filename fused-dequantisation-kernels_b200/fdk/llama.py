"""Custom-llama decode loop on the native kernels, single GPU or tensor parallel.

The reference benchmarks decode by wrapping transformers' LlamaForCausalLM in a greedy
`Generator` (prefill once, then one captured decode step per token; src/fdk/models.py:225-340)
and replacing its nn.Linear layers with quantised ones.  This module is that decode step
written out -- embedding, [RMSNorm, fused q|k|v projection, rotary + KV append, attention,
o projection, RMSNorm, fused gate|up projection, SiLU*up, down projection] x layers, final
norm, lm_head (left in bf16, as the reference's default `skip="^lm_head$"` does), argmax --
with every projection a `QuantisedLinear` running libfdk_b200's fused kernel (or a bf16
`nn.Linear` for the 16-bit baseline) and the glue -- norm + residual, rotary + cache append,
split-context attention over the static KV cache, SiLU * up -- in four fused CUDA kernels.

Tensor parallelism (not in the reference, which is single-GPU): Megatron-style.  q|k|v and
gate|up are split by output rows (whole heads), o and down by input columns; block scales run
along K inside a row, so sharding the bf16 weight and then quantising equals quantising and
then sharding.  The [batch, hidden] partial sums of o and down are added over the ranks either
by an NCCL all-reduce, or ("fused", batches up to 16) by the projection kernel storing them
into every rank's exchange buffer over NVLink and the next RMSNorm kernel adding them up.
Embedding and norms are replicated; lm_head is split by vocabulary rows and the logits gathered.
"""

from __future__ import annotations

import re
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor, nn

from . import native
from .models import LlamaDims, QuantisationConfig, QuantisedLinear


PAIR_GROUP = 32  # gate / up rows alternate in groups of this many (see _shard_layer_weights)
# row order of a q or k head in the fused q|k|v weight: the two dimensions that the rotary
# embedding combines (i, i + 64) in one 64-row tile of the projection kernel
ROPE_ROW_ORDER = list(range(0, 32)) + list(range(64, 96)) + list(range(32, 64)) + list(range(96, 128))


@dataclass
class TensorParallel:
    rank: int = 0
    size: int = 1
    group: "dist.ProcessGroup | None" = None
    fused: bool = False  # push from the projection kernel + sum in the RMSNorm kernel, where possible

    def all_reduce(self, t: Tensor) -> None:
        if self.size > 1:
            dist.all_reduce(t, group=self.group)

    def open_exchange(self, slot_elems: int, device: torch.device) -> "native.TpExchange":
        """One exchange buffer per rank, each mapped by all the others (CUDA IPC; one node)."""
        nbytes = native.tp_exchange_bytes(self.size, slot_elems)
        mine, handle = native.tp_buffer_create(nbytes, device)
        handles: list = [None] * self.size
        dist.all_gather_object(handles, handle, group=self.group)
        buffers = [mine if j == self.rank else native.tp_buffer_open(handles[j], device) for j in range(self.size)]
        dist.barrier(group=self.group)
        return native.make_exchange(self.size, self.rank, buffers, slot_elems)


def shard_rows(n: int, tp: TensorParallel) -> slice:
    assert n % tp.size == 0, f"{n} rows do not split over {tp.size} ranks"
    per = n // tp.size
    return slice(tp.rank * per, (tp.rank + 1) * per)


def shard_columns(k: int, tp: TensorParallel) -> slice:
    assert k % (64 * tp.size) == 0, f"{k} columns do not split over {tp.size} ranks in multiples of 64"
    per = k // tp.size
    return slice(tp.rank * per, (tp.rank + 1) * per)


class DecoderLayer(nn.Module):
    def __init__(self, qkv: nn.Module, o: nn.Module, gate_up: nn.Module, down: nn.Module,
                 input_norm: Tensor, post_norm: Tensor):
        super().__init__()
        self.qkv, self.o, self.gate_up, self.down = qkv, o, gate_up, down
        self.input_norm = nn.Parameter(input_norm, requires_grad=False)
        self.post_norm = nn.Parameter(post_norm, requires_grad=False)


def _make_linear(weight: Tensor, config: QuantisationConfig | None, lut: Tensor | None) -> nn.Module:
    """weight [N, K] bf16 on the device -> QuantisedLinear (config) or nn.Linear (16-bit baseline)."""
    if config is None:
        layer = nn.Linear(weight.shape[1], weight.shape[0], bias=False, device=weight.device, dtype=weight.dtype)
        layer.weight = nn.Parameter(weight, requires_grad=False)
        return layer
    layer = QuantisedLinear.create(weight, config, lut=lut)
    if config.kernel != "torch.compile":
        layer.tiled()
    return layer


class LlamaDecoder(nn.Module):
    """Decode-only Llama.  Build with `random_init` (synthetic weights created shard by shard on
    the device) or `from_hf` (weights of a transformers LlamaForCausalLM)."""

    def __init__(self, dims: LlamaDims, layers: list[DecoderLayer], embed: Tensor, final_norm: Tensor,
                 lm_head: Tensor, tp: TensorParallel, config: QuantisationConfig | None = None,
                 lut: Tensor | None = None):
        super().__init__()
        self.dims, self.tp = dims, tp
        self.layers = nn.ModuleList(layers)
        self.embed = nn.Embedding.from_pretrained(embed, freeze=True)
        self.final_norm = nn.Parameter(final_norm, requires_grad=False)
        # lm_head: split by vocabulary rows over the ranks (logits are gathered), and quantised
        # like the other projections unless the configuration's `skip` pattern matches its name
        # (the reference's default "^lm_head$" does; src/fdk/models.py:27,144)
        self.vocab_sharded = tp.size > 1 and dims.vocab_size % tp.size == 0
        if self.vocab_sharded:
            lm_head = lm_head[shard_rows(dims.vocab_size, tp)].contiguous()
        skipped = config is None or (config.skip is not None and re.search(config.skip, "lm_head") is not None)
        self.lm_head = _make_linear(lm_head, None if skipped else config, lut)
        self.q_heads = dims.num_attention_heads // tp.size
        self.kv_heads = dims.num_key_value_heads // tp.size
        assert dims.num_key_value_heads % tp.size == 0, "KV heads must split evenly over the ranks"
        assert dims.head_dim == 128
        # how the fused decode step applies its RMSNorms: split between the projections that write
        # and read the residual stream (True: the reading projection takes its x fragments straight
        # from L2 like every other projection and scales its sums; one bf16 rounding per element
        # of x sits elsewhere than in the framework model), or by the reading projection while it
        # copies x into shared memory, with the framework model's roundings (False).  Measured on
        # the 4B shape, tokens/s split / while copying: batch 1: 754 / 740, 2: 1456 / 1426,
        # 4: 2426 / 2298
        self.deferred_norm = True
        # largest batch whose projections carry the decode-step fusions.  Measured on the 4B shape
        # (tokens/s fused against separate glue kernels): batch 1: 754 / 719, 2: 1456 / 1397,
        # 4: 2426 / 2374, 8: 3780 / 3838 -- the single finisher warp goes through all batch rows,
        # and the small glue kernels overlap their neighbours well
        self.fuse_rows = 4
        # largest batch whose q|k|v projection does the rotary embedding + KV append in its epilogue
        # in the tensor-parallel step (where the norms cannot be fused)
        self.rope_rows = 16

    # ---- construction -----------------------------------------------------------------

    @staticmethod
    def _shard_layer_weights(q, k, v, o, gate, up, down, dims: LlamaDims, tp: TensorParallel):
        d = dims.head_dim
        qs = shard_rows(dims.num_attention_heads, tp)
        ks = shard_rows(dims.num_key_value_heads, tp)
        order = torch.tensor(ROPE_ROW_ORDER, device=q.device)

        def paired(w):  # [heads * 128, hidden] -> the same with every head's rows in ROPE_ROW_ORDER
            return w.unflatten(0, (-1, d))[:, order].flatten(0, 1)

        qkv = torch.cat([paired(q[qs.start * d: qs.stop * d]), paired(k[ks.start * d: ks.stop * d]), v[ks.start * d: ks.stop * d]])
        fs = shard_rows(dims.intermediate_size, tp)
        # rows in groups of 64: 32 gate rows, then the 32 matching up rows, so that one 64-row
        # tile of the projection kernel holds both factors of 32 outputs of SiLU(gate) * up
        assert (fs.stop - fs.start) % PAIR_GROUP == 0, "the FFN width per rank must be a multiple of 32"
        gate_up = torch.stack([gate[fs].unflatten(0, (-1, PAIR_GROUP)), up[fs].unflatten(0, (-1, PAIR_GROUP))], dim=1).flatten(0, 2)
        o_s = o[:, qs.start * d: qs.stop * d].contiguous()
        down_s = down[:, fs].contiguous()
        return qkv, o_s, gate_up, down_s

    @classmethod
    def random_init(cls, dims: LlamaDims, config: QuantisationConfig | None, device: torch.device,
                    tp: TensorParallel | None = None, seed: int = 0, lut: Tensor | None = None,
                    std: float = 0.02) -> "LlamaDecoder":
        """Random bf16 weights ~ N(0, std^2), generated per layer on the device with a seed that
        does not depend on the rank (every rank draws the full matrix and keeps its shard)."""
        tp = tp or TensorParallel()
        gen = torch.Generator(device=device).manual_seed(seed)
        h, f, d = dims.hidden_size, dims.intermediate_size, dims.head_dim

        def draw(n, k):
            return (torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * std).bfloat16()

        layers = []
        for _ in range(dims.num_hidden_layers):
            q, k, v = draw(dims.num_attention_heads * d, h), draw(dims.num_key_value_heads * d, h), draw(dims.num_key_value_heads * d, h)
            o = draw(h, dims.num_attention_heads * d)
            gate, up, down = draw(f, h), draw(f, h), draw(h, f)
            qkv_w, o_w, gu_w, down_w = cls._shard_layer_weights(q, k, v, o, gate, up, down, dims, tp)
            del q, k, v, o, gate, up, down
            ones = torch.ones(h, device=device, dtype=torch.bfloat16)
            layers.append(DecoderLayer(
                _make_linear(qkv_w, config, lut), _make_linear(o_w, config, lut),
                _make_linear(gu_w, config, lut), _make_linear(down_w, config, lut), ones, ones.clone(),
            ))
        embed = draw(dims.vocab_size, h)
        lm_head = draw(dims.vocab_size, h)
        return cls(dims, layers, embed, torch.ones(h, device=device, dtype=torch.bfloat16), lm_head, tp, config, lut)

    @classmethod
    def from_hf(cls, model, config: QuantisationConfig | None, device: torch.device,
                tp: TensorParallel | None = None, lut: Tensor | None = None) -> "LlamaDecoder":
        """Takes the weights of a transformers LlamaForCausalLM (any float dtype)."""
        tp = tp or TensorParallel()
        c = model.config
        dims = LlamaDims(
            name=getattr(c, "_name_or_path", "llama"), hidden_size=c.hidden_size, num_hidden_layers=c.num_hidden_layers,
            num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
            intermediate_size=c.intermediate_size, vocab_size=c.vocab_size,
            head_dim=getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads,
            rope_theta=float(getattr(c, "rope_theta", None) or c.rope_parameters["rope_theta"]),
            rms_norm_eps=c.rms_norm_eps,
        )

        def w(t):
            return t.detach().to(device=device, dtype=torch.bfloat16)

        layers = []
        for hl in model.model.layers:
            a, m = hl.self_attn, hl.mlp
            qkv_w, o_w, gu_w, down_w = cls._shard_layer_weights(
                w(a.q_proj.weight), w(a.k_proj.weight), w(a.v_proj.weight), w(a.o_proj.weight),
                w(m.gate_proj.weight), w(m.up_proj.weight), w(m.down_proj.weight), dims, tp,
            )
            layers.append(DecoderLayer(
                _make_linear(qkv_w, config, lut), _make_linear(o_w, config, lut),
                _make_linear(gu_w, config, lut), _make_linear(down_w, config, lut),
                w(hl.input_layernorm.weight), w(hl.post_attention_layernorm.weight),
            ))
        return cls(dims, layers, w(model.model.embed_tokens.weight), w(model.model.norm.weight), w(model.lm_head.weight), tp,
                   config, lut)

    # ---- decode state -----------------------------------------------------------------

    def allocate(self, batch: int, max_len: int) -> None:
        """Static KV caches [layer][batch, kv_heads, max_len, 128] and activation buffers."""
        dev, dt = self.final_norm.device, torch.bfloat16
        h, f = self.dims.hidden_size, self.dims.intermediate_size // self.tp.size
        self.batch, self.max_len = batch, max_len
        self.k_cache = [torch.zeros((batch, self.kv_heads, max_len, 128), device=dev, dtype=dt) for _ in self.layers]
        self.v_cache = [torch.zeros((batch, self.kv_heads, max_len, 128), device=dev, dtype=dt) for _ in self.layers]
        self.hidden = torch.empty((batch, h), device=dev, dtype=dt)
        self.normed = torch.empty((batch, h), device=dev, dtype=dt)
        self.q = torch.empty((batch, self.q_heads * 128), device=dev, dtype=dt)
        self.act = torch.empty((batch, f), device=dev, dtype=dt)
        self.attn = torch.empty((batch, self.q_heads * 128), device=dev, dtype=dt)
        self.position = torch.zeros((), device=dev, dtype=torch.int64)
        self.host_position = 0  # eager calls made so far (graph replays are bounded on the device instead)
        self.splits = native.attention_slices(batch, self.q_heads, self.kv_heads, max_len)
        self.attn_scratch, self.attn_counters = native.attention_scratch(batch, self.q_heads, self.kv_heads, self.splits, dev)
        # the projections do the norms, the residual adds and the rotary embedding themselves where
        # they can: native quantised layers, one rank, batches up to 16 rows, x small enough to be staged
        native_layers = all(
            isinstance(m, QuantisedLinear) and m.kernel != "torch.compile"
            for l in self.layers for m in (l.qkv, l.o, l.gate_up, l.down)
        )
        self.fusions = None
        self.rope_fusions = None
        if native_layers and batch <= 16:
            self.rope_tab = torch.zeros(64, device=dev, dtype=torch.int32)
            self.sumsq = torch.zeros((batch, h // 64), device=dev, dtype=torch.float32)
            self.hw = torch.zeros((batch, h), device=dev, dtype=torch.bfloat16)  # norm weight * residual stream
            normed = [m for l in self.layers for m in (l.qkv, l.gate_up)]
            # small batches only (see fuse_rows)
            fits = self.deferred_norm or all(native.linear_norm_fits(batch, h, m.bits) for m in normed)
            if self.tp.size == 1 and batch <= self.fuse_rows and h % 64 == 0 and fits:
                self.fusions = [self._layer_fusions(i) for i in range(len(self.layers))]
            elif batch <= self.rope_rows:
                # tensor parallel: the norms add the ranks' partial sums; the rotary epilogue still applies
                self.rope_fusions = [self._layer_fusions(i, rope_only=True) for i in range(len(self.layers))]
        # fused push + reduce instead of NCCL: quantised row-parallel projections, batch <= 16
        self.close()
        can_push = all(
            isinstance(m, QuantisedLinear) and m.kernel != "torch.compile" for l in self.layers for m in (l.o, l.down)
        )
        if self.tp.size > 1 and self.tp.fused and batch <= 16 and can_push and h % 64 == 0:
            self.exchange = self.tp.open_exchange(16 * h, dev)

    def check_status(self) -> None:
        """Reads the device-side status words the kernels of this decoder report to (synchronises):
        the workspace of the projections, the attention scratch and the tensor-parallel exchange.
        Raises if a bounded wait ran out or a kernel found shared memory laid out differently
        from the host's plan -- outputs computed since the last check are then not to be trusted."""
        dev = self.final_norm.device
        words = {"projection workspace": native.device_status(dev)}
        if getattr(self, "attn_counters", None) is not None and self.splits > 1:
            words["attention scratch"] = native.attention_status(self.attn_counters, self.batch, self.kv_heads)
        if self.exchange is not None:
            words["tensor-parallel exchange"] = native.tp_exchange_status(self.exchange)
        bad = {k: v for k, v in words.items() if v}
        if bad:
            raise native.FdkError(-1, "device-side status", f"non-zero status words: {bad}")

    def _layer_fusions(self, i: int, rope_only: bool = False):
        """The fusion descriptors of layer i (pointers into this decoder's buffers)."""
        layer, eps = self.layers[i], self.dims.rms_norm_eps
        if rope_only:
            return native.LinearFusion(
                rope_pos=self.position.data_ptr(), rope_table=self.rope_tab.data_ptr(), q_out=self.q.data_ptr(),
                k_cache=self.k_cache[i].data_ptr(), v_cache=self.v_cache[i].data_ptr(), q_heads=self.q_heads,
                kv_heads=self.kv_heads, max_len=self.max_len)

        def norm(weight: Tensor) -> dict:
            return dict(norm_h=self.hidden.data_ptr(), norm_weight=weight.data_ptr(), norm_sumsq=self.sumsq.data_ptr(),
                        norm_tiles=self.sumsq.shape[1], norm_eps=eps)

        resid = dict(resid_h=self.hidden.data_ptr(), resid_sumsq=self.sumsq.data_ptr())
        rope = dict(rope_pos=self.position.data_ptr(), rope_table=self.rope_tab.data_ptr(), q_out=self.q.data_ptr(),
                    k_cache=self.k_cache[i].data_ptr(), v_cache=self.v_cache[i].data_ptr(), q_heads=self.q_heads,
                    kv_heads=self.kv_heads, max_len=self.max_len)
        if self.deferred_norm:
            # the norm split in two: the projection that writes the residual stream also writes
            # norm weight * h (the x of the next projection), which scales its sums by the norm factor
            scale = dict(scale_sumsq=self.sumsq.data_ptr(), scale_tiles=self.sumsq.shape[1], scale_eps=eps)
            after = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else None

            def folded(weight: Tensor | None) -> dict:
                return {} if weight is None else dict(resid_norm_weight=weight.data_ptr(), resid_x=self.hw.data_ptr())

            return (
                native.LinearFusion(**scale, **rope),                        # q|k|v of hw
                native.LinearFusion(**resid, **folded(layer.post_norm)),     # o
                native.LinearFusion(**scale),                                # gate|up of hw
                native.LinearFusion(**resid, **folded(after)),               # down
            )
        return (
            native.LinearFusion(**norm(layer.input_norm), **rope),  # q|k|v
            native.LinearFusion(**resid),                           # o
            native.LinearFusion(**norm(layer.post_norm)),           # gate|up
            native.LinearFusion(**resid),                           # down
        )

    def _gated(self, layer: DecoderLayer) -> None:
        """self.act = SiLU(gate) * up of self.normed."""
        if isinstance(layer.gate_up, QuantisedLinear):
            layer.gate_up.forward_silu_pairs(self.normed, self.act)
        else:
            native.silu_mul(layer.gate_up(self.normed), self.act, group=PAIR_GROUP)

    def close(self) -> None:
        """Unmaps the other ranks' exchange buffers and frees this rank's (collective: every rank
        calls it).  Without it they live until the process exits."""
        ex = getattr(self, "exchange", None)
        self.exchange = None
        if ex is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.tp.group)
        for j in range(ex.tp):
            if j != ex.rank:
                native.tp_buffer_close(ex.buffers[j])
        dist.barrier(group=self.tp.group)
        native.tp_buffer_destroy(ex.buffers[ex.rank])

    def fill_cache_synthetic(self, context: int, seed: int = 1) -> None:
        """Benchmark aid: pretend `context` tokens have been decoded (random keys and values)."""
        gen = torch.Generator(device=self.hidden.device).manual_seed(seed + self.tp.rank)
        for kc, vc in zip(self.k_cache, self.v_cache):
            kc[:, :, :context].copy_(torch.randn(kc[:, :, :context].shape, generator=gen, device=kc.device, dtype=torch.float32))
            vc[:, :, :context].copy_(torch.randn(vc[:, :, :context].shape, generator=gen, device=vc.device, dtype=torch.float32))
        self.position.fill_(context)
        self.host_position = context

    # ---- prefill -----------------------------------------------------------------------

    def prefill(self, ids: Tensor) -> Tensor:
        """ids [batch, T] at positions 0 .. T - 1 of freshly allocated caches -> logits of the last
        position [batch, vocab]; fills the KV caches and leaves the position at T.  One pass over
        the whole prompt, as the reference's Generator does with transformers' model
        (src/fdk/models.py:241-243): the projections run the fused kernels on [batch * T, K]
        (the tensor-core kernel from 17 rows on), the norms the RMSNorm kernel; rotary embedding and
        causal attention over the prompt are torch ops (this path runs once per sequence)."""
        dims, eps = self.dims, self.dims.rms_norm_eps
        batch, t = ids.shape
        assert batch == self.batch and t <= self.max_len, f"prompt {tuple(ids.shape)} for caches of {self.batch} x {self.max_len}"
        dev = ids.device
        rows = batch * t
        hidden = self.embed.weight[ids.reshape(-1)].contiguous()  # [rows, hidden]
        normed = torch.empty_like(hidden)
        unpair = torch.argsort(torch.tensor(ROPE_ROW_ORDER, device=dev))  # paired row order -> dimensions 0 .. 127
        inv_freq = 1.0 / (dims.rope_theta ** (torch.arange(0, 128, 2, dtype=torch.float32, device=dev) / 128))
        angles = torch.arange(t, dtype=torch.float32, device=dev)[:, None] * inv_freq[None, :]
        emb = torch.cat((angles, angles), dim=-1)
        cos, sin = emb.cos().bfloat16()[None, :, None, :], emb.sin().bfloat16()[None, :, None, :]  # [1, T, 1, 128]

        def rotate(x):  # [batch, T, heads, 128], transformers' rotate-half form
            return x * cos + torch.cat((-x[..., 64:], x[..., :64]), dim=-1) * sin

        delta = None
        for i, layer in enumerate(self.layers):
            native.rmsnorm(hidden, delta, layer.input_norm, normed, eps)
            qkv = layer.qkv(normed).view(batch, t, self.q_heads + 2 * self.kv_heads, 128)
            q = rotate(qkv[:, :, : self.q_heads][..., unpair])
            k = rotate(qkv[:, :, self.q_heads: self.q_heads + self.kv_heads][..., unpair])
            v = qkv[:, :, self.q_heads + self.kv_heads:]
            self.k_cache[i][:, :, :t] = k.transpose(1, 2)
            self.v_cache[i][:, :, :t] = v.transpose(1, 2)
            attn = nn.functional.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True
            ).transpose(1, 2).reshape(rows, self.q_heads * 128).contiguous()
            delta = layer.o(attn)
            self.tp.all_reduce(delta)
            native.rmsnorm(hidden, delta, layer.post_norm, normed, eps)
            if isinstance(layer.gate_up, QuantisedLinear):
                act = torch.empty((rows, layer.gate_up.out_features // 2), device=dev, dtype=torch.bfloat16)
                layer.gate_up.forward_silu_pairs(normed, act)
            else:
                act = torch.empty((rows, layer.gate_up.out_features // 2), device=dev, dtype=torch.bfloat16)
                native.silu_mul(layer.gate_up(normed), act, group=PAIR_GROUP)
            delta = layer.down(act)
            self.tp.all_reduce(delta)
        last = hidden.view(batch, t, -1)[:, -1].contiguous()
        last_delta = delta.view(batch, t, -1)[:, -1].contiguous()
        native.rmsnorm(last, last_delta, self.final_norm, self.normed, eps)
        self.hidden.copy_(last)
        self.position.fill_(t)
        self.host_position = t
        return self._logits()

    # ---- one decode step --------------------------------------------------------------

    def forward(self, tokens: Tensor) -> Tensor:
        """tokens [batch] int64 at position `self.position` -> logits [batch, vocab]; advances the
        position.  No host synchronisation, fixed shapes: capturable in a CUDA graph."""
        dims, eps = self.dims, self.dims.rms_norm_eps
        if self.host_position >= self.max_len:
            raise RuntimeError(f"decode step at position {self.host_position}: the KV cache was allocated for {self.max_len} positions")
        self.host_position += 1
        torch.index_select(self.embed.weight, 0, tokens, out=self.hidden)
        if self.exchange is not None:
            return self._forward_fused()
        if self.fusions is not None:
            return self._forward_glue_fused()
        delta = None
        for i, layer in enumerate(self.layers):
            native.rmsnorm(self.hidden, delta, layer.input_norm, self.normed, eps)
            qkv = layer.qkv(self.normed)
            native.rope_append(qkv, self.position, self.q, self.k_cache[i], self.v_cache[i], self.q_heads, self.kv_heads,
                               dims.rope_theta, paired=True)
            native.decode_attention(self.q, self.k_cache[i], self.v_cache[i], self.position, self.attn,
                                    self.attn_scratch, self.attn_counters, self.q_heads, self.kv_heads, self.splits)
            delta = layer.o(self.attn)
            self.tp.all_reduce(delta)
            native.rmsnorm(self.hidden, delta, layer.post_norm, self.normed, eps)
            self._gated(layer)
            delta = layer.down(self.act)
            self.tp.all_reduce(delta)
        native.rmsnorm(self.hidden, delta, self.final_norm, self.normed, eps)
        logits = self._logits()
        self.position += 1
        return logits

    def _forward_glue_fused(self) -> Tensor:
        """The same step in five kernels per layer: the q|k|v projection does the rotary embedding
        + KV append in its epilogue; the o and down projections add their result to the residual
        stream and leave the sums of squares for the next norm; the gate|up projection writes
        SiLU(gate) * up.  The RMSNorms are either split (`deferred_norm`, the default): the
        projection that writes the residual stream also writes norm weight * h, and the one that
        reads it multiplies its sums by the norm factor; or applied by the q|k|v and gate|up
        projections while they copy x into shared memory."""
        dims, eps, b = self.dims, self.dims.rms_norm_eps, self.batch
        native.rope_table(self.position, self.rope_tab, dims.rope_theta)
        if self.deferred_norm:
            native.norm_prepare(self.hidden, self.layers[0].input_norm, self.hw, self.sumsq)
            normed_x = self.hw
        else:
            native.sumsq_tiles(self.hidden, self.sumsq)
            normed_x = None  # the projection normalises self.hidden itself while it stages x
        for i, layer in enumerate(self.layers):
            f_qkv, f_o, f_gate, f_down = self.fusions[i]
            layer.qkv.fused(normed_x, None, b, f_qkv)
            native.decode_attention(self.q, self.k_cache[i], self.v_cache[i], self.position, self.attn,
                                    self.attn_scratch, self.attn_counters, self.q_heads, self.kv_heads, self.splits)
            layer.o.fused(self.attn, None, b, f_o)
            layer.gate_up.fused(normed_x, self.act, b, f_gate, silu_pairs=True)
            layer.down.fused(self.act, None, b, f_down)
        native.rmsnorm(self.hidden, None, self.final_norm, self.normed, eps)
        logits = self._logits()
        self.position += 1
        return logits

    def _logits(self) -> Tensor:
        """lm_head of self.normed -> [batch, vocab]; the ranks' vocabulary slices are gathered."""
        local = self.lm_head(self.normed)
        if not self.vocab_sharded:
            return local
        gathered = torch.empty((self.tp.size,) + tuple(local.shape), device=local.device, dtype=local.dtype)
        dist.all_gather_into_tensor(gathered, local.contiguous(), group=self.tp.group)
        return gathered.permute(1, 0, 2).reshape(local.shape[0], -1)


    def _forward_fused(self) -> Tensor:
        """The same step with each row-parallel projection pushing its partial sums to all ranks
        and the following RMSNorm adding them: no collective launches."""
        dims, eps, ex = self.dims, self.dims.rms_norm_eps, self.exchange
        if self.rope_fusions is not None:
            native.rope_table(self.position, self.rope_tab, dims.rope_theta)
        for i, layer in enumerate(self.layers):
            if i == 0:
                native.rmsnorm(self.hidden, None, layer.input_norm, self.normed, eps)
            else:
                native.rmsnorm_reduce(self.hidden, ex, layer.input_norm, self.normed, eps)
            if self.rope_fusions is not None:  # rotary embedding + KV append in the projection's epilogue
                layer.qkv.fused(self.normed, None, self.batch, self.rope_fusions[i])
            else:
                qkv = layer.qkv(self.normed)
                native.rope_append(qkv, self.position, self.q, self.k_cache[i], self.v_cache[i], self.q_heads,
                                   self.kv_heads, dims.rope_theta, paired=True)
            native.decode_attention(self.q, self.k_cache[i], self.v_cache[i], self.position, self.attn,
                                    self.attn_scratch, self.attn_counters, self.q_heads, self.kv_heads, self.splits)
            layer.o.push(self.attn, ex)
            native.rmsnorm_reduce(self.hidden, ex, layer.post_norm, self.normed, eps)
            self._gated(layer)
            layer.down.push(self.act, ex)
        native.rmsnorm_reduce(self.hidden, ex, self.final_norm, self.normed, eps)
        logits = self._logits()
        self.position += 1
        return logits



class Generator:
    """Greedy decoding with the reference Generator's interface (src/fdk/models.py:225-259):
    construct with a prompt (prefilled in one pass, LlamaDecoder.prefill), call step() per
    generated token, read `tokens`.  step() is capturable in a CUDA graph."""

    def __init__(self, model: LlamaDecoder, prompt_ids: Tensor, steps: int, synthetic_context: int | None = None) -> None:
        batch_size, prompt_n = prompt_ids.shape
        context = prompt_n if synthetic_context is None else synthetic_context
        max_length = context + steps + 1
        self.model = model
        device = model.final_norm.device
        model.allocate(batch_size, max_length)
        self.input_ids = torch.zeros((batch_size, max_length), dtype=torch.long, device=device)
        with torch.no_grad():
            if synthetic_context is None:
                self.input_ids[:, :prompt_n] = prompt_ids
                if prompt_n > 1 and model.exchange is None:
                    logits = model.prefill(prompt_ids)  # the whole prompt in one pass
                else:
                    logits = None
                    for t in range(prompt_n):
                        logits = model(self.input_ids[:, t].contiguous())
            else:  # keys and values of a made-up context; only the last prompt token is run
                self.input_ids[:, context - 1] = prompt_ids[:, -1]
                model.fill_cache_synthetic(context - 1)
                logits = model(self.input_ids[:, context - 1].contiguous())
            self.last_token = torch.empty(batch_size, dtype=torch.long, device=device)
            self._choose(logits)
            self.input_ids[:, context] = self.last_token
        self.last_index = torch.tensor(context, device=device)
        self.last_logits = logits
        model.check_status()

    def _choose(self, logits: Tensor) -> None:
        """Greedy choice (`logits.argmax(dim=-1)` in the reference, src/fdk/models.py:252) into
        `last_token`, by the native kernel (torch's row-wise argmax runs one thread block over the
        whole vocabulary: ~45 us at 128 k entries against ~5)."""
        if logits.is_cuda and logits.dim() == 2 and logits.is_contiguous() and logits.dtype in (torch.bfloat16, torch.float16):
            native.argmax(logits, self.last_token)
        else:
            self.last_token[...] = logits.argmax(dim=-1)

    def step(self) -> None:
        with torch.no_grad():
            logits = self.model(self.last_token)
            self.last_logits = logits
            self._choose(logits)
            self.last_index += 1
            token = self.last_token[:, None]
            self.input_ids.scatter_(1, self.last_index[None, None].expand_as(token), token)

    @property
    def tokens(self) -> Tensor:
        return self.input_ids[:, : self.last_index + 1]
