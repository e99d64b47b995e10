"""Decode loop on the native kernels against the reference's own model path: transformers'
LlamaForCausalLM with its Linears replaced by quantised ones evaluated with the torch reference
operator (what `quantise(..., kernel="torch.compile")` gives).  The reference pins no model
outputs, so the comparison is made here: per-step logits, teacher forced, rel-RMS error."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny_hf(seed=0):
    import transformers

    cfg = transformers.models.llama.modeling_llama.LlamaConfig(
        vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        head_dim=128, intermediate_size=512, rope_theta=500000, rms_norm_eps=1e-6, tie_word_embeddings=False,
        attn_implementation="eager",
    )
    torch.manual_seed(seed)
    return transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)


@pytest.mark.parametrize("bits", [4, 2])
def test_decode_logits_match_quantised_hf_model(bits):
    from fdk import llama, models

    device = torch.device("cuda")
    hf = _tiny_hf()
    cfg_ref = models.QuantisationConfig(bits, 64, kernel="torch.compile")
    ref = models.quantise(hf, cfg_ref, device, torch.bfloat16).eval()
    ours = llama.LlamaDecoder.from_hf(hf, models.QuantisationConfig(bits, 64), device)

    batch, steps = 3, 12
    ids = torch.randint(0, 512, (batch, steps), generator=torch.Generator().manual_seed(1)).to(device)
    with torch.no_grad():
        expected = ref(ids).logits.float()  # [batch, steps, vocab], causal
        ours.allocate(batch, steps + 1)
        got = torch.stack([ours(ids[:, t].contiguous()).float() for t in range(steps)], dim=1)
    err = (got - expected).pow(2).sum().div(expected.pow(2).sum()).sqrt().item()
    assert err < 3e-2, f"rel-RMS error of logits {err}"
    # greedy tokens agree on almost every step (bf16 noise can flip near-ties)
    agree = (got.argmax(-1) == expected.argmax(-1)).float().mean().item()
    assert agree > 0.8


def test_generator_runs_under_cuda_graph_and_counts_bytes():
    from fdk import bench, llama, models

    device = torch.device("cuda")
    dims = models.LlamaDims("tiny", 256, 2, 4, 2, 512, vocab_size=512)
    model = llama.LlamaDecoder.random_init(dims, models.QuantisationConfig(4, 64), device, seed=3)
    per_layer = (4 * 128 + 2 * 2 * 128) * 256 + 256 * 512 + 2 * 512 * 256 + 256 * 512
    expected_bytes = 2 * (per_layer * 4 // 8 + per_layer // 64 * 2) + 2 * 2 * 256 * 2 + 256 * 2 + 512 * 256 * 2
    assert models.count_parameter_read_bytes(model) == expected_bytes
    prompt = torch.randint(0, 512, (2, 5), device=device)
    gen = llama.Generator(model, prompt, steps=16)
    eager_tokens = []
    for _ in range(4):
        gen.step()
        eager_tokens.append(gen.last_token.clone())
    # same model, fresh generator, steps replayed from a CUDA graph
    gen2 = llama.Generator(model, prompt, steps=16)
    t, _ = bench.measure_time(lambda _: gen2.step(), inner_reps=1, outer_reps=2)
    assert t > 0
    assert gen2.tokens.shape[1] == 5 + 1 + int(gen2.last_index - 5)
    result = models.benchmark(model, batch_size=2, reps=3, context=16)
    assert result.avg_time > 0 and result.bytes_rw == expected_bytes


def test_glue_kernels_against_torch():
    from fdk import native

    torch.manual_seed(0)
    dev = "cuda"
    h = torch.randn(5, 3072, device=dev).bfloat16()
    delta = torch.randn(5, 3072, device=dev).bfloat16()
    w = (1 + 0.1 * torch.randn(3072, device=dev)).bfloat16()
    out = torch.empty_like(h)
    h2 = h.clone()
    native.rmsnorm(h2, delta, w, out, 1e-6)
    hs = h + delta
    ref = w * (hs.float() * torch.rsqrt(hs.float().pow(2).mean(-1, keepdim=True) + 1e-6)).bfloat16()
    assert torch.equal(h2, hs)
    assert (out.float() - ref.float()).abs().max() <= 2 * ref.float().abs().max() * 2**-8
    gu = torch.randn(4, 2 * 1024, device=dev).bfloat16()
    act = torch.empty(4, 1024, device=dev, dtype=torch.bfloat16)
    native.silu_mul(gu, act)
    ref = torch.nn.functional.silu(gu[:, :1024]) * gu[:, 1024:]
    assert (act.float() - ref.float()).abs().max() <= 2**-7 * ref.float().abs().max()
    # the same values with gates and ups alternating in groups of 32 columns
    paired = torch.stack([gu[:, :1024].unflatten(1, (-1, 32)), gu[:, 1024:].unflatten(1, (-1, 32))], dim=2).flatten(1).contiguous()
    act2 = torch.empty_like(act)
    native.silu_mul(paired, act2, group=32)
    assert torch.equal(act2, act)


def test_lm_head_is_quantised_when_the_skip_pattern_does_not_match_it():
    """The reference leaves lm_head in 16 bits by default (skip="^lm_head$") and quantises it
    like any other projection when the pattern does not match (src/fdk/models.py:27,144)."""
    from fdk import kernels, llama, models

    dev = torch.device("cuda")
    dims = models.LlamaDims("tiny", 256, 1, 2, 2, 512, vocab_size=1000)
    kept = llama.LlamaDecoder.random_init(dims, models.QuantisationConfig(4, 64), dev, seed=3)
    assert isinstance(kept.lm_head, torch.nn.Linear)
    cfg = models.QuantisationConfig(4, 64, skip="^$")
    model = llama.LlamaDecoder.random_init(dims, cfg, dev, seed=3)
    assert isinstance(model.lm_head, models.QuantisedLinear) and model.lm_head.out_features == 1000
    model.allocate(2, 8)
    with torch.no_grad():
        logits = model(torch.tensor([5, 7], device=dev))
    head = model.lm_head
    want = kernels.mm_lut_ref(model.normed, head.weight_data, head.lut, head.scale)
    err = (logits.float() - want.float()).pow(2).sum().div(want.float().pow(2).sum()).sqrt().item()
    assert err < 1e-2, err


@pytest.mark.parametrize("bits", [4])
def test_prefill_equals_token_by_token_decode(bits):
    """The one-pass prefill (projections on [batch * T, K], causal attention over the prompt) leaves
    the caches and the logits of the last position as T decode steps do, up to the kernels'
    different summation orders; and decoding goes on from there."""
    from fdk import llama, models

    device = torch.device("cuda")
    dims = models.LlamaDims("tiny", 512, 2, 8, 2, 1024, vocab_size=640)
    model = llama.LlamaDecoder.random_init(dims, models.QuantisationConfig(bits, 64), device, seed=9, std=0.05)
    batch, t = 3, 21
    ids = torch.randint(0, 640, (batch, t + 1), generator=torch.Generator().manual_seed(4)).to(device)
    with torch.no_grad():
        model.allocate(batch, t + 4)
        for step in range(t):
            stepwise = model(ids[:, step].contiguous()).float()
        after_stepwise = model(ids[:, t].contiguous()).float()
        k_stepwise = [c[:, :, :t].clone() for c in model.k_cache]
        model.allocate(batch, t + 4)
        once = model.prefill(ids[:, :t]).float()
        after_once = model(ids[:, t].contiguous()).float()
    torch.cuda.synchronize()
    rel = lambda a, b: (a - b).pow(2).sum().div(b.pow(2).sum()).sqrt().item()
    assert rel(once, stepwise) < 3e-2
    assert rel(after_once, after_stepwise) < 3e-2
    for a, b in zip(model.k_cache, k_stepwise):
        assert rel(a[:, :, :t].float(), b.float()) < 3e-2
