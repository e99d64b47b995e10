"""The decode step's glue kernels called directly through the C-ABI library, against fp32 torch
restatements of what the reference takes from transformers' Llama (src/fdk/models.py:238-251):

  * fdk_decode_attention vs softmax(q K^T / sqrt(d)) V computed in fp32 on the same bf16 cache:
    every grouped-query ratio the models use (3: 4B, 5: 12B, 6: 31B) and the extremes, one and
    several context slices (the split path with its merge by the first slice, empty slices, clamped
    tail reads), positions at slice boundaries and beyond 2048, each launch repeated on the same
    scratch and counters (use counts and tagged words);
  * fdk_rope_append vs the rotate-half formula with cos/sin rounded to bf16, at positions 0, 1024
    and 2175 (angles up to ~2176 rad), and a position outside the cache.
"""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_LEN = 2304
KV_HEADS = 2


@pytest.fixture(scope="module")
def native():
    from fdk import native as nat

    nat.lib()
    return nat


_caches: dict = {}


def _cache(batch: int):
    if batch not in _caches:
        gen = torch.Generator(device="cuda").manual_seed(100 + batch)
        shape = (batch, KV_HEADS, MAX_LEN, 128)
        _caches[batch] = (
            torch.randn(shape, generator=gen, device="cuda").bfloat16(),
            torch.randn(shape, generator=gen, device="cuda").bfloat16(),
        )
    return _caches[batch]


def attention_reference(q, k_cache, v_cache, pos: int, group: int):
    """fp32: q [b, kv * group, 128], caches [b, kv, max_len, 128], keys 0 .. pos."""
    b = q.shape[0]
    qf = q.float().view(b, KV_HEADS, group, 128)
    k = k_cache[:, :, : pos + 1].float()
    v = v_cache[:, :, : pos + 1].float()
    scores = torch.einsum("bhgd,bhpd->bhgp", qf, k) / math.sqrt(128.0)
    return torch.einsum("bhgp,bhpd->bhgd", scores.softmax(dim=-1), v).reshape(b, -1)


@pytest.mark.parametrize("batch", [1, 16])
@pytest.mark.parametrize("splits", [1, 4, 9, 16])
@pytest.mark.parametrize("group", [1, 2, 3, 4, 5, 6, 7, 8])
def test_decode_attention_matches_fp32_reference(native, group, splits, batch):
    q_heads = group * KV_HEADS
    k_cache, v_cache = _cache(batch)
    scratch, counters = native.attention_scratch(batch, q_heads, KV_HEADS, splits, torch.device("cuda"))
    gen = torch.Generator(device="cuda").manual_seed(7 * group + splits + batch)
    launches = 0
    for pos_value in (0, 127, 128, 1023, 2175):
        q = torch.randn((batch, q_heads * 128), generator=gen, device="cuda").bfloat16()
        pos = torch.tensor(pos_value, device="cuda", dtype=torch.int64)
        expected = attention_reference(q.view(batch, q_heads, 128), k_cache, v_cache, pos_value, group)
        for repeat in range(2):  # later launches find scratch and counters as the earlier ones left them
            out = torch.full((batch, q_heads * 128), float("nan"), device="cuda", dtype=torch.bfloat16)
            native.decode_attention(q, k_cache, v_cache, pos, out, scratch, counters, q_heads, KV_HEADS, splits)
            torch.cuda.synchronize()
            launches += 1
            if splits > 1:  # every (batch row, KV head) counts its uses; the last word is the status
                assert counters[:-1].tolist() == [launches] * (batch * KV_HEADS)
            assert native.attention_status(counters, batch, KV_HEADS) == 0
            err = (out.float() - expected).pow(2).sum().div(expected.pow(2).sum()).sqrt().item()
            assert err < 6e-3, f"pos={pos_value} repeat={repeat}: rel-RMS error {err}"  # bf16 output rounding ~2e-3
            worst = (out.float() - expected).abs().max().item()
            assert worst <= 2.0**-7 * expected.abs().max().item() + 1e-3, f"pos={pos_value}: max error {worst}"


@pytest.mark.parametrize("group", [3, 6])  # the scalar and the tensor-core kernel
def test_decode_attention_position_outside_the_cache_is_clamped(native, group):
    """A position past the cache reads the whole cache and nothing beyond it."""
    batch, splits = 2, 4
    q_heads = group * KV_HEADS
    k_cache, v_cache = _cache(16)
    k_cache, v_cache = k_cache[:batch].contiguous(), v_cache[:batch].contiguous()
    scratch, counters = native.attention_scratch(batch, q_heads, KV_HEADS, splits, torch.device("cuda"))
    q = torch.randn((batch, q_heads * 128), device="cuda").bfloat16()
    out = torch.empty_like(q)
    native.decode_attention(q, k_cache, v_cache, torch.tensor(MAX_LEN + 5, device="cuda"), out, scratch, counters,
                            q_heads, KV_HEADS, splits)
    expected = attention_reference(q.view(batch, q_heads, 128), k_cache, v_cache, MAX_LEN - 1, group)
    torch.cuda.synchronize()
    assert (out.float() - expected).pow(2).sum().div(expected.pow(2).sum()).sqrt().item() < 6e-3
    assert native.attention_status(counters, batch, KV_HEADS) == 0


def test_decode_attention_rejects_misaligned_pointers(native):
    """The kernels read 16 bytes per lane: a q that starts 8 bytes into an allocation is refused
    on the host (nothing is launched)."""
    batch, q_heads = 2, 6
    k_cache, v_cache = _cache(16)
    k_cache, v_cache = k_cache[:batch].contiguous(), v_cache[:batch].contiguous()
    buffer = torch.zeros(batch * q_heads * 128 + 8, device="cuda", dtype=torch.bfloat16)
    q = buffer[4:4 + batch * q_heads * 128].view(batch, q_heads * 128)
    out = torch.empty((batch, q_heads * 128), device="cuda", dtype=torch.bfloat16)
    scratch, counters = native.attention_scratch(batch, q_heads, KV_HEADS, 1, torch.device("cuda"))
    with pytest.raises(native.FdkError):
        native.decode_attention(q, k_cache, v_cache, torch.tensor(5, device="cuda"), out, scratch, counters,
                                q_heads, KV_HEADS, 1)
    torch.cuda.synchronize()


def rope_reference(x, pos: int, theta: float):
    """transformers' Llama: inv_freq and angles in fp32, cos/sin rounded to the activation type,
    x * cos + rotate_half(x) * sin in that type.  x [..., 128] bf16."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32, device=x.device) / 128))
    freqs = float(pos) * inv_freq
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos().to(x.dtype), emb.sin().to(x.dtype)
    x1, x2 = x[..., :64], x[..., 64:]
    rotated = torch.cat((-x2, x1), dim=-1)
    return (x * cos) + (rotated * sin)


@pytest.mark.parametrize("pos_value", [0, 1024, 2175])
def test_rope_append_matches_rotate_half_formula(native, pos_value):
    rows, q_heads, theta = 3, 6, 500000.0
    gen = torch.Generator(device="cuda").manual_seed(pos_value + 1)
    qkv = torch.randn((rows, (q_heads + 2 * KV_HEADS) * 128), generator=gen, device="cuda").bfloat16()
    k_cache = torch.full((rows, KV_HEADS, MAX_LEN, 128), 7.0, device="cuda", dtype=torch.bfloat16)
    v_cache = torch.full((rows, KV_HEADS, MAX_LEN, 128), 7.0, device="cuda", dtype=torch.bfloat16)
    q_out = torch.empty((rows, q_heads * 128), device="cuda", dtype=torch.bfloat16)
    native.rope_append(qkv, torch.tensor(pos_value, device="cuda"), q_out, k_cache, v_cache, q_heads, KV_HEADS, theta)
    torch.cuda.synchronize()
    heads = qkv.view(rows, q_heads + 2 * KV_HEADS, 128)
    want_q = rope_reference(heads[:, :q_heads], pos_value, theta)
    want_k = rope_reference(heads[:, q_heads: q_heads + KV_HEADS], pos_value, theta)
    want_v = heads[:, q_heads + KV_HEADS:]

    def close(got, want, what):
        # cos/sin of a large angle may differ in the last fp32 place between two correct
        # implementations, which can move a bf16 result by one unit in the last place
        diff = (got.float() - want.float()).abs()
        assert bool((diff <= 2.0**-7 * want.float().abs() + 1e-6).all()), f"{what}: more than one bf16 place off"
        assert (diff > 0).float().mean().item() < 0.02, f"{what}: too many last-place differences"

    close(q_out.view(rows, q_heads, 128), want_q, "q")
    close(k_cache[:, :, pos_value], want_k, "k")
    assert torch.equal(v_cache[:, :, pos_value], want_v)
    untouched = torch.ones(MAX_LEN, dtype=torch.bool, device="cuda")
    untouched[pos_value] = False
    assert bool((k_cache[:, :, untouched] == 7.0).all()) and bool((v_cache[:, :, untouched] == 7.0).all())


@pytest.mark.parametrize("pos_value", [MAX_LEN, MAX_LEN + 100, -1])
def test_rope_append_outside_the_cache_writes_nothing(native, pos_value):
    rows, q_heads = 2, 3
    qkv = torch.randn((rows, (q_heads + 2 * KV_HEADS) * 128), device="cuda").bfloat16()
    k_cache = torch.full((rows, KV_HEADS, 64, 128), 7.0, device="cuda", dtype=torch.bfloat16)
    v_cache = k_cache.clone()
    guard = torch.full((4096,), 7.0, device="cuda", dtype=torch.bfloat16)  # allocated right after the caches
    q_out = torch.full((rows, q_heads * 128), float("nan"), device="cuda", dtype=torch.bfloat16)
    # max_len is taken from the cache shape (64): positions 2304, 2404 and -1 are all outside it
    native.rope_append(qkv, torch.tensor(pos_value, device="cuda"), q_out, k_cache, v_cache, q_heads, KV_HEADS, 500000.0)
    torch.cuda.synchronize()
    assert bool((k_cache == 7.0).all()) and bool((v_cache == 7.0).all()) and bool((guard == 7.0).all())
    assert not bool(torch.isnan(q_out.float()).any())  # q is still rotated and written


@pytest.mark.parametrize("rows,n", [(1, 128256), (3, 1000), (16, 32000), (2, 7)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_argmax_matches_torch(native, rows, n, dtype):
    """fdk_argmax = torch.argmax on rows without ties; the lowest index among equal maxima; a NaN wins."""
    gen = torch.Generator(device="cuda").manual_seed(rows * n)
    x = torch.randn((rows, n), generator=gen, device="cuda").to(dtype)
    out = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
    native.argmax(x, out)
    picked = x.gather(1, out[:, None])[:, 0]
    assert torch.equal(picked, x.max(dim=1).values)          # a maximum ...
    is_max = x == x.max(dim=1, keepdim=True).values
    first = torch.where(is_max, torch.arange(n, device="cuda")[None, :], n).min(dim=1).values
    assert torch.equal(out, first)                           # ... and the first of them
    # ties, negative rows and a NaN
    y = torch.full((3, 100), -2.0, device="cuda", dtype=dtype)
    y[0, 40] = y[0, 70] = 5.0
    y[1, 99] = -1.0
    y[2, 13] = float("nan")
    y[2, 50] = 9.0
    out = torch.empty(3, dtype=torch.int64, device="cuda")
    native.argmax(y, out)
    assert out.tolist() == [40, 99, 13]


@pytest.mark.parametrize("group", [1, 2, 3, 4, 5, 6, 7, 8])
def test_decode_attention_on_a_grid_larger_than_the_gpu(native, group):
    """80 batch rows x 2 KV heads = 160 CTAs: more than the SMs, which selects the tensor-core
    kernel (two CTAs per SM) for every ratio, on an unsliced context."""
    batch, q_heads, max_len = 80, group * KV_HEADS, 320
    gen = torch.Generator(device="cuda").manual_seed(group)
    k_cache = torch.randn((batch, KV_HEADS, max_len, 128), generator=gen, device="cuda").bfloat16()
    v_cache = torch.randn((batch, KV_HEADS, max_len, 128), generator=gen, device="cuda").bfloat16()
    scratch, counters = native.attention_scratch(batch, q_heads, KV_HEADS, 1, torch.device("cuda"))
    for pos_value in (0, 7, 15, 16, 129, 300, 319):  # around the 16-key steps and the 128-key rounds of the CTA
        q = torch.randn((batch, q_heads * 128), generator=gen, device="cuda").bfloat16()
        out = torch.full((batch, q_heads * 128), float("nan"), device="cuda", dtype=torch.bfloat16)
        native.decode_attention(q, k_cache, v_cache, torch.tensor(pos_value, device="cuda"), out, scratch, counters,
                                q_heads, KV_HEADS, 1)
        expected = attention_reference(q.view(batch, q_heads, 128), k_cache, v_cache, pos_value, group)
        torch.cuda.synchronize()
        assert not bool(torch.isnan(out.float()).any())
        err = (out.float() - expected).pow(2).sum().div(expected.pow(2).sum()).sqrt().item()
        assert err < 6e-3, f"pos={pos_value}: rel-RMS error {err}"
        worst = (out.float() - expected).abs().max().item()
        assert worst <= 2.0**-7 * expected.abs().max().item() + 1e-3, f"pos={pos_value}: max error {worst}"
