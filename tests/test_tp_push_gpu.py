"""Row-parallel projection fused with its all-reduce, checked on ONE GPU.

The ranks of a tensor-parallel group are emulated in sequence on one device: each "rank" owns
an exchange buffer, every push stores into all of them, and only after every rank's push has
been launched is any reduce launched -- so the reduce never waits for a kernel that has not
run yet (kernels that wait on one another must not share a GPU).  The sum of the pushed
partial products must equal what the plain entry points give: linear_lut per rank, the partial
outputs added in fp32 in rank order and rounded to bf16, then rmsnorm with that sum as `delta`
-- bit for bit up to 8 rows, where linear_lut runs the same kernel as the push."""

import numpy as np
import pytest
import torch

from gpu_util import from_bits, random_problem, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from fdk import native as n

    return n


def _exchange_buffers(native, tp, slot_elems):
    nbytes = native.tp_exchange_bytes(tp, slot_elems)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(tp)]
    exs = [native.make_exchange(tp, r, [b.data_ptr() for b in bufs], slot_elems) for r in range(tp)]
    return bufs, exs


@pytest.mark.parametrize("bits,m,n,k,tp", [
    (4, 1, 512, 256, 2), (4, 2, 5120, 1024, 2), (4, 5, 1024, 640, 3), (4, 8, 2048, 512, 2), (4, 16, 1024, 256, 2),
    (2, 1, 1024, 512, 4), (1, 3, 512, 1024, 2), (8, 1, 512, 192, 2), (3, 2, 512, 512, 2), (4, 1, 8192, 2048, 8),
    (4, 9, 512, 128, 2),
])
def test_push_then_reduce_equals_plain_path(native, bits, m, n, k, tp):
    slot = 16 * n
    bufs, exs = _exchange_buffers(native, tp, slot)
    rng = np.random.default_rng(bits * 1000 + m)
    problems = []
    for r in range(tp):
        codes, lut, scale, x = random_problem(n, k, bits, m, seed=17 * r + bits + m)
        tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, 64)
        problems.append((tiled, from_bits(lut)))
    weight = torch.randn(n, device="cuda").to(torch.bfloat16)
    h_plain = torch.randn((m, n), generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    h_rank = [h_plain.clone() for _ in range(tp)]
    for step in range(5):  # odd and even halves of the double buffer, several times over
        xs = [from_bits(rng.integers(0x3C00, 0x4000, size=(m, k), dtype=np.uint16) ^ rng.integers(0, 2, size=(m, k), dtype=np.uint16) * 0x8000) for _ in range(tp)]
        total = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        for r in range(tp):
            part = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            native.linear_lut(xs[r], problems[r][0], problems[r][1], part, n, k, bits)
            total += part.float()  # rank order, fp32
        delta = total.to(torch.bfloat16)
        want_norm = torch.empty_like(h_plain)
        native.rmsnorm(h_plain, delta, weight, want_norm, 1e-5)

        for r in range(tp):
            native.linear_lut_push(xs[r], problems[r][0], problems[r][1], exs[r], n, k, bits, pdl=(step % 2 == 1))
        for r in range(tp):
            got_norm = torch.empty_like(h_plain)
            native.rmsnorm_reduce(h_rank[r], exs[r], weight, got_norm, 1e-5)
            torch.cuda.synchronize()
            if m <= 16:  # the plain products come from the same kernel
                assert np.array_equal(to_bits(h_rank[r]), to_bits(h_plain)), (step, r)
                assert np.array_equal(to_bits(got_norm), to_bits(want_norm)), (step, r)
            else:  # 17 rows and more: the plain products come from the tensor-core kernel
                assert (h_rank[r].float() - h_plain.float()).abs().max() <= 0.05 * h_plain.float().abs().max(), (step, r)
                h_rank[r].copy_(h_plain)  # keep the streams identical for the next step
    for r in range(tp):
        assert native.tp_exchange_status(exs[r]) == 0
        words = bufs[r][:256].view(torch.int32).cpu()
        assert words[32].item() == 5 and words[33].item() == 0  # reduces done; finished-CTA count back at zero
    assert native.device_status() == 0


def test_push_argument_checks(native):
    n, k = 128, 64
    bufs, exs = _exchange_buffers(native, 2, 16 * n)
    codes, lut, scale, x = random_problem(n, k, 4, 1, seed=1)
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, 4, 64)
    with pytest.raises(native.FdkError) as e:  # batches above 16 rows do not push
        native.linear_lut_push(torch.zeros((17, k), dtype=torch.bfloat16, device="cuda"), tiled, from_bits(lut), exs[0], n, k, 4)
    assert e.value.status == 2
    small = native.make_exchange(2, 0, [b.data_ptr() for b in bufs], 64)
    with pytest.raises(native.FdkError) as e:  # slot too small for [1, 128]
        native.linear_lut_push(from_bits(x), tiled, from_bits(lut), small, n, k, 4)
    assert e.value.status == 2
    bad_rank = native.make_exchange(2, 2, [b.data_ptr() for b in bufs], 16 * n)
    with pytest.raises(native.FdkError) as e:
        native.linear_lut_push(from_bits(x), tiled, from_bits(lut), bad_rank, n, k, 4)
    assert e.value.status == 1
    h = torch.zeros((1, n), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(native.FdkError) as e:
        native.rmsnorm_reduce(h, small, h[0], torch.empty_like(h), 1e-5)
    assert e.value.status == 2


def test_reduce_gives_up_when_a_word_never_comes(native):
    """Nothing was pushed by rank 1: the reduce of rank 0's first push waits out its limit (two
    seconds), records status 1 and returns; the context stays usable."""
    n, k = 128, 64
    bufs, exs = _exchange_buffers(native, 2, 16 * n)
    codes, lut, scale, x = random_problem(n, k, 4, 1, seed=2)
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, 4, 64)
    native.linear_lut_push(from_bits(x), tiled, from_bits(lut), exs[0], n, k, 4)
    h = torch.zeros((1, n), dtype=torch.bfloat16, device="cuda")
    native.rmsnorm_reduce(h, exs[0], torch.ones(n, dtype=torch.bfloat16, device="cuda"), torch.empty_like(h), 1e-5)
    torch.cuda.synchronize()
    assert native.tp_exchange_status(exs[0]) == 1
    assert torch.isfinite(h.float()).all()


def test_exchange_buffer_create_and_destroy(native):
    nbytes = native.tp_exchange_bytes(2, 1024)
    assert nbytes == 256 + 2 * 2 * 1024 * 4
    ptr, handle = native.tp_buffer_create(nbytes, torch.device("cuda", 0))
    assert ptr % 256 == 0 and len(handle) == 64
    native.tp_buffer_destroy(ptr)
