"""GPU parity tests: every call goes through the C-ABI library (fdk.native) and is checked
against the CPU oracle on the same seeded inputs.  Bit-exact for byte / index work
(repack, unpack, dequantise); rel-RMS error <= 1e-2 (the reference's own tolerance for its
LUT kernels, src/fdk/kernels.py:196,502) for the fused products -- measured values are
~1e-3, the bf16 output rounding."""

import numpy as np
import pytest
import torch

import fdk_oracle as O
import tiled_layout as TL
from gpu_util import from_bits, oracle_dense, random_problem, to_bits

pytestmark = pytest.mark.gpu

TOL = 1e-2

SHAPES = [(64, 64), (16, 256), (100, 384), (256, 1024), (200, 4096), (1024, 768)]


@pytest.fixture(scope="module")
def native():
    from fdk import native as nat

    nat.lib()
    return nat


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("n,k", SHAPES)
def test_repack_matches_host_model_and_round_trips(native, bits, n, k):
    codes, lut, scale, _ = random_problem(n, k, bits, 1, seed=n + k + bits)
    d_codes = torch.from_numpy(codes).cuda()
    d_scale = from_bits(scale)
    tiled = native.repack(d_codes, d_scale, n, k, bits, 64)
    assert tiled.numel() == TL.tiled_size(n, k, bits)
    assert np.array_equal(tiled.cpu().numpy(), TL.repack(codes, scale, bits))
    back_codes, back_scale = native.unpack(tiled, n, k, bits, 64, torch.bfloat16)
    assert np.array_equal(back_codes.cpu().numpy(), codes)
    assert np.array_equal(to_bits(back_scale), scale)


@pytest.mark.parametrize("block_size", [128, 256])
def test_repack_wider_blocks(native, block_size):
    n, k, bits = 96, 512, 4
    codes, lut, scale, x = random_problem(n, k, bits, 3, seed=9, g=block_size)
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, block_size)
    assert np.array_equal(tiled.cpu().numpy(), TL.repack(codes, scale, bits))
    w = native.dequantise_tiled(tiled, from_bits(lut), n, k, bits)
    assert np.array_equal(to_bits(w), O.dequantise(codes, lut, scale))


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("n,k", SHAPES)
def test_dequantise_bit_exact(native, bits, n, k):
    codes, lut, scale, _ = random_problem(n, k, bits, 1, seed=3 * n + k + bits)
    expected = oracle_dense(codes, lut, scale, bits, k)
    d_codes, d_lut, d_scale = torch.from_numpy(codes).cuda(), from_bits(lut), from_bits(scale)
    w = native.dequantise(d_codes, d_lut, d_scale, bits)
    assert np.array_equal(to_bits(w), expected)
    tiled = native.repack(d_codes, d_scale, n, k, bits, 64)
    w2 = native.dequantise_tiled(tiled, d_lut, n, k, bits)
    assert np.array_equal(to_bits(w2), expected)


def test_dequantise_bit_exact_fp16_and_small_blocks(native):
    n, k, bits = 64, 256, 4
    rng = np.random.default_rng(5)
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    base = O.f32_to_f16(np.arange(-8, 8, dtype=np.float32))
    lut = np.stack([base[np.arange(256) >> 4], base[np.arange(256) & 15]], axis=1)
    scale = O.f32_to_f16(rng.random((n, k // 32), dtype=np.float32))
    w = native.dequantise(torch.from_numpy(codes).cuda(), from_bits(lut, torch.float16), from_bits(scale, torch.float16), bits)
    assert np.array_equal(to_bits(w), O.dequantise(codes, lut, scale, dtype="f16"))


@pytest.mark.parametrize("name,bit_list", [("quantise_linspace.npz", [8, 4, 2, 1]), ("quantise_codebook.npz", [4, 2])])
def test_dequantise_golden_vectors(native, golden_dir, name, bit_list):
    z = np.load(golden_dir / name)
    for bits in bit_list:
        p = f"b{bits}_"
        w = native.dequantise(torch.from_numpy(z[p + "weight_data"]).cuda(), from_bits(z[p + "lut"]), from_bits(z[p + "scale"]), bits)
        assert np.array_equal(to_bits(w), z[p + "w_deq"]), f"bits={bits}"


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("m", [1, 2, 5, 8, 9, 16, 17, 40])
@pytest.mark.parametrize("n,k", [(64, 64), (100, 384), (256, 1024), (1024, 768)])
def test_linear_lut_matches_oracle(native, bits, m, n, k):
    codes, lut, scale, x = random_problem(n, k, bits, m, seed=m + n + k + bits)
    expected = O.mm_dense(x, oracle_dense(codes, lut, scale, bits, k))
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, 64)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.linear_lut(from_bits(x), tiled, from_bits(lut), out, n, k, bits)
    err = O.rmsen(O.bf16_to_f32(expected), O.bf16_to_f32(to_bits(out)))
    assert err < TOL, f"rmsen={err}"
    assert err < 4e-3  # fp32 accumulation + one bf16 output rounding (2^-9 / sqrt(3) .. 2^-8 / sqrt(3))


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("n,k", [(4096, 4096), (3072, 8192), (8192, 3072), (13824, 5120)])
def test_linear_lut_large_shapes(native, bits, n, k):
    m = 3
    codes, lut, scale, x = random_problem(n, k, bits, m, seed=n + bits)
    expected = O.mm_dense(x, oracle_dense(codes, lut, scale, bits, k))
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, 64)
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    native.linear_lut(from_bits(x), tiled, from_bits(lut), out, n, k, bits)
    err = O.rmsen(O.bf16_to_f32(expected), O.bf16_to_f32(to_bits(out)))
    assert err < 3e-3, f"rmsen={err}"


def test_linear_lut_is_deterministic(native):
    n, k, bits, m = 4096, 4096, 4, 4
    codes, lut, scale, x = random_problem(n, k, bits, m, seed=1)
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, 64)
    d_x, d_lut = from_bits(x), from_bits(lut)
    outs = []
    for _ in range(5):
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        native.linear_lut(d_x, tiled, d_lut, out, n, k, bits)
        outs.append(to_bits(out))
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    ws = native.workspace(torch.device("cuda", torch.cuda.current_device()))
    torch.cuda.synchronize()
    assert native.device_status() == 0


@pytest.mark.parametrize("n,k,m", [(256, 512, 3), (256, 512, 40), (1024, 2048, 200)])
def test_linear_lut_fp16(native, n, k, m):
    """fp16 activations, scales and table (the Marlin selectors' type): the GEMV kernel up to 16
    rows, the tensor-core kernel above."""
    bits = 4
    rng = np.random.default_rng(11)
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    base = O.f32_to_f16(np.arange(-8, 8, dtype=np.float32))
    lut = np.stack([base[np.arange(256) >> 4], base[np.arange(256) & 15]], axis=1)
    scale = O.f32_to_f16(rng.random((n, k // 64), dtype=np.float32) * np.float32(0.01))
    x = O.f32_to_f16(rng.standard_normal((m, k)).astype(np.float32))
    expected = O.mm_dense(x, O.dequantise(codes, lut, scale, dtype="f16"), dtype="f16")
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale, torch.float16), n, k, bits, 64)
    out = torch.empty((m, n), dtype=torch.float16, device="cuda")
    native.linear_lut(from_bits(x, torch.float16), tiled, from_bits(lut, torch.float16), out, n, k, bits)
    assert O.rmsen(O.f16_to_f32(expected), O.f16_to_f32(to_bits(out))) < 2e-3


@pytest.mark.parametrize("bits,m,n,k", [(4, 1, 512, 256), (4, 3, 16384, 3072), (2, 8, 1024, 512), (1, 16, 640, 1024), (4, 12, 2048, 192), (3, 2, 128, 256)])
def test_linear_lut_silu_pairs_equals_two_steps(native, bits, m, n, k):
    """FDK_FLAG_SILU_PAIRS: the projection kernel writes silu(gate) * up itself; what the plain
    projection followed by fdk_silu_mul (group 32) gives -- bit for bit: both run the same kernel."""
    codes, lut, scale, x = random_problem(n, k, bits, m, seed=3 * n + m)
    scale = O.f32_to_bf16(O.bf16_to_f32(scale) * np.float32(8.0))  # products of order one: SiLU is not just x / 2
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, 64)
    d_x, d_lut = from_bits(x), from_bits(lut)
    full = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    native.linear_lut(d_x, tiled, d_lut, full, n, k, bits)
    want = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
    native.silu_mul(full, want, group=32)
    got = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.linear_lut(d_x, tiled, d_lut, got, n, k, bits, silu_pairs=True)
    torch.cuda.synchronize()
    assert np.array_equal(to_bits(got), to_bits(want))  # the same kernel both ways (up to 16 rows)
    assert native.device_status() == 0
    with pytest.raises(native.FdkError):  # batches above 16 rows do not take the flag
        native.linear_lut(torch.zeros((17, k), dtype=torch.bfloat16, device="cuda"), tiled, d_lut,
                          torch.empty((17, n // 2), dtype=torch.bfloat16, device="cuda"), n, k, bits, silu_pairs=True)


def test_linear_lut_cuda_graph_capture(native):
    n, k, bits, m = 1024, 1024, 4, 1
    codes, lut, scale, x = random_problem(n, k, bits, m, seed=2)
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, 64)
    d_x, d_lut = from_bits(x), from_bits(lut)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        native.linear_lut(d_x, tiled, d_lut, out, n, k, bits)  # allocates this stream's workspace
        torch.cuda.synchronize()
        eager = to_bits(out).copy()
        out.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(3):
                native.linear_lut(d_x, tiled, d_lut, out, n, k, bits)
        graph.replay()
        torch.cuda.synchronize()
    assert np.array_equal(to_bits(out), eager)


def test_error_statuses_on_device(native):
    x = torch.zeros((1, 128), dtype=torch.bfloat16, device="cuda")
    tiled = torch.zeros(native.tiled_size(64, 128, 4), dtype=torch.uint8, device="cuda")
    lut = torch.zeros((256, 2), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((1, 64), dtype=torch.bfloat16, device="cuda")
    lib = native.lib()
    ws = native.workspace(x.device)
    args = lambda xp, wsp, wsn: lib.fdk_linear_lut(xp, tiled.data_ptr(), lut.data_ptr(), None, out.data_ptr(), 1, 64, 128, 4, 0, wsp, wsn, 0, None)
    assert args(x.data_ptr() + 2, ws.data_ptr(), ws.numel()) == 3  # misaligned x
    assert args(x.data_ptr(), ws.data_ptr(), 100) == 6  # workspace too small
    assert args(x.data_ptr(), None, 0) == 6
    assert args(x.data_ptr(), ws.data_ptr(), ws.numel()) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("m,n,k", [(17, 128, 64), (32, 192, 256), (64, 1024, 1024), (200, 4096, 4096), (192, 768, 4096), (256, 2048, 3072), (300, 256, 512),
                                   (24, 320, 192), (40, 64, 448), (256, 5120, 1728)])
def test_tensor_core_gemm_matches_oracle(native, bits, m, n, k):
    """Batches above 16 rows run the tcgen05 kernel, whose W is the reference's bf16 W bit for
    bit; its outputs differ from the oracle's only by fp32 summation order and the last bf16
    rounding."""
    codes, lut, scale, x = random_problem(n, k, bits, m, seed=m + n + k + bits)
    expected = O.mm_dense(x, oracle_dense(codes, lut, scale, bits, k))
    tiled = native.repack(torch.from_numpy(codes).cuda(), from_bits(scale), n, k, bits, 64)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.linear_lut(from_bits(x), tiled, from_bits(lut), out, n, k, bits)
    torch.cuda.synchronize()
    assert native.device_status() == 0
    err = O.rmsen(O.bf16_to_f32(expected), O.bf16_to_f32(to_bits(out)))
    assert err < 4e-3, f"rmsen={err}"
    mismatched = np.mean(to_bits(out) != expected)
    assert mismatched < 0.05  # a few last-bit roundings at most


def test_reference_mm_test_recipe(native):
    """test_mm_4b_lut8 of the reference (src/fdk/kernels.py:492-502) through the operator API."""
    from fdk import bench

    bench.test_mm_4b_lut8()
    bench.test_mv_4b_lut8()


@pytest.mark.parametrize("m", [1, 5, 16, 40])
def test_forward_host_equals_forward(m):
    """QuantisedLinear.forward_host (fdk_linear_lut_host: copy in, projection, copy out, synchronise)
    gives the bits of forward() on the same activations."""
    from fdk import models

    torch.manual_seed(m)
    w = (torch.randn((640, 512), device="cuda") * 0.05).bfloat16()
    layer = models.QuantisedLinear.create(w, models.QuantisationConfig(4, 64))
    x_host = torch.randn((m, 512)).bfloat16().pin_memory()
    out_host = torch.full((m, 640), float("nan")).bfloat16().pin_memory()
    back = layer.forward_host(x_host, out_host)
    assert back is out_host  # valid on return: no synchronisation needed here
    want = layer(x_host.cuda())
    torch.cuda.synchronize()
    assert torch.equal(out_host, want.cpu())
    assert torch.equal(layer.forward_host(x_host), want.cpu())  # allocates a pinned output itself
    # host memory that is not page-locked takes the cudaMemcpyAsync route inside the library
    pageable_x = x_host.clone()
    pageable_out = torch.full((m, 640), float("nan")).bfloat16()
    assert not pageable_x.is_pinned() and not pageable_out.is_pinned()
    layer.forward_host(pageable_x, pageable_out)
    assert torch.equal(pageable_out, want.cpu())
    # queued without synchronisation: valid once the stream has been synchronised
    outs = [torch.full((m, 640), float("nan")).bfloat16().pin_memory() for _ in range(3)]
    for o in outs:
        layer.forward_host(x_host, o, synchronise=False)
    torch.cuda.synchronize()
    assert all(torch.equal(o, want.cpu()) for o in outs)
