"""Kernel micro-benchmarks -- drop-in for the reference's `python -m fdk.bench`
(src/fdk/bench.py): same flags, same registry names, same timing method (CUDA graph of
`inner_reps` calls cycling through `copies` argument sets, replayed `outer_reps` times
between CUDA events), same JSONL rows, plus roofline fields.

Registry (reference names, bench.py:396-410):
  mv_ref, mm_ref             torch.matmul (cuBLAS) on 16-bit weights
  mv, mm                     the reference has Triton kernels here; cuBLAS stands in
  mv_lut8_ref, mm_lut8_ref   torch dequantise-then-matmul (eager)
  mv_lut8_ref_unscaled, mm_lut8_ref_unscaled   the same without block scales
  mv_lut8, mm_lut8           the native fused kernels of libfdk_b200
  marlin                     the native kernel in its fp16 / linear-grid configuration
"""

from __future__ import annotations

import datetime
import gc
import itertools
import json
import math
import os
import re
import subprocess
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch
from torch import Tensor

from . import kernels, native

LOG_DIR = Path("out/dev")


def _current_timestamp() -> str:
    return datetime.datetime.now().isoformat(timespec="seconds").replace(":", "-")


def _meta() -> dict[str, Any]:
    try:
        commit = subprocess.check_output(["git", "rev-parse", "HEAD"], stderr=subprocess.DEVNULL).decode().strip()
    except Exception:  # not a git checkout
        commit = None
    cuda = torch.cuda.is_available()
    return dict(
        device=torch.cuda.get_device_name(torch.cuda.current_device()) if cuda else "cpu",
        cuda_version=torch.version.cuda,
        torch_version=torch.__version__,
        fdk_b200_version=native.lib().fdk_version(),
        commit=commit,
    )


class Log:
    """JSONL log at out/dev/{key}-{timestamp}.jsonl; every row carries the run's metadata."""

    def __init__(self, key: str) -> None:
        self.id = f"{key}-{_current_timestamp()}"
        self.meta = dict(id=self.id, **_meta())
        LOG_DIR.mkdir(parents=True, exist_ok=True)
        self.path = LOG_DIR / f"{self.id}.jsonl"
        self.file = self.path.open("w", encoding="utf-8")

    def __call__(self, entry: dict[str, Any]) -> None:
        print(json.dumps({**entry, **self.meta}), file=self.file, flush=True)

    def __enter__(self) -> "Log":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.file.close()


def measure_time(fn: Callable[[int], None], inner_reps: int, outer_reps: int) -> tuple[float, float]:
    """Mean seconds per call and its standard error.  `inner_reps` calls fn(0..inner_reps-1)
    are captured in one CUDA graph on a side stream; the graph is replayed `outer_reps` times,
    each replay bracketed by events."""
    # One untimed pass over every argument set: the native operators repack a weight matrix into
    # the kernels' tile layout the first time they see it, and that one-time conversion must
    # neither be captured into the graph (it would be replayed with every call) nor be timed.
    for i in range(inner_reps):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(torch.cuda.Stream()):
        fn(0)  # the side stream's own workspace is allocated before capture
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for i in range(inner_reps):
                fn(i)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times: list[float] = []
    for _ in range(outer_reps):
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / inner_reps / 1000)
    t = torch.tensor(times)
    return t.mean().item(), t.std().item() / math.sqrt(len(t)) if len(t) > 1 else 0.0


def sizeof(*tensors: Tensor) -> int:
    return sum(t.element_size() * t.nelement() for t in tensors)


@dataclass
class Settings:
    m: int
    k: int
    n: int
    g: int
    bits: int
    copies: int
    inner_reps: int
    outer_reps: int

    def __post_init__(self) -> None:
        assert self.copies <= self.inner_reps, "insufficient inner_reps to cycle through all copies"

    def __str__(self) -> str:
        return f"m={self.m} k={self.k} n={self.n} g={self.g} bits={self.bits}"


@dataclass
class Result:
    name: str
    bytes_rw: int
    ops: int
    time_s: float
    stderr_s: float

    def __str__(self) -> str:
        return "  ".join(
            [
                f"{self.name:<25}",
                f"{self.time_s*1e6:>6.1f} us",
                f"{self.bytes_rw / self.time_s / 1e9:>6.1f} GB/s",
                f"{self.ops / self.time_s / 1e12:>6.1f} TFLOPS",
            ]
        )


class UnsupportedSettings(Exception):
    pass


BENCHMARKS: dict[str, "Benchmark"] = {}


class Benchmark:
    def __init__(self, name: str):
        assert name not in BENCHMARKS, f"Benchmark {name} already registered"
        self.name = name
        BENCHMARKS[name] = self

    def bytes_rw(self, s: Settings) -> int:
        raise NotImplementedError

    def ops(self, s: Settings) -> int:
        return 2 * s.m * s.k * s.n

    def setup(self, s: Settings) -> Callable[[int], None]:
        raise NotImplementedError

    def run(self, s: Settings) -> Result:
        torch.manual_seed(42)
        fn = self.setup(s)
        time_s, stderr_s = measure_time(fn, s.inner_reps, s.outer_reps)
        return Result(self.name, self.bytes_rw(s), self.ops(s), time_s, stderr_s)


class DenseBenchmark(Benchmark):
    """16-bit weights: fn(a, b, out) with a [m, k] (or [k] when vector=True), b [n, k]."""

    def __init__(self, name: str, fn: Callable[..., Any], vector: bool, dtype: torch.dtype = torch.bfloat16):
        super().__init__(name)
        self.fn, self.vector, self.dtype = fn, vector, dtype

    def bytes_rw(self, s: Settings) -> int:
        return (s.m * s.k + s.n * s.k + s.m * s.n) * self.dtype.itemsize

    def setup(self, s: Settings) -> Callable[[int], None]:
        if s.bits != 16 or (self.vector and s.m != 1):
            raise UnsupportedSettings(f"{self.name}: bits=16" + (", m=1" if self.vector else "") + " only")
        a_shape = (s.copies, s.k) if self.vector else (s.copies, s.m, s.k)
        o_shape = (s.copies, s.n) if self.vector else (s.copies, s.m, s.n)
        a = torch.randn(a_shape, device="cuda", dtype=self.dtype)
        b = torch.randn((s.copies, s.n, s.k), device="cuda", dtype=self.dtype)
        out = torch.empty(o_shape, device="cuda", dtype=self.dtype)
        return lambda i: self.fn(a[i % s.copies], b[i % s.copies], out=out[i % s.copies])


class LutBenchmark(Benchmark):
    """Packed weights: fn(a, bq, lut8, bs, out).  Inputs as the reference draws them
    (bench.py:239-256): uniform random bytes, linspace codebook, rand scales, seed 42."""

    def __init__(self, name: str, fn: Callable[..., Any], vector: bool, dtype: torch.dtype = torch.bfloat16):
        super().__init__(name)
        self.fn, self.vector, self.dtype = fn, vector, dtype

    def bytes_rw(self, s: Settings) -> int:
        # the lookup table is not counted: it is shared by all copies
        return s.n * (s.k * s.bits) // 8 + (s.m * s.k + s.n * (s.k // s.g) + s.m * s.n) * self.dtype.itemsize

    def setup(self, s: Settings) -> Callable[[int], None]:
        if s.bits not in (1, 2, 4, 8) or (self.vector and s.m != 1):
            raise UnsupportedSettings(f"{self.name}: bits in 1/2/4/8" + (", m=1" if self.vector else "") + " only")
        assert s.k % s.g == 0, "k must be divisible by g"
        torch.manual_seed(42)
        a_shape = (s.copies, s.k) if self.vector else (s.copies, s.m, s.k)
        o_shape = (s.copies, s.n) if self.vector else (s.copies, s.m, s.n)
        a = torch.randn(a_shape, device="cuda", dtype=self.dtype)
        bq = torch.randint(0, 256, (s.copies, s.n, (s.k * s.bits) // 8), device="cuda", dtype=torch.uint8)
        lut = torch.linspace(-1, 1, 2**s.bits, device="cuda", dtype=self.dtype)
        lut8 = torch.cartesian_prod(*[lut] * (8 // s.bits)).view(256, -1)
        bs = torch.rand((s.copies, s.n, s.k // s.g), device="cuda", dtype=self.dtype)
        out = torch.empty(o_shape, device="cuda", dtype=self.dtype)
        # one tensor object per weight set, made once: the native operators keep the repacked form
        # of a weight tensor per tensor OBJECT, and a fresh view per call would be repacked per call
        bqs, bss = list(bq.unbind(0)), list(bs.unbind(0))
        fn = lambda i: self.fn(a[i % s.copies], bqs[i % s.copies], lut8, bss[i % s.copies], out[i % s.copies])
        for i in range(s.copies):  # one-time work per weight set (the native path repacks it) stays out of the timing
            fn(i)
        return fn


class MarlinBenchmark(Benchmark):
    """The reference's Marlin row (bench.py:335-379): fp16, 4 bits, g in {64, 128}, inputs drawn
    as there (random int32 words in Marlin format, randn scales, a random [256, 2] table), through
    `fdk.marlin.mul`."""

    def __init__(self) -> None:
        super().__init__("marlin")

    def bytes_rw(self, s: Settings) -> int:
        # the lookup table and the workspace are not counted: they are shared by all copies
        return s.n * (s.k * 4) // 8 + (s.m * s.k + s.n * (s.k // s.g) + s.m * s.n) * torch.float16.itemsize

    def setup(self, s: Settings) -> Callable[[int], None]:
        if s.bits != 4 or s.g not in (64, 128):
            raise UnsupportedSettings("marlin: bits=4, g=64 or 128 only")
        assert s.k % s.g == 0, "k must be divisible by g"
        if s.k % 128 != 0 or s.n % 256 != 0:
            raise UnsupportedSettings("marlin: k a multiple of 128 and n of 256 only")
        from . import marlin

        torch.manual_seed(42)
        a = torch.randn((s.copies, s.m, s.k), device="cuda", dtype=torch.float16)
        ii = torch.iinfo(torch.int32)
        b = [torch.randint(ii.min, ii.max, (s.k // 16, 2 * s.n), device="cuda", dtype=torch.int32) for _ in range(s.copies)]
        bs = [torch.randn((s.k // s.g, s.n), device="cuda", dtype=torch.float16) for _ in range(s.copies)]
        out = torch.empty((s.copies, s.m, s.n), device="cuda", dtype=torch.float16)
        centroids = torch.randn((256, 2), device="cuda", dtype=torch.float16)
        workspace = torch.zeros(s.n // 128 * 16, dtype=torch.int)
        fn = lambda i: marlin.mul(a[i % s.copies], b[i % s.copies], out[i % s.copies], bs[i % s.copies], centroids, workspace)
        for i in range(s.copies):  # the one-time conversion of every weight set stays out of the timing
            fn(i)
        return fn


def mm_lut_ref_unscaled(a: Tensor, bq: Tensor, lut8: Tensor, bs: Tensor, out: Tensor | None = None) -> Tensor:
    b = lut8[bq.long()].flatten(start_dim=1)
    return torch.matmul(a, b.T, out=out)


def _ref_vec(fn: Callable[..., Tensor]) -> Callable[..., None]:
    return lambda a, bq, lut8, bs, out: out.copy_(fn(a, bq, lut8, bs))


# mv
DenseBenchmark("mv_ref", lambda a, b, out: torch.matmul(a[None], b.T, out=out[None]), vector=True)
DenseBenchmark("mv", kernels.run_mv, vector=True)
LutBenchmark("mv_lut8_ref_unscaled", _ref_vec(mm_lut_ref_unscaled), vector=True)
LutBenchmark("mv_lut8_ref", _ref_vec(kernels.mm_lut_ref), vector=True)
LutBenchmark("mv_lut8", kernels.run_mv_lut, vector=True)
# mm
DenseBenchmark("mm_ref", lambda a, b, out: torch.matmul(a, b.T, out=out), vector=False)
DenseBenchmark("mm", kernels.run_mm, vector=False)
LutBenchmark("mm_lut8_ref_unscaled", _ref_vec(mm_lut_ref_unscaled), vector=False)
LutBenchmark("mm_lut8_ref", _ref_vec(kernels.mm_lut_ref), vector=False)
LutBenchmark("mm_lut8", kernels.run_mm_lut, vector=False)
# marlin
MarlinBenchmark()


# Tests run before benchmarking, as the reference's CLI does (bench.py:416-424, kernels.py test_*)


def test_mv_4b_lut8() -> None:
    n, k, g = 128, 4096, 64
    torch.manual_seed(42)
    a = torch.randn((k,), device="cuda", dtype=torch.bfloat16)
    bq = torch.randint(0, 256, (n, k // 2), device="cuda", dtype=torch.uint8)
    lut4 = torch.linspace(-1, 1, 16, device="cuda", dtype=torch.bfloat16)
    lut8 = torch.cartesian_prod(lut4, lut4)
    bs = torch.rand((n, k // g), device="cuda", dtype=torch.bfloat16)
    out = torch.empty((n,), device="cuda", dtype=torch.bfloat16)
    kernels.run_mv_lut(a, bq, lut8, bs, out)
    kernels._assert_rmsen(kernels.mm_lut_ref(a, bq, lut8, bs), out, tol=1e-2)


def test_mm_4b_lut8() -> None:
    torch.manual_seed(42)
    m, k, n, g = 192, 4096, 768, 64
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randint(0, 256, (n, k // 2), device="cuda", dtype=torch.uint8)
    lut4 = torch.linspace(-1, 1, 16, device="cuda", dtype=torch.bfloat16)
    lut8 = torch.cartesian_prod(lut4, lut4)
    bs = torch.rand((n, k // g), device="cuda", dtype=torch.bfloat16)
    out = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    kernels.run_mm_lut(a, b, lut8, bs, out=out)
    kernels._assert_rmsen(kernels.mm_lut_ref(a, b, lut8, bs), out, tol=1e-2)


def run_tests() -> None:
    for name, fn in list(globals().items()):
        if name.startswith("test_") and callable(fn):
            fn()


def hbm_peak_gbs() -> tuple[float, str]:
    """The HBM bandwidth that fractions are quoted against: a measured value handed in through
    FDK_HBM_PEAK_GBS, else an earlier measurement on B200 as a fallback."""
    value = os.environ.get("FDK_HBM_PEAK_GBS")
    if value:
        try:
            return float(value), "measured"
        except ValueError:
            pass
    return 6650.0, "fallback"


def run_attention_benchmark(batches: list[int], context: int, q_heads: int, kv_heads: int, log: "Log",
                            slices: int | None = None) -> None:
    """Times the decode attention kernel alone: one query token per batch row against a static
    bf16 KV cache (the layout of fdk.llama), a CUDA graph of 20 launches replayed 10 times;
    logs microseconds per launch, the rate at which keys and values are read and the largest
    deviation from torch's scaled_dot_product_attention on the same inputs."""
    from . import native

    device = torch.device("cuda")
    peak, peak_kind = hbm_peak_gbs()
    for batch in batches:
        max_len = context + 129
        splits = slices or native.attention_slices(batch, q_heads, kv_heads, max_len)
        k_cache = torch.randn((batch, kv_heads, max_len, 128), device=device).bfloat16()
        v_cache = torch.randn((batch, kv_heads, max_len, 128), device=device).bfloat16()
        q = torch.randn((batch, q_heads * 128), device=device).bfloat16()
        out = torch.empty_like(q)
        pos = torch.tensor(context, device=device)
        scratch, counters = native.attention_scratch(batch, q_heads, kv_heads, splits, device)
        call = lambda _: native.decode_attention(q, k_cache, v_cache, pos, out, scratch, counters, q_heads, kv_heads, splits)
        time_s, stderr_s = measure_time(call, inner_reps=20, outer_reps=10)
        kv_bytes = batch * kv_heads * (context + 1) * 128 * 2 * 2
        ref = torch.nn.functional.scaled_dot_product_attention(
            q.view(batch, q_heads, 1, 128), k_cache[:, :, : context + 1], v_cache[:, :, : context + 1], enable_gqa=True
        ).view(batch, -1)
        err = (out.float() - ref.float()).abs().max().item()
        print(f"attention batch {batch:3d} context {context} slices {splits:2d}: {time_s * 1e6:7.2f} us  "
              f"{kv_bytes / time_s / 1e9:7.1f} GB/s  max error {err:.2e}", file=sys.stderr)
        log(dict(test="decode_attention", batch=batch, context=context, q_heads=q_heads, kv_heads=kv_heads, slices=splits,
                 avg_time=time_s, avg_time_stderr=stderr_s, kv_bytes=kv_bytes, kv_gbs=kv_bytes / time_s / 1e9,
                 hbm_peak_gbs=peak, hbm_peak_kind=peak_kind, max_abs_error=err))
        del k_cache, v_cache


def run_benchmarks(settings: Settings, only: str, include: str, exclude: str, log: Log) -> None:
    gc.collect()
    torch.cuda.empty_cache()
    kernels.clear_tiled_cache()
    peak, peak_kind = hbm_peak_gbs()
    header_printed = False
    for name, benchmark in BENCHMARKS.items():
        if only != "" and only != name:
            continue
        if include != "" and not re.search(include, name):
            continue
        if exclude != "" and re.search(exclude, name):
            continue
        try:
            result = benchmark.run(settings)
        except UnsupportedSettings:
            continue
        if not header_printed:
            print(f"# {settings}", file=sys.stderr)
            header_printed = True
        print(result, file=sys.stderr)
        row = dict(
            test=name, **settings.__dict__, bytes_rw=result.bytes_rw, ops=result.ops,
            avg_time=result.time_s, avg_time_stderr=result.stderr_s,
        )
        if settings.bits < 16:
            packed = settings.n * settings.k * settings.bits // 8 + settings.n * (settings.k // settings.g) * 2
            row.update(
                packed_weight_bytes=packed,
                packed_weight_gbs=packed / result.time_s / 1e9,
                hbm_peak_gbs=peak,
                hbm_peak_kind=peak_kind,
                hbm_fraction=packed / result.time_s / 1e9 / peak,
            )
        log(row)
        kernels.clear_tiled_cache()
    if header_printed:
        print(file=sys.stderr)


def _main() -> None:
    import argparse

    parser = argparse.ArgumentParser()
    parser.add_argument("-m", default=[1, 4, 16, 64, 256], type=int, nargs="+", help="Dimension m")
    parser.add_argument("-k", default=[4096], type=int, nargs="+", help="Dimension k")
    parser.add_argument("-n", default=["k"], nargs="+", help="Dimension n (int or 'k' for square)")
    parser.add_argument("-g", default=[64], type=int, nargs="+", help="Dimension g (block size)")
    parser.add_argument("-b", "--bits", default=[16, 4, 1], type=int, nargs="+", help="Bits per element")
    parser.add_argument("--copies", default=100, type=int, help="Number of arg copies")
    parser.add_argument("--inner-reps", default=100, type=int, help="Number of reps")
    parser.add_argument("--outer-reps", default=100, type=int, help="Number of rep samples")
    parser.add_argument("--profile", default="", help="Select a specific method to profile (skip tests)")
    parser.add_argument("--include", default="", help="Methods to include (regex)")
    parser.add_argument("--exclude", default="_ref", help="Methods to exclude (regex)")
    parser.add_argument("--pdl", action="store_true",
                        help="Launch the native LUT operators with programmatic dependent launch (as a decode loop does)")
    parser.add_argument("--attention", action="store_true",
                        help="Time the decode attention kernel instead (batch sizes from -m, see --context, --heads)")
    parser.add_argument("--context", default=1024, type=int, help="--attention: positions in the KV cache")
    parser.add_argument("--heads", default=[24, 8], type=int, nargs=2, help="--attention: query heads, KV heads")
    parser.add_argument("--slices", default=None, type=int, help="--attention: context slices (default: as fdk.llama picks)")
    args = parser.parse_args()

    if args.attention:
        with Log("py") as log:
            run_attention_benchmark(args.m, args.context, args.heads[0], args.heads[1], log, args.slices)
        return

    kernels.programmatic_launch = args.pdl
    if args.profile == "":
        run_tests()

    with Log("py") as log:
        keys = ["m", "k", "n", "g", "bits"]
        for values in itertools.product(*(getattr(args, k) for k in keys)):
            s = dict(zip(keys, values))
            s["n"] = s["k"] if s["n"] == "k" else int(s["n"])
            run_benchmarks(
                Settings(**s, copies=args.copies, inner_reps=args.inner_reps, outer_reps=args.outer_reps),
                only=args.profile, include=args.include, exclude=args.exclude, log=log,
            )


if __name__ == "__main__":
    _main()
