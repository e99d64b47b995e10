"""Headline benchmark: packed-weight HBM GB/s of the fused 4-bit LUT GEMV.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): y = x . W^T with K = N = 8192, batch 1, 4-bit codes, block 64, a
16-entry k-means-like codebook -- the largest shape of the reference's kernel sweep
(`python -m fdk.bench -k 8192 -b 4 -m 1`, README of the reference).  One STEP is 32 passes
over `copies` independent weight sets (8 x 35.7 MB, more than the 126 MB L2, so every
pass streams from HBM), 256 GEMV launches captured once as a CUDA graph the way the
reference's harness does (src/fdk/bench.py:67-99) and replayed per step: about 3 ms, so that
even a 20-step run is timed over more than 50 ms and the clock samples fall under load.

Printed JSON line: `value` = packed-weight bytes (codes + block scales) of all GPUs per
second, device-timed with inputs resident in HBM; `e2e` = the same bytes per second
through the module's host-buffer call `QuantisedLinear.forward_host` (one C-ABI call per GEMV:
pinned x copied in, the projection, y copied out to pinned memory; the calls of a step are queued
asynchronously and the step's results awaited once); `roofline` relates the per-launch time to the measured HBM copy bandwidth;
`cpu_baseline` times the CPU oracle port of the reference operator on the host cores.

N > 1: the kernel benchmark does not shard (one matrix, one GPU); ranks run independent
replicas (weak scaling), timed as the max over ranks.  The part of the path that does shard,
the decode loop, is reported in the extra `decode` object: tokens/s of a 4-bit custom-llama
with tensor parallelism over the N ranks (NCCL all-reduce after each row-parallel projection).

`--impl reference` times the reference's CPU path (eager torch dequantise-then-matmul,
the oracle port) on the same workload, one GEMV per step.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "fused-dequantisation-kernels_b200"))

K = N = 8192
BITS = 4
BLOCK = 64
BATCH = 1
COPIES = 8
PASSES = 32  # passes over the weight sets per step (one CUDA graph): a step is ~3 ms, 20 steps > 50 ms
WORKLOAD = f"gemv_lut k={K} n={N} m={BATCH} bits={BITS} g={BLOCK} codebook=kmeans16 copies={COPIES}"
PACKED_BYTES = N * K * BITS // 8 + N * (K // BLOCK) * 2  # codes + bf16 block scales


def measured_traffic(key: str):
    """DRAM bytes (read + write) of one launch, from the table kept beside the ncu summaries
    (profiles/dram_traffic.json); null when the kernel's source has changed since the capture."""
    import hashlib

    try:
        table = json.loads((ROOT / "profiles" / "dram_traffic.json").read_text())
        entry = table[key]
        source = ROOT / "fused-dequantisation-kernels_b200" / "csrc" / entry["source"]
        if hashlib.sha256(source.read_bytes()).hexdigest()[:16] != entry["source_sha16"]:
            return None
        return int(entry["dram_bytes"])
    except Exception:
        return None


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------
# synthetic inputs (seeded; same recipe for every arm)
# ---------------------------------------------------------------------------------------


def kmeans_codebook(bits: int, seed: int):
    import torch

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(20000, generator=g).sort().values
    c = torch.quantile(x, (torch.arange(2**bits) + 0.5) / 2**bits)
    for _ in range(8):
        idx = torch.bucketize(x, (c[1:] + c[:-1]) / 2)
        c = torch.stack([x[idx == i].mean() if (idx == i).any() else c[i] for i in range(2**bits)])
    return c.sort().values.bfloat16()


def make_weight(seed: int, device):
    """bf16 W ~ N(0, 1/K), drawn on `device`."""
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn((N, K), generator=g, device=device, dtype=torch.float32) * K**-0.5).bfloat16()


# ---------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------


class ClockSampler:
    """Samples nvidia-smi while the timed region runs (reading only)."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[tuple[float, str]] = []  # (time the line was read, line)
        self.window = (0.0, float("inf"))

    def mark(self, start: float, end: float) -> None:
        """Only samples read between these two time.monotonic() values count (the timed region)."""
        self.window = (start, end)

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.03)  # let the last sample of the region be read
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for when, line in self.lines:
            if not (self.window[0] <= when <= self.window[1] + 0.02):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference operator, timed on the host cores
# ---------------------------------------------------------------------------------------


def cpu_reference_times(reps: int, warmup: int) -> tuple[list[float], int, str]:
    """Seconds per GEMV of the eager-torch reference operator on the host (all cores)."""
    import torch

    sys.path.insert(0, str(ROOT / "oracle"))
    import fdk_oracle_torch as OT

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cpu = torch.device("cpu")
    w = make_weight(100, cpu)
    data, scale, table = OT.quantise_weight(w, BITS, BLOCK, lut=kmeans_codebook(BITS, 0))
    del w
    x = torch.randn((BATCH, K), generator=torch.Generator().manual_seed(1)).bfloat16()
    times = []
    for i in range(warmup + reps):
        t0 = time.perf_counter()
        OT.mm_lut_ref(x, data, table, scale)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return times, torch.get_num_threads(), f"{reps} GEMVs of the workload's shape, one weight set (eager torch dequantise-then-matmul, bf16)"


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times, cores, sample = cpu_reference_times(args.steps, args.warmup)
    mean = statistics.fmean(times)
    value = PACKED_BYTES / mean / 1e9
    line = {
        "impl": "reference",
        "metric": "packed_weight_gbs_gemv",
        "value": value,
        "unit": "GB/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": mean * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": "one GEMV on the host CPU (bounded sample of the GPU arm's step)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------


def run_gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from fdk import models, native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fdk kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    native.lib()

    # `copies` quantised layers through the public API (quantise -> QuantisedLinear)
    config = models.QuantisationConfig(bits=BITS, block_size=BLOCK)
    codebook = kmeans_codebook(BITS, 0).to(device)
    layers = []
    for c in range(COPIES):
        w = make_weight(100 + c, device)
        layer = models.QuantisedLinear.create(w, config, lut=codebook)
        layer.tiled()
        layers.append(layer)
        del w
    gx = torch.Generator(device=device).manual_seed(1)
    xs = [torch.randn((BATCH, K), generator=gx, device=device).bfloat16() for _ in range(COPIES)]
    outs = [torch.empty((BATCH, N), device=device, dtype=torch.bfloat16) for _ in range(COPIES)]

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        def one_pass():
            for layer, x, out in zip(layers, xs, outs):
                native.linear_lut(x, layer.tiled(), layer.lut, out, N, K, BITS, pdl=True)

        one_pass()  # allocates this stream's workspace before capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(PASSES):
                one_pass()
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        torch.cuda.synchronize()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            time.sleep(0.05)  # the sampler is up before the region starts
            barrier()
            t_start = time.monotonic()
            start.record()
            for _ in range(args.steps):
                graph.replay()
            end.record()
            barrier()
            clocks.mark(t_start, time.monotonic())
        elapsed_ms = start.elapsed_time(end)

        # end to end through the module's host-buffer call, per GEMV: pinned x -> device,
        # the projection, y -> pinned host memory, stream synchronisation (QuantisedLinear.forward_host).
        e2e_steps = max(1, min(args.steps, 5))
        e2e_s = float("nan")
        if not args.kernel_only:
            x_host = [x.cpu().pin_memory() for x in xs]
            y_host = torch.empty((BATCH, N), dtype=torch.bfloat16).pin_memory()
            for layer, xh in zip(layers, x_host):  # warm-up
                layer.forward_host(xh, y_host)
            barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                # one step = PASSES x COPIES GEMVs, each with its own copy in and copy out, queued
                # without waiting for each other; the step's results are awaited once, at its end
                for _ in range(PASSES):
                    for layer, xh in zip(layers, x_host):
                        layer.forward_host(xh, y_host, synchronise=False)
                torch.cuda.synchronize()  # every y of the step has landed in host memory
            e2e_s = time.perf_counter() - t0
        status = native.device_status(device)
        if status != 0:  # a bounded wait ran out inside the timed region: the numbers mean nothing
            raise RuntimeError(f"device-side status word {status} after the timed region")

    t = torch.tensor([elapsed_ms, e2e_s], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_s = float(t[0]), float(t[1])

    decode = None
    if not args.kernel_only and not args.no_decode:
        decode = decode_extra(device, world, rank)

    launches = PASSES * COPIES * args.steps
    ms_per_step = elapsed_ms / args.steps
    value = world * PASSES * COPIES * PACKED_BYTES / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * PASSES * COPIES * e2e_steps * PACKED_BYTES / e2e_s / 1e9
    per_launch_s = elapsed_ms * 1e-3 / launches
    achieved = PACKED_BYTES / per_launch_s / 1e9
    peak, peak_kind = measured_peak_gbs()

    if rank == 0:
        cpu_baseline = None
        if world == 1 and not args.kernel_only:  # the CPU arm is reported beside the single-GPU number only
            cpu_times, cores, sample = cpu_reference_times(reps=20, warmup=2)
            cpu_value = PACKED_BYTES / statistics.fmean(cpu_times) / 1e9
            cpu_baseline = {"value": cpu_value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
        traffic = measured_traffic(f"linear_lut_kernel bits={BITS} n={N} k={K} m={BATCH}")
        line = {
            "metric": "packed_weight_gbs_gemv",
            "value": value,
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "step": f"{PASSES} passes over {COPIES} weight sets = {PASSES * COPIES} GEMV launches, one CUDA graph, programmatic dependent launch",
                "cache": f"inputs larger than L2: {COPIES} x {PACKED_BYTES} B of weights cycled",
                "parallelism": "replicas" if world > 1 else "single",
            },
            "roofline": {
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": traffic,
                "peak_kind": f"of {peak_kind}",
                "kernel": "linear_lut_kernel<4,1,bf16>",
                "us_per_launch": per_launch_s * 1e6,
            },
            "cpu_baseline": cpu_baseline,
            "e2e": {
                "value": e2e_value,
                "unit": "GB/s",
                "h2d_bytes_per_step": PASSES * COPIES * BATCH * K * 2,
                "d2h_bytes_per_step": PASSES * COPIES * BATCH * N * 2,
            },
            "gpu_launches": launches,
            "clocks": clocks.summary(),
            "decode": decode,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # captured graphs that hold collectives must be gone before the communicator is
        import gc

        gc.collect()
        torch.cuda.synchronize()
        dist.destroy_process_group()


def decode_extra(device, world: int, rank: int) -> dict:
    """Second figure of the metric: greedy-decode tokens/s of the custom-llama shapes with 4-bit
    block-64 weights, one decode step per CUDA-graph replay as the reference times it
    (src/fdk/models.py:313-340), synthetic KV-cache contents of the stated context.
      N = 1: "b200-4B" (32 layers, d 3072, FFN 8192, 24/8 heads), context 1024, batch 1 to 256,
             lm_head in bf16 as the reference leaves it; the same with lm_head quantised too at
             batch 1 and 16; the same loop with bf16 nn.Linear layers (cuBLAS) at batch 1 and 16; and
             "b200-31B" (64 layers, d 6144, FFN 20480, 48/8 heads), context 2048, batch 1.
      N > 1: the models tensor parallel over the N ranks (31B at context 2048, batch 1 and 16; 4B
             at context 1024, batch 1): the o and down projections push their partial sums to
             every rank from the kernel and the next RMSNorm adds them; the same run with NCCL
             all-reduces instead is timed beside it; and the logits of a two-layer slice are
             compared with those of the same slice run on one rank."""
    import torch

    from fdk import llama, models, native

    lut = kmeans_codebook(4, 0).to(device)
    config = models.QuantisationConfig(4, 64)
    out = {"bits": 4, "block_size": 64, "tp": world, "runs": []}

    def run(model, name, batch, context, reps=30):
        r = models.benchmark(model, batch, reps, context)
        return {"model": name, "batch": batch, "context": context, "tokens_per_s": batch / r.avg_time,
                "weight_gbs": r.bytes_rw / r.avg_time / 1e9}

    try:
        tp = llama.TensorParallel(rank, world, fused=True)
        if world == 1:
            dims = models.get_custom_llama_dims("b200-4B")
            model = llama.LlamaDecoder.random_init(dims, config, device, tp, lut=lut)
            for batch in (1, 4, 16, 64, 256):
                out["runs"].append(run(model, "custom-llama-b200-4B", batch, 1024))
            del model
            torch.cuda.empty_cache()
            # every linear layer quantised, lm_head included (the reference's default leaves it in
            # bf16, skip="^lm_head$", as the runs above do)
            every = models.QuantisationConfig(4, 64, skip=None)
            model = llama.LlamaDecoder.random_init(dims, every, device, tp, lut=lut)
            for batch in (1, 16):
                entry = run(model, "custom-llama-b200-4B", batch, 1024)
                entry["lm_head"] = "4-bit"
                out["runs"].append(entry)
            del model
            torch.cuda.empty_cache()
            base = llama.LlamaDecoder.random_init(dims, None, device, tp)
            for batch in (1, 16):
                entry = run(base, "custom-llama-b200-4B", batch, 1024)
                entry["layers"] = "bf16 cuBLAS"
                out["runs"].append(entry)
            del base
            torch.cuda.empty_cache()
            big = llama.LlamaDecoder.random_init(models.get_custom_llama_dims("b200-31B"), config, device, tp, lut=lut)
            out["runs"].append(run(big, "custom-llama-b200-31B", 1, 2048, reps=10))
            del big
            torch.cuda.empty_cache()
        else:
            out["slice_check"] = tp_slice_check(device, world, rank, lut)
            for name, context, batches in (("b200-31B", 2048, (1, 16)), ("b200-4B", 1024, (1,))):
                dims = models.get_custom_llama_dims(name)
                model = llama.LlamaDecoder.random_init(dims, config, device, tp, lut=lut)
                for batch in batches:
                    entry = run(model, f"custom-llama-{name}", batch, context, reps=20)
                    entry["tp_reduce"] = "fused push" if model.exchange is not None else "nccl"
                    if model.exchange is not None:
                        entry["exchange_status"] = native.tp_exchange_status(model.exchange)
                    model.close()
                    model.tp = llama.TensorParallel(rank, world)
                    entry["nccl_tokens_per_s"] = batch / models.benchmark(model, batch, 20, context).avg_time
                    model.tp = tp
                    out["runs"].append(entry)
                model.close()
                del model
                torch.cuda.empty_cache()
        # the flat keys of the first run, as earlier records had them
        first = out["runs"][0]
        out.update(model=first["model"], batch=first["batch"], context=first["context"], tokens_per_s=first["tokens_per_s"],
                   weight_gbs=first["weight_gbs"])
        bf16 = [r for r in out["runs"] if r.get("layers") == "bf16 cuBLAS" and r["batch"] == 1]
        if bf16:
            out["bf16_cublas_tokens_per_s"] = bf16[0]["tokens_per_s"]
    except Exception as e:  # the headline line must still be printed
        out["error"] = repr(e)
    return out


def tp_slice_check(device, world: int, rank: int, lut) -> dict:
    """Values, not just status words: a two-layer slice of the 4B shape decoded for four steps on
    all ranks (fused exchange) and on one rank alone (rank 0, same seed); the logits must agree
    to the tolerance of the tensor-parallel tests (rel-RMS 2e-2: the ranks add partial sums of
    bf16-rounded products in another order) and be identical on every rank."""
    import dataclasses

    import torch
    import torch.distributed as dist

    from fdk import llama, models

    dims = dataclasses.replace(models.get_custom_llama_dims("b200-4B"), num_hidden_layers=2, vocab_size=4096)
    config = models.QuantisationConfig(4, 64)
    ids = torch.randint(0, dims.vocab_size, (2, 4), generator=torch.Generator().manual_seed(3)).to(device)

    def decode(tp):
        model = llama.LlamaDecoder.random_init(dims, config, device, tp, seed=11, lut=lut)
        model.allocate(2, 8)
        with torch.no_grad():
            logits = torch.stack([model(ids[:, t].contiguous()).float() for t in range(4)], dim=1)
        torch.cuda.synchronize()
        model.close()
        return logits

    sharded = decode(llama.TensorParallel(rank, world, fused=True))
    gathered = [torch.empty_like(sharded) for _ in range(world)]
    dist.all_gather(gathered, sharded)
    same = all(torch.equal(g, gathered[0]) for g in gathered)
    result = {"identical_on_all_ranks": bool(same)}
    if rank == 0:
        alone = decode(llama.TensorParallel(0, 1))
        err = (sharded - alone).pow(2).sum().div(alone.pow(2).sum()).sqrt().item()
        result.update(rel_rms_vs_one_rank=err, ok=bool(same and err < 2e-2))
    return result


def main() -> None:
    global COPIES, PASSES, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    # profiling aids (the defaults are the benchmark): smaller footprint, kernel launches only
    ap.add_argument("--copies", type=int, default=COPIES, help="weight sets cycled per step")
    ap.add_argument("--passes", type=int, default=PASSES, help="passes over the weight sets per step")
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end, CPU and decode legs")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode tokens/s leg")
    args = ap.parse_args()
    PASSES = args.passes
    if args.copies != COPIES:
        COPIES = args.copies
        WORKLOAD = f"gemv_lut k={K} n={N} m={BATCH} bits={BITS} g={BLOCK} codebook=kmeans16 copies={COPIES}"
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
