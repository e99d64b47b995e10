"""Times the decode attention kernel alone:  python -m fdk.attention_bench [--batch ...]

One query token per batch row against a static bf16 KV cache (the layout of fdk.llama), a CUDA
graph of 20 launches replayed 10 times, CUDA events; prints microseconds per launch, the rate
at which keys and values are read, and the largest deviation from torch's
scaled_dot_product_attention on the same inputs."""

from __future__ import annotations

import argparse

import torch

from . import native


def run(batch: int, context: int, splits: int, q_heads: int, kv_heads: int, device: torch.device) -> None:
    max_len = context + 129
    k_cache = torch.randn((batch, kv_heads, max_len, 128), device=device).bfloat16()
    v_cache = torch.randn((batch, kv_heads, max_len, 128), device=device).bfloat16()
    q = torch.randn((batch, q_heads * 128), device=device).bfloat16()
    out = torch.empty_like(q)
    pos = torch.tensor(context, device=device)
    scratch, counters = native.attention_scratch(batch, q_heads, kv_heads, splits, device)
    call = lambda: native.decode_attention(q, k_cache, v_cache, pos, out, scratch, counters, q_heads, kv_heads, splits)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        call()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(20):
                call()
        graph.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(10):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1000 / 200
    kv_bytes = batch * kv_heads * (context + 1) * 128 * 2 * 2
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.view(batch, q_heads, 1, 128), k_cache[:, :, : context + 1], v_cache[:, :, : context + 1], enable_gqa=True
    ).view(batch, -1)
    err = (out.float() - ref.float()).abs().max().item()
    print(f"batch {batch:3d} context {context} slices {splits:2d}: {us:7.2f} us  {kv_bytes / us / 1e3:7.1f} GB/s  max error {err:.2e}", flush=True)


def _main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--batch", type=int, nargs="+", default=[1, 16, 64, 256])
    parser.add_argument("--context", type=int, default=1024)
    parser.add_argument("--slices", type=int, nargs="+", default=None, help="context slices per (row, KV head); default: as fdk.llama picks")
    parser.add_argument("--q-heads", type=int, default=24)
    parser.add_argument("--kv-heads", type=int, default=8)
    args = parser.parse_args()
    device = torch.device("cuda")
    for batch in args.batch:
        picked = max(1, min((args.context + 35) // 128, 148 // (batch * args.kv_heads), 16))
        for splits in args.slices or [picked]:
            run(batch, args.context, splits, args.q_heads, args.kv_heads, device)


if __name__ == "__main__":
    _main()
