"""Tensor-parallel sharding of the quantised projections, checked on CPU with two gloo ranks:
column-parallel shards concatenate, and row-parallel shards sum (all-reduce), to the unsharded
layer -- with the packed tensors of every shard bit-identical to slices of the unsharded ones
(block scales run along K inside a row, so shard-then-quantise equals quantise-then-shard)."""

import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fdk import kernels, llama, models


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp = llama.TensorParallel(rank, world)
        dims = models.LlamaDims("tiny", 256, 1, 4, 2, 512, vocab_size=64)
        cfg = models.QuantisationConfig(4, 64, kernel="torch.compile")
        g = torch.Generator().manual_seed(5)
        d = dims.head_dim
        draw = lambda n, k: (torch.randn((n, k), generator=g) * 0.05).bfloat16()
        q, k, v = draw(4 * d, 256), draw(2 * d, 256), draw(2 * d, 256)
        o, gate, up, down = draw(256, 4 * d), draw(512, 256), draw(512, 256), draw(256, 512)
        qkv_w, o_w, gu_w, down_w = llama.LlamaDecoder._shard_layer_weights(q, k, v, o, gate, up, down, dims, tp)
        x = (torch.randn((3, 256), generator=g)).bfloat16()

        # column parallel: this rank's q rows equal the matching rows of the unsharded layer (every
        # head's rows in the order the rotary epilogue wants: ROPE_ROW_ORDER)
        full_q = models.QuantisedLinear.create(q, cfg)
        mine = models.QuantisedLinear.create(qkv_w, cfg)
        rows = llama.shard_rows(4, tp)
        n_q = (rows.stop - rows.start) * d
        order = torch.tensor(llama.ROPE_ROW_ORDER)
        paired = lambda t: t.unflatten(0, (-1, d))[:, order].flatten(0, 1)  # rows of every head reordered
        assert torch.equal(mine.weight_data[:n_q], paired(full_q.weight_data[rows.start * d: rows.stop * d]))
        assert torch.equal(mine.scale[:n_q], paired(full_q.scale[rows.start * d: rows.stop * d]))
        y_mine = mine(x)[:, :n_q].contiguous()
        gathered = [torch.empty_like(y_mine) for _ in range(world)]
        dist.all_gather(gathered, y_mine)
        assert torch.equal(torch.cat(gathered, dim=1), paired(full_q(x).T).T)

        # row parallel: packed shard = byte-column slice; partial products all-reduce to the full one
        full_down = models.QuantisedLinear.create(down, cfg)
        mine_down = models.QuantisedLinear.create(down_w, cfg)
        cols = llama.shard_rows(512, tp)
        assert torch.equal(mine_down.weight_data, full_down.weight_data[:, cols.start // 2: cols.stop // 2])
        assert torch.equal(mine_down.scale, full_down.scale[:, cols.start // 64: cols.stop // 64])
        act = torch.randn((3, 512), generator=g).bfloat16()
        partial = mine_down(act[:, cols].contiguous()).float()
        tp.all_reduce(partial)
        full = full_down(act).float()
        err = (partial - full).pow(2).sum().div(full.pow(2).sum()).sqrt().item()
        assert err < 1e-2, err
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_sharding_identities_two_ranks():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = 29500 + os.getpid() % 2000
        procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(results) == {0: "ok", 1: "ok"}


def test_shard_helpers_reject_uneven_splits():
    import pytest

    with pytest.raises(AssertionError):
        llama.shard_rows(10, llama.TensorParallel(0, 4))
    with pytest.raises(AssertionError):
        llama.shard_columns(96, llama.TensorParallel(0, 2))
    assert llama.shard_columns(6144, llama.TensorParallel(7, 8)) == slice(5376, 6144)


def test_gate_up_rows_alternate_in_groups_of_32():
    """The fused gate|up weight holds, per 64 rows, 32 gate rows and then the 32 matching up
    rows (what FDK_FLAG_SILU_PAIRS and fdk_silu_mul with group 32 expect), for every rank."""
    dims = models.LlamaDims("tiny", 128, 1, 4, 2, 256, vocab_size=64)
    g = torch.Generator().manual_seed(1)
    d = dims.head_dim
    draw = lambda n, k: torch.randn((n, k), generator=g).bfloat16()
    q, k, v, o = draw(4 * d, 128), draw(2 * d, 128), draw(2 * d, 128), draw(128, 4 * d)
    gate, up, down = draw(256, 128), draw(256, 128), draw(128, 256)
    for rank in range(2):
        tp = llama.TensorParallel(rank, 2)
        _, _, gu, down_s = llama.LlamaDecoder._shard_layer_weights(q, k, v, o, gate, up, down, dims, tp)
        rows = llama.shard_rows(256, tp)
        assert gu.shape == (2 * (rows.stop - rows.start), 128)
        blocks = gu.unflatten(0, (-1, 2, llama.PAIR_GROUP))
        assert torch.equal(blocks[:, 0].flatten(0, 1), gate[rows])
        assert torch.equal(blocks[:, 1].flatten(0, 1), up[rows])
        assert torch.equal(down_s, down[:, rows])
