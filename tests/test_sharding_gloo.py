"""World-size-2 gloo tests of the row-sharding host logic (CPU; the per-rank matvec is done by the oracle here)."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vinf_3080ti_b200.sharding import NO_INDEX, pick_best, shard_rows


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import dequant_np as O
        from vinf_3080ti_b200.gguf_types import GGUFTensorType as T, row_bytes
        from vinf_3080ti_b200.sharding import combine_argmax, gather_rows
        from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

        rng = np.random.default_rng(7)  # same seed on every rank: the same full tensor
        rows, cols, m = 1030, 512, 3
        raw = synthetic_blocks(T.Q6_K, rows, cols, rng)
        x = synthetic_activations(m, cols, rng)
        full = O.matvec(raw, int(T.Q6_K), rows, cols, x)
        b, e = shard_rows(rows, rank, world)
        mine = O.matvec(raw[b:e], int(T.Q6_K), e - b, cols, x)  # this rank's rows only
        gathered = gather_rows(torch.from_numpy(mine), rows)
        ok_gather = bool(np.array_equal(gathered.numpy(), full))
        vals = torch.from_numpy(mine.max(axis=1))
        ids = torch.from_numpy(mine.argmax(axis=1) + b)
        ok_argmax = combine_argmax(vals, ids).tolist() == [int(v) for v in O.argmax_rows(full)]
        out[rank] = (ok_gather, ok_argmax, row_bytes(T.Q6_K, cols) * (e - b))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gather_rows_and_combine_argmax():
    world = 2
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert all(out[r][0] and out[r][1] for r in range(world)), dict(out)
        assert sum(out[r][2] for r in range(world)) == 1030 * 420  # the shards cover the tensor exactly once


def test_shard_rows_cover_every_benchmark_row_count():
    for rows in (17408, 5120, 6144, 1024, 151936, 1030):
        for world in (1, 2, 4, 8):
            cuts = [shard_rows(rows, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == rows
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
            assert all(b % 2 == 0 for b, _ in cuts)
    with pytest.raises(ValueError):
        shard_rows(10, 3, 2)


def test_pick_best_tie_and_empty_rules():
    inf = float("inf")
    values = torch.tensor([[1.0, 5.0, -inf, float("nan")], [1.0, 4.0, -inf, 2.0]], dtype=torch.float64)
    ids = torch.tensor([[7, 3, NO_INDEX, 1], [2, 9, NO_INDEX, 8]])
    assert pick_best(values, ids).tolist() == [2, 3, NO_INDEX, 8]
