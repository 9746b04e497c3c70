"""The fused matvec + all-gather (qmv_push) on ONE GPU: two runtimes play two ranks that share the device, run one after
the other (a rank never waits for a flag that has not been raised yet, except in the last test, which lets a bounded
wait run out on purpose - one rank pushes a slot the other never pushes - and checks that it is reported instead of hanging)."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import dequant_np as O
from vinf_3080ti_b200.gguf_types import GGUFTensorType as T
from vinf_3080ti_b200.sharding import ExchangeLayout, shard_rows
from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

pytestmark = pytest.mark.gpu


def rel_l2(got, ref):
    return float(np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref))


@pytest.fixture()
def two_ranks(codebooks):
    from vinf_3080ti_b200.runtime import Runtime

    m, rows, cols, rows2 = 3, 1032, 1024, 520
    layout = ExchangeLayout(4 * m * (rows + rows2), n_slots=3)
    rts = [Runtime(codebooks["iq3s_grid"], codebooks) for _ in range(2)]
    addrs = [rt.exchange_create(layout.total)[1] for rt in rts]
    for rank, rt in enumerate(rts):
        rt.exchange_config(rank, addrs, layout.flag_off, layout.count_off, layout.n_slots)
        rt.bind("gathered", addrs[rank], m * rows)                       # slot 0's vector, [m][rows]
        rt.bind("gathered2", addrs[rank] + 4 * m * rows, m * rows2)      # slot 1's vector
        rt.bind("flags", addrs[rank] + layout.flag_off, layout.n_slots * 8)
    yield rts, layout, (m, rows, cols, rows2)
    for rt in rts:
        rt.close()


def test_push_gathers_slices_on_every_rank_and_chains(two_ranks, codebooks):
    rts, layout, (m, rows, cols, rows2) = two_ranks
    rng = np.random.default_rng(11)
    raw = synthetic_blocks(T.Q6_K, rows, cols, rng)
    raw2 = synthetic_blocks(T.Q4_K, rows2, rows - 8, rng)  # consumes the first 1024 gathered values of each row... see below
    x = synthetic_activations(m, cols, rng)
    ref = O.matvec(raw, int(T.Q6_K), rows, cols, x, codebooks)
    for rank, rt in enumerate(rts):
        b, e = shard_rows(rows, rank, 2)
        rt.upload("w", raw[b:e], int(T.Q6_K), cols, e - b)
        rt.alloc("x", m * cols)
        rt.alloc("y", m * (e - b))
        rt.write("x", x)
    for epoch in (1, 2):  # two passes: the flags carry the number of pushes of the slot
        for rank, rt in enumerate(rts):
            b, e = shard_rows(rows, rank, 2)
            rt.qmv_push("w", "x", "y", m, slot=0, dst_off=0, rows_total=rows, row_begin=b)
            rt.synchronize()
        for rt in rts:
            got = rt.read_array("gathered").reshape(m, rows)
            assert rel_l2(got, ref) <= 1e-5
            flags = np.frombuffer(rt.read("flags"), dtype=np.uint32).reshape(layout.n_slots, 8)
            assert list(flags[0, :2]) == [epoch, epoch] and not flags[1:].any()
    # a consumer whose input is the gathered vector: the flags of slot 0 are already up, so its wait passes at once
    x2 = rts[0].read_array("gathered").reshape(m, rows)[:, : rows - 8].copy()
    ref2 = O.matvec(raw2, int(T.Q4_K), rows2, rows - 8, x2, codebooks)
    for rank, rt in enumerate(rts):
        b, e = shard_rows(rows2, rank, 2)
        rt.upload("w2", raw2[b:e], int(T.Q4_K), rows - 8, e - b)
        rt.alloc("x2", m * (rows - 8))
        rt.write("x2", x2)
        rt.alloc("y2", m * (e - b))
        rt.qmv_push("w2", "x2", "y2", m, slot=1, dst_off=4 * m * rows, rows_total=rows2, row_begin=b, wait_slot=0)
        rt.synchronize()
    for rt in rts:
        assert rel_l2(rt.read_array("gathered2").reshape(m, rows2), ref2) <= 1e-5


def test_push_of_a_group_launch_fills_both_gathered_vectors(two_ranks, codebooks):
    """Two tensors that share x in one launch per rank (q/k-like), short enough to be split by columns as well: each
    tensor's slice lands in its own gathered vector on every rank, one flag slot covers the launch."""
    rts, layout, (m, rows, cols, rows2) = two_ranks
    rng = np.random.default_rng(14)
    cols = 2048
    raw_a, raw_b = synthetic_blocks(T.Q6_K, rows, cols, rng), synthetic_blocks(T.Q6_K, rows2, cols, rng)
    x = synthetic_activations(m, cols, rng)
    ref_a, ref_b = O.matvec(raw_a, int(T.Q6_K), rows, cols, x, codebooks), O.matvec(raw_b, int(T.Q6_K), rows2, cols, x, codebooks)
    for rank, rt in enumerate(rts):
        (ba, ea), (bb, eb) = shard_rows(rows, rank, 2), shard_rows(rows2, rank, 2)
        rt.upload("wa", raw_a[ba:ea], int(T.Q6_K), cols, ea - ba)
        rt.upload("wb", raw_b[bb:eb], int(T.Q6_K), cols, eb - bb)
        rt.alloc("x", m * cols)
        rt.alloc("ya", m * (ea - ba))
        rt.alloc("yb", m * (eb - bb))
        rt.write("x", x)
        rt.qmv_push_group(["wa", "wb"], "x", ["ya", "yb"], m, slot=0, dst_offs=[0, 4 * m * rows], rows_totals=[rows, rows2],
                          row_begins=[ba, bb])
        rt.synchronize()
        assert rel_l2(rt.read_array("ya").reshape(m, ea - ba), ref_a[:, ba:ea]) <= 1e-5
    for rt in rts:
        assert rel_l2(rt.read_array("gathered").reshape(m, rows), ref_a) <= 1e-5
        assert rel_l2(rt.read_array("gathered2").reshape(m, rows2), ref_b) <= 1e-5
        flags = np.frombuffer(rt.read("flags"), dtype=np.uint32).reshape(layout.n_slots, 8)
        assert list(flags[0, :2]) == [1, 1]


def test_push_with_fused_argmax_reports_global_rows(two_ranks, codebooks):
    rts, layout, (m, rows, cols, rows2) = two_ranks
    rng = np.random.default_rng(12)
    raw = synthetic_blocks(T.Q6_K, rows, cols, rng)
    x = synthetic_activations(m, cols, rng)
    ref = O.matvec(raw, int(T.Q6_K), rows, cols, x, codebooks)
    best = []
    for rank, rt in enumerate(rts):
        b, e = shard_rows(rows, rank, 2)
        rt.upload("w", raw[b:e], int(T.Q6_K), cols, e - b)
        rt.set_argmax_row_base("w", b)
        rt.alloc("x", m * cols)
        rt.alloc("y", m * (e - b))
        rt.write("x", x)
        rt.qmv_push("w", "x", "y", m, slot=0, dst_off=0, rows_total=rows, row_begin=b, with_argmax=True)
        best.append(rt.argmax_fetch(m, with_values=True))
    import torch

    from vinf_3080ti_b200.sharding import pick_best

    ids = pick_best(torch.tensor([b[1] for b in best], dtype=torch.float64), torch.tensor([b[0] for b in best]))
    assert ids.tolist() == [int(v) for v in O.argmax_rows(ref)]


def test_a_wait_that_nothing_satisfies_runs_out_and_is_reported(two_ranks):
    rts, layout, (m, rows, cols, rows2) = two_ranks
    rt = rts[0]
    rng = np.random.default_rng(13)
    rt.upload("w", synthetic_blocks(T.Q8_0, 64, 256, rng), int(T.Q8_0), 256, 64)
    rt.alloc("x", m * 256)
    rt.alloc("y", m * 64)
    rt.qmv_push("w", "x", "y", m, slot=2, dst_off=0, rows_total=64, row_begin=0)  # this rank pushes slot 2, the other never does
    rt.synchronize()
    rt.qmv_push("w", "x", "y", m, slot=-1, dst_off=0, rows_total=64, row_begin=0, wait_slot=2)
    with pytest.raises(RuntimeError, match="status 2"):
        rt.synchronize()
    rt.qmv("w", "x", "y", m)  # the context is still usable
    rt.synchronize()
