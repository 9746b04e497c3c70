"""Output-row sharding of the quantized matvec over several GPUs (one process per GPU, torch.distributed).

Rows of W are independent, so rank g owns a contiguous slice of the output rows of every weight tensor and
computes y[:, slice] locally; the slices are combined with an all-gather, and the argmax of a sharded LM head
with a local argmax followed by an all-gather of (value, index) pairs.  The reference has no multi-GPU code
(it is a single-GPU engine); the tie rule of the combined argmax is the one of its argmax_kernel
(engine/csrc/megakernel/qwen_runtime.cu:851-876): highest value, lowest index among equals, 0x7fffffff when no
rank saw a value above -inf.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

NO_INDEX = 0x7FFFFFFF


def shard_rows(rows: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the rows owned by `rank`.  Every slice but the last has (rows // world) rounded down to
    an even number of rows, which keeps a slice of a 2-byte-aligned block format 4-byte aligned like the tensor."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    per = (rows // world) & ~1
    if per == 0:
        raise ValueError(f"{rows} rows cannot be split over {world} ranks")
    begin = rank * per
    end = rows if rank == world - 1 else begin + per
    return begin, end


def gather_rows(y_local: torch.Tensor, rows: int, group=None) -> torch.Tensor:
    """y_local: [M, rows of this rank] -> [M, rows] on every rank (all-gather of the row slices)."""
    world = dist.get_world_size(group)
    m = y_local.shape[0]
    sizes = [shard_rows(rows, k, world)[1] - shard_rows(rows, k, world)[0] for k in range(world)]
    widest = max(sizes)  # the last slice may be a few rows longer: pad to equal sizes for the collective
    mine = y_local.contiguous()
    if mine.shape[1] < widest:
        mine = torch.cat([mine, mine.new_zeros((m, widest - mine.shape[1]))], dim=1)
    parts = [torch.empty((m, widest), dtype=y_local.dtype, device=y_local.device) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    return torch.cat([p[:, :n] for p, n in zip(parts, sizes)], dim=1)


def combine_argmax(values: torch.Tensor, ids: torch.Tensor, group=None) -> torch.Tensor:
    """values [M] (fp32 best logit of this rank), ids [M] (its global row, NO_INDEX if none) -> global ids [M]."""
    world = dist.get_world_size(group)
    pair = torch.stack([values.to(torch.float64), ids.to(torch.float64)], dim=0).contiguous()
    pairs = [torch.empty_like(pair) for _ in range(world)]
    dist.all_gather(pairs, pair, group=group)
    return pick_best(torch.stack([p[0] for p in pairs]), torch.stack([p[1] for p in pairs]).to(torch.int64))


def pick_best(values: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """values, ids: [ranks, M] -> [M]; highest value wins, lowest id on ties, NO_INDEX if nothing is above -inf."""
    values = torch.where(torch.isnan(values) | (ids == NO_INDEX), torch.full_like(values, float("-inf")), values)
    best = values.max(dim=0).values
    candidate = torch.where((values == best) & (values > float("-inf")), ids, torch.full_like(ids, NO_INDEX))
    return candidate.min(dim=0).values


class ExchangeLayout:
    """Byte layout of a rank's exchange region for the fused push (Runtime.qmv_push): gathered vectors first, then
    the flag table unsigned[n_slots][8], then this rank's own push counts unsigned[n_slots]."""

    def __init__(self, data_bytes: int, n_slots: int) -> None:
        self.data_bytes = (int(data_bytes) + 255) // 256 * 256
        self.n_slots = int(n_slots)
        self.flag_off = self.data_bytes
        self.count_off = self.flag_off + self.n_slots * 8 * 4
        self.total = (self.count_off + self.n_slots * 4 + 255) // 256 * 256


def connect_exchange(rt, layout: ExchangeLayout, group=None) -> list[int]:
    """Creates this rank's exchange region, trades CUDA IPC handles with the other ranks of the process group and
    configures the runtime.  Returns every rank's region address as seen from this process."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    handle, own = rt.exchange_create(layout.total)
    handles: list = [None] * world
    dist.all_gather_object(handles, handle, group=group)
    addrs = [own if k == rank else rt.exchange_open(handles[k]) for k in range(world)]
    rt.exchange_config(rank, addrs, layout.flag_off, layout.count_off, layout.n_slots)
    dist.barrier(group)
    return addrs
