"""Batch sharding for multi-GPU inference: one process per GPU, contiguous batch shards,
weights replicated, no collective on the block's forward path.  The only exchange is one
all-gather of the (small) per-sample outputs at the end, as the reference's data-parallel
evaluation does with its leading device axis (main.py:522-561, src/training/distributed.py:
241-301).  Works with the `nccl` backend on GPUs and the `gloo` backend on CPU."""
from __future__ import annotations

import datetime
from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of rank's contiguous shard of n samples; the first n % world ranks get one
    extra sample, so shards differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_sizes(n: int, world: int) -> List[int]:
    return [shard_bounds(n, r, world)[1] - shard_bounds(n, r, world)[0] for r in range(world)]


def gather_outputs(local: torch.Tensor, n_total: int) -> torch.Tensor:
    """All-gathers per-sample outputs (shard_size, ...) from every rank into (n_total, ...),
    in rank order.  Ragged shards are padded to the largest shard for the collective."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    sizes = shard_sizes(n_total, world)
    if local.shape[0] != sizes[dist.get_rank()]:
        raise ValueError(f"rank {dist.get_rank()} holds {local.shape[0]} samples, expected "
                         f"{sizes[dist.get_rank()]}")
    mx = max(sizes)
    pad = torch.zeros((mx,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    out = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(out, pad)
    return torch.cat([o[:s] for o, s in zip(out, sizes)], dim=0)


def max_over_ranks(value: float, device) -> float:
    """Slowest rank's time: what a multi-GPU throughput figure must be computed from."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class PeerTimeout(RuntimeError):
    """Raised by check_peers: `missing` lists the ranks that did not report in time."""

    def __init__(self, missing):
        super().__init__(f"ranks {missing} did not report before the collective")
        self.missing = list(missing)


def check_peers(store, rank: int, world: int, step: int, timeout_s: float = 30.0) -> None:
    """Host-side roll call before a collective: every rank posts a key for `step` in the c10d
    store and waits, with a time limit, for the keys of all ranks.  A rank that died or raised
    before the collective never posts, so the others learn of it here, on the host, instead of
    hanging inside the all-gather (the reference probes NCCL the same way before its first pmap
    step and falls back to one device: main.py:1257-1288).  Raises PeerTimeout."""
    store.set(f"cssm_step{step}_rank{rank}", "1")
    deadline = datetime.timedelta(seconds=float(timeout_s))
    keys = [f"cssm_step{step}_rank{r}" for r in range(world)]
    try:
        store.wait(keys, deadline)
    except Exception:
        missing = []
        for r, k in enumerate(keys):
            try:
                store.wait([k], datetime.timedelta(milliseconds=50))
            except Exception:
                missing.append(r)
        raise PeerTimeout(missing or list(range(world))) from None


def gather_outputs_checked(local: torch.Tensor, n_total: int, store, step: int,
                           timeout_s: float = 30.0):
    """gather_outputs behind a roll call.  Returns (outputs, None) when every rank reported, else
    (this rank's own shard, PeerTimeout): the caller keeps its local results and decides."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local, None
    try:
        check_peers(store, dist.get_rank(), dist.get_world_size(), step, timeout_s)
    except PeerTimeout as e:
        return local, e
    return gather_outputs(local, n_total), None
