"""Data-parallel replicas: the only multi-GPU form of the batch-1 decode path.

The 1B-shape decode path does not shard: a token step is one dependent chain over the whole
model.  With N GPUs, N processes (one per GPU) each run an independent replica on its own
sequences; there is no collective on the data path.  ``torch.distributed`` is used only to line
the ranks up around the timed region and to combine their timings:

    value = (tokens all ranks produced) / (time of the slowest rank)

The helpers work on any backend (``nccl`` on GPUs, ``gloo`` on CPU for the tests).
"""
from __future__ import annotations

import os
from typing import List, Sequence, Tuple


def dist_env() -> Tuple[int, int, int]:
    """(rank, local_rank, world_size) from the launcher's environment (1 process if unset)."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def shard_sequences(n_sequences: int, rank: int, world: int) -> range:
    """Contiguous, balanced share of ``n_sequences`` independent sequences for ``rank``:
    the first ``n % world`` ranks take one more.  Shares are disjoint and cover everything."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(max(0, n_sequences), world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def _reduce(value: float, op: str, device) -> float:
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "sum": dist.ReduceOp.SUM}[op])
    return float(t.item())


def combine_timings(ms: float, tokens: int, e2e_tok_s: float, world: int, device="cpu") -> dict:
    """Whole-job figures from one rank's device-timed ``ms`` for ``tokens`` tokens and its
    end-to-end tok/s.  Every rank must call this (it is a collective when ``world > 1``).

    ``value``  = all ranks' tokens / slowest rank's time;
    ``e2e``    = world * slowest rank's end-to-end rate (a lower bound of the aggregate)."""
    if world > 1:
        ms_max = _reduce(ms, "max", device)
        tok_sum = _reduce(tokens, "sum", device)
        e2e_min = _reduce(e2e_tok_s, "min", device)
    else:
        ms_max, tok_sum, e2e_min = ms, float(tokens), e2e_tok_s
    return {"ms": ms_max, "tokens": int(round(tok_sum)), "value": tok_sum / (ms_max * 1e-3), "e2e": e2e_min * world}


def gather_generated(local: Sequence[Sequence[int]], world: int) -> List[List[int]]:
    """All ranks' generated id lists in rank order (rank 0's sequences first).  A collective."""
    if world <= 1:
        return [list(x) for x in local]
    import torch.distributed as dist
    out: List[object] = [None] * world
    dist.all_gather_object(out, [list(map(int, x)) for x in local])
    return [seq for part in out for seq in part]        # type: ignore[union-attr]
