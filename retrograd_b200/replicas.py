"""Multi-GPU layout of the decode step: independent engine replicas, one process per GPU.

The path shards by request: sequences are independent, the only cross-request state (the prefix
cache) is per engine. So there is no data-path collective. What the ranks share is (a) the rule
that sends a request to a replica and (b) the reduction of their timing at the end of a run.

The routing rule keeps requests that can share KV on one replica: the replica is chosen by a hash
of the first `min_prefix_len` prompt tokens (the reference's scheduler only reuses prefixes of at
least `min_prefix_len` tokens, crates/retrograd-infer/src/scheduler.rs:103-104,128), so a GRPO
group, an identical prompt or a conversation sharing its system prompt lands where its prefix is
resident.
"""
from __future__ import annotations

from typing import Sequence


def route(prompt_tokens: Sequence[int], n_replicas: int, min_prefix_len: int = 8) -> int:
    """Replica index of a request: FNV-1a over its first `min_prefix_len` token ids."""
    h = 0xCBF29CE484222325
    for t in list(prompt_tokens)[:min_prefix_len]:
        for shift in (0, 8, 16, 24):
            h ^= (int(t) >> shift) & 0xFF
            h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h % max(n_replicas, 1)


def aggregate(times_ms: Sequence[float], counts: Sequence[float], dist=None, device=None):
    """Whole-job figures from one rank's: MAX over ranks of every time, SUM of every count.

    `dist` is torch.distributed (initialised) or None for a single process. Returns (times, counts)
    as lists of floats, identical on every rank.
    """
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [float(x) for x in times_ms], [float(x) for x in counts]
    import torch

    t = torch.tensor(list(times_ms), dtype=torch.float64, device=device)
    c = torch.tensor(list(counts), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(c, op=dist.ReduceOp.SUM)
    return t.tolist(), c.tolist()


def all_ranks_ready(ready: bool, dist=None) -> bool:
    """The rule every expert-parallel step opens with, for a caller that wants the answer on the host before it
    submits anything: each rank says whether it has a valid step to run, and the step runs only if all of them
    do. (The engine applies the same rule inside `retro_engine_step*` over its own communicator: a rank whose
    plan is refused still joins the exchange, its peers skip the step with a runtime error, nobody waits for a
    partner that never comes.) `dist` is torch.distributed, initialised, or None for one process."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return bool(ready)
    flags = [None] * dist.get_world_size()
    dist.all_gather_object(flags, bool(ready))
    return all(flags)
