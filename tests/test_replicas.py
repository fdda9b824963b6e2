"""The N > 1 layout on CPU ranks (gloo, world_size 2): routing rule and whole-job reduction."""
import os
import socket

import numpy as np


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch.distributed as dist

    from retrograd_b200.replicas import aggregate, route

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)                      # the same request stream on every rank
    prompts = [rng.integers(3, 1000, 20).tolist() for _ in range(64)]
    mine = [i for i, p in enumerate(prompts) if route(p, world) == rank]
    # every rank times its own steps; the job's time is the slowest rank's, its tokens the sum
    times, counts = aggregate([10.0 + rank, 5.0 - rank], [len(mine), 100.0 * (rank + 1)], dist)
    out.put((rank, mine, times, counts))
    dist.barrier()
    dist.destroy_process_group()


def test_two_cpu_ranks_partition_requests_and_reduce_timing():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, mine0, t0, c0), (r1, mine1, t1, c1) = results
    assert sorted(mine0 + mine1) == list(range(64)) and not set(mine0) & set(mine1)
    assert len(mine0) > 8 and len(mine1) > 8
    assert t0 == t1 == [11.0, 5.0]                       # MAX over ranks
    assert c0 == c1 == [64.0, 300.0]                     # SUM over ranks


def test_routing_keeps_shared_prefixes_together():
    from retrograd_b200.replicas import route

    rng = np.random.default_rng(1)
    prefix = rng.integers(3, 1000, 8).tolist()
    group = [prefix + rng.integers(3, 1000, int(rng.integers(1, 50))).tolist() for _ in range(16)]
    assert len({route(p, 8) for p in group}) == 1
    spread = {route(rng.integers(3, 1000, 12).tolist(), 8) for _ in range(200)}
    assert spread == set(range(8))
    assert route([], 4) == route([], 4)


def _agreement_worker(rank, world, port, out):
    import torch.distributed as dist

    from retrograd_b200.replicas import all_ranks_ready

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ran = []
    for step in range(4):
        # rank 1's plan for step 2 is refused on the host (an invalid row): it still joins the exchange
        local_ok = not (rank == 1 and step == 2)
        if all_ranks_ready(local_ok, dist):
            ran.append(step)
    out.put((rank, ran))
    dist.barrier()
    dist.destroy_process_group()


def test_a_refused_step_on_one_rank_is_skipped_by_all_ranks():
    """Expert-parallel ranks step in lock-step: a refusal on one rank must make every rank skip that step, and
    the steps after it stay aligned."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_agreement_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == {0: [0, 1, 3], 1: [0, 1, 3]}
