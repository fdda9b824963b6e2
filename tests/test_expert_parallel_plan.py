"""Expert-parallel exchange plan on CPU: the host arithmetic every rank runs on the all-gathered pair
offsets, and a world_size-2 gloo run of the whole dispatch -> expert work -> combine round trip with
that plan (CPU tensors stand in for the device buffers; the expert's work is a per-expert affine map,
so a row that reached the wrong expert or came back to the wrong pair shows)."""
import os
import socket

import numpy as np
import pytest


def _offsets(pair_expert, n_expert):
    counts = np.bincount(pair_expert, minlength=n_expert)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


@pytest.mark.parametrize("world,n_expert,seed", [(1, 8, 0), (2, 8, 1), (4, 32, 2), (8, 32, 3), (2, 2, 4)])
def test_plans_of_all_ranks_agree_and_cover_every_pair(rb, world, n_expert, seed):
    rng = np.random.default_rng(seed)
    per = n_expert // world
    pair_expert = [rng.integers(0, n_expert, rng.integers(0, 60)) for _ in range(world)]
    if seed == 3:
        pair_expert[2] = np.zeros(0, dtype=np.int64)          # an idle rank
    all_off = np.stack([_offsets(p, n_expert) for p in pair_expert])
    plans = [rb.ep_plan(all_off, r) for r in range(world)]
    for r, plan in enumerate(plans):
        # what r sends to p is what p expects from r
        for p in range(world):
            assert plan["send_count"][p] == plans[p]["recv_count"][r]
            assert plan["send_begin"][p] == all_off[r][p * per]
        assert plan["send_count"].sum() == len(pair_expert[r])
        # the receive buffer is the peers' blocks back to back; the grouping covers it exactly once
        assert list(plan["recv_begin"]) == list(np.concatenate([[0], np.cumsum(plan["recv_count"])[:-1]]))
        n_recv = int(plan["recv_count"].sum())
        assert sorted(plan["sorted"].tolist()) == list(range(n_recv))
        assert plan["offsets"][0] == 0 and plan["offsets"][-1] == n_recv
        # rows grouped under expert e really are pairs of expert e: rebuild the receive buffer's expert ids
        recv_expert = np.concatenate([np.sort(pair_expert[p])[(np.sort(pair_expert[p]) // per) == r] for p in range(world)] or [np.zeros(0)])
        for e in range(n_expert):
            rows = plan["sorted"][plan["offsets"][e]: plan["offsets"][e + 1]]
            if e // per != r:
                assert len(rows) == 0
            else:
                assert (recv_expert[rows] == e).all()
                assert len(rows) == sum(int((p == e).sum()) for p in pair_expert)


def test_plan_rejects_an_expert_count_the_world_does_not_divide(rb):
    with pytest.raises(rb.InvalidArgument):
        rb.ep_plan(np.zeros((3, 9), dtype=np.int32), 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _exchange(dist, torch, send, send_begin, send_count, recv, recv_begin, recv_count, rank, world):
    """Rows [begin, begin + count) of `send` to each peer, the peers' rows into `recv`: the CPU twin of the engine's grouped send / recv."""
    ops = []
    for p in range(world):
        if p == rank:
            recv[recv_begin[p]: recv_begin[p] + recv_count[p]] = send[send_begin[p]: send_begin[p] + send_count[p]]
            continue
        if send_count[p]:
            ops.append(dist.P2POp(dist.isend, send[send_begin[p]: send_begin[p] + send_count[p]].contiguous(), p))
        if recv_count[p]:
            ops.append(dist.P2POp(dist.irecv, recv[recv_begin[p]: recv_begin[p] + recv_count[p]], p))
    for work in (dist.batch_isend_irecv(ops) if ops else []):
        work.wait()


def _worker(rank, world, port, out):
    import torch
    import torch.distributed as dist

    import retrograd_b200 as rb

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_expert, k, d = 8, 2, 5
    rng = np.random.default_rng(100 + rank)
    n_tokens = 7 + 4 * rank
    x = torch.from_numpy(rng.normal(size=(n_tokens, d)).astype(np.float32))
    pair_expert = np.stack([rng.permutation(n_expert)[:k] for _ in range(n_tokens)]).reshape(-1)     # pair = token * k + slot
    order = np.argsort(pair_expert, kind="stable").astype(np.int32)                                     # pairs grouped by expert
    mine = torch.from_numpy(_offsets(pair_expert, n_expert))
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    plan = rb.ep_plan(torch.stack(gathered).numpy(), rank)
    n_recv = int(plan["recv_count"].sum())
    send = x[torch.from_numpy(order // k)]
    recv = torch.zeros(n_recv, d)
    _exchange(dist, torch, send, plan["send_begin"], plan["send_count"], recv, plan["recv_begin"], plan["recv_count"], rank, world)
    # the expert's work: y = (e + 1) * x + e, applied group by group as the grouped GEMM does
    y = torch.zeros_like(recv)
    for e in range(n_expert):
        rows = torch.from_numpy(plan["sorted"][plan["offsets"][e]: plan["offsets"][e + 1]].astype(np.int64))
        y[rows] = (e + 1) * recv[rows] + e
    back = torch.zeros(len(order), d)
    _exchange(dist, torch, y, plan["recv_begin"], plan["recv_count"], back, plan["send_begin"], plan["send_count"], rank, world)
    pair_y = torch.zeros(len(order), d)
    pair_y[torch.from_numpy(order.astype(np.int64))] = back
    want = torch.stack([(e + 1) * x[i // k] + e for i, e in enumerate(pair_expert)])
    out.put((rank, bool(torch.equal(pair_y, want)), n_recv))
    dist.barrier()
    dist.destroy_process_group()


def test_two_cpu_ranks_round_trip_their_pairs_through_the_owning_experts():
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
    assert [r[1] for r in results] == [True, True]
    assert results[0][2] + results[1][2] == (7 + 11) * 2          # every pair was served by exactly one rank
