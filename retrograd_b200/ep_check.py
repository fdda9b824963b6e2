"""Expert parallelism against a plain engine on the same rows: the check behind the two-GPU test and the
benchmark's `ep_parity` record.

Every rank runs its own requests twice - through a plain engine, then through an engine that joined an
expert-parallel group of `world` ranks and serves n_expert / world experts. Per-pair arithmetic does not
depend on where a (token, expert) pair is computed, so logits, tokens and logprobs must be equal bit for
bit. The last step has the last rank idle: it only serves its experts to the others.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

SPEC = dict(arch="olmoe", layers=2, d=128, heads=4, kv_heads=4, ff=64, vocab=512, experts=8, experts_used=2,
            dtype="q8_0", expert_dtype="mxfp4", seed=21)


def _run(rb, engine, rank: int, idle_last: bool, expert_parallel: bool):
    greedy = rb.SamplingParamsV2.greedy()
    rng = np.random.default_rng(50 + rank)
    prompts = [rng.integers(3, 512, 7 + 5 * i + 2 * rank).tolist() for i in range(2 + rank % 2)]
    out = rb.StepOutput()
    n = len(prompts)

    def snapshot():
        return [out.row(i).token for i in range(n)], [out.row(i).logprob for i in range(n)], [engine.last_logits(i).copy() for i in range(n)]

    engine.step([rb.StepRow(i, i, p, 0, sample=True, sampling=greedy, want_logprob=True) for i, p in enumerate(prompts)], out)
    trace = [snapshot()]
    for step in range(3):
        if idle_last and step == 2:
            if expert_parallel:
                engine.ep_idle_step()
            continue
        last = trace[-1][0]
        engine.step([rb.StepRow(i, i, [last[i]], len(p) + step, sample=True, sampling=greedy, want_logprob=True) for i, p in enumerate(prompts)], out)
        trace.append(snapshot())
    return trace


def plain_vs_expert_parallel(rb, rank: int, world: int, unique_id: bytes, workdir: Path) -> dict:
    """Runs both passes on this rank (collective over the `world` ranks that share `unique_id`); returns
    {"steps": compared steps, "bit_exact": bool, "footprint_split": bool} and leaves the expert-parallel engine closed."""
    model = Path(workdir) / f"ep_check_rank{rank}.gguf"
    rb.synth_gguf(model, **SPEC)
    cfg = rb.EngineConfig(n_ctx=512, n_seq_max=4, n_batch=64, n_ubatch=64)
    idle_last = rank == world - 1
    plain = rb.Engine(str(model), cfg)
    want = _run(rb, plain, rank, idle_last, expert_parallel=False)
    plain.close()
    engine = rb.Engine(str(model), cfg)
    banks = sum(b["n_bytes"] for b in engine.expert_banks())
    before = engine.memory_report()["model_weight_bytes"]
    engine.ep_init(rank, world, unique_id)
    # the rank now holds its own experts only: (world - 1) / world of the banks' bytes are gone (the banks are held
    # in the format's own bytes or re-coded at up to twice that, hence the bounds)
    freed = before - engine.memory_report()["model_weight_bytes"]
    footprint_split = world == 1 or banks * (world - 1) / world * 0.95 <= freed <= 2.1 * banks
    got = _run(rb, engine, rank, idle_last, expert_parallel=True)
    equal = len(got) == len(want)
    for (t0, l0, x0), (t1, l1, x1) in zip(want, got):
        equal = equal and t0 == t1 and l0 == l1 and all(np.array_equal(a, b) for a, b in zip(x0, x1))
    return {"steps": len(got), "bit_exact": bool(equal), "footprint_split": bool(footprint_split), "engine": engine}
