"""Expert parallelism on two GPUs: each rank runs its own requests through an engine that serves half
of the experts, exchanging (token, expert) pairs over NCCL in every MoE layer. Per-pair arithmetic does
not depend on where a pair is computed, so every rank's logits, tokens and logprobs must equal, bit
for bit, those of a plain engine given the same rows. The last step has rank 1 idle: it only serves.

The ranks are child processes (one GPU each) started by the test; this file is also their program."""
import os
import subprocess
import sys
import time
from pathlib import Path

import numpy as np
import pytest

SPEC = dict(arch="olmoe", layers=2, d=128, heads=4, kv_heads=4, ff=64, vocab=512, experts=8, experts_used=2,
            dtype="q8_0", expert_dtype="mxfp4", seed=21)


def _steps(rb, rank):
    """The rows of each lock-step step of `rank` (None: the rank has nothing to run in that step)."""
    greedy = rb.SamplingParamsV2.greedy()
    rng = np.random.default_rng(50 + rank)
    prompts = [rng.integers(3, 512, 7 + 5 * i + 2 * rank).tolist() for i in range(2 + rank)]
    return prompts, greedy


def _run(rb, engine, rank, idle_last, ep):
    prompts, greedy = _steps(rb, rank)
    out = rb.StepOutput()
    trace = []
    engine.step([rb.StepRow(i, i, p, 0, sample=True, sampling=greedy, want_logprob=True) for i, p in enumerate(prompts)], out)
    last = [out.row(i).token for i in range(len(prompts))]
    trace.append((list(last), [out.row(i).logprob for i in range(len(prompts))], [engine.last_logits(i).copy() for i in range(len(prompts))]))
    for step in range(3):
        if idle_last and step == 2:
            if ep:
                engine.ep_idle_step()
            continue
        rows = [rb.StepRow(i, i, [last[i]], len(p) + step, sample=True, sampling=greedy, want_logprob=True) for i, p in enumerate(prompts)]
        engine.step(rows, out)
        last = [out.row(i).token for i in range(len(prompts))]
        trace.append((list(last), [out.row(i).logprob for i in range(len(prompts))], [engine.last_logits(i).copy() for i in range(len(prompts))]))
    return trace


def _rank_main(rank: int, world: int, workdir: Path) -> None:
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import retrograd_b200 as rb

    model = workdir / f"moe_rank{rank}.gguf"
    rb.synth_gguf(model, **SPEC)
    cfg = rb.EngineConfig(n_ctx=512, n_seq_max=4, n_batch=64, n_ubatch=64)
    plain = rb.Engine(str(model), cfg)
    want = _run(rb, plain, rank, idle_last=(rank == 1), ep=False)
    plain.close()

    id_path = workdir / "nccl_id.bin"
    if rank == 0:
        tmp = workdir / "nccl_id.tmp"
        tmp.write_bytes(rb.nccl_unique_id())
        tmp.rename(id_path)
    deadline = time.time() + 120
    while not id_path.exists():
        if time.time() > deadline:
            raise SystemExit("no NCCL id from rank 0")
        time.sleep(0.05)
    engine = rb.Engine(str(model), cfg)
    engine.ep_init(rank, world, id_path.read_bytes())
    got = _run(rb, engine, rank, idle_last=(rank == 1), ep=True)
    engine.close()
    assert len(got) == len(want)
    for (t0, l0, x0), (t1, l1, x1) in zip(want, got):
        assert t0 == t1 and l0 == l1
        for a, b in zip(x0, x1):
            assert np.array_equal(a, b)
    print(f"rank {rank}: {len(got)} steps equal to the plain engine")


@pytest.mark.gpu
@pytest.mark.parametrize("experts", ["tensor_cores", "rows"])
def test_two_ranks_with_half_the_experts_each_equal_the_plain_engine(tmp_path, experts):
    """Both forms of the expert FFN: banks re-coded for the grouped tensor-core GEMM, and (RB200_MOE=rows)
    the MXFP4 bytes on the CUDA-core grouped kernel."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    procs = []
    for rank in range(2):
        env = dict(os.environ, CUDA_VISIBLE_DEVICES=str(rank), NCCL_NVLS_ENABLE="0")
        if experts == "rows":
            env["RB200_MOE"] = "rows"
        else:
            env.pop("RB200_MOE", None)
        procs.append(subprocess.Popen([sys.executable, __file__, str(rank), "2", str(tmp_path)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outputs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=300)
            outputs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for rank, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out[-3000:]}"
        assert "steps equal to the plain engine" in out


@pytest.mark.gpu
def test_expert_parallel_init_is_refused_for_dense_models_and_bad_worlds(rb, c1_model, models):
    engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=256, n_seq_max=2, n_batch=32, n_ubatch=32))
    with pytest.raises(rb.InvalidArgument):
        engine.ep_init(0, 2, bytes(128))
    with pytest.raises(rb.InvalidArgument):
        engine.ep_idle_step()
    engine.close()
    moe = rb.Engine(str(models("moe_flat", **SPEC)), rb.EngineConfig(n_ctx=256, n_seq_max=2, n_batch=32, n_ubatch=32))
    with pytest.raises(rb.InvalidArgument):
        moe.ep_init(0, 3, bytes(128))            # 8 experts over 3 ranks
    with pytest.raises(rb.InvalidArgument):
        moe.ep_init(2, 2, bytes(128))            # rank outside the world
    moe.close()


if __name__ == "__main__":
    _rank_main(int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3]))
