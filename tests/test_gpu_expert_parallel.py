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

import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from retrograd_b200.ep_check import SPEC


def _rank_main(rank: int, world: int, workdir: Path) -> None:
    import retrograd_b200 as rb
    from retrograd_b200.ep_check import plain_vs_expert_parallel

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
    result = plain_vs_expert_parallel(rb, rank, world, id_path.read_bytes(), workdir)
    engine = result["engine"]
    assert result["bit_exact"], "expert-parallel results differ from the plain engine's"
    assert result["footprint_split"], "the rank still holds other ranks' expert banks"
    # A plan refused on one rank: rank 1 submits a row in a slot the context does not have. It gets its own -3,
    # rank 0 (whose plan is fine) gets a runtime error instead of waiting for a partner that never comes, nothing
    # of rank 0's step becomes resident, and the next common step runs as usual.
    greedy = rb.SamplingParamsV2.greedy()
    out = rb.StepOutput()
    before = engine.seq_pos(3)
    try:
        engine.step([rb.StepRow(90, 99 if rank == 1 else 3, [5, 6, 7], 0, sample=True, sampling=greedy)], out)
        raise SystemExit("the refused step was not reported")
    except rb.InvalidArgument as err:
        assert rank == 1 and "slot is outside" in str(err)
    except rb.EngineError as err:
        assert rank == 0 and "another rank of the expert-parallel group refused its step" in str(err)
    assert engine.seq_pos(3) == before == (-1, -1)
    engine.step([rb.StepRow(91, 3, [5, 6, 7], 0, sample=True, sampling=greedy)], out)
    assert engine.seq_pos(3) == (0, 2)
    engine.close()
    print(f"rank {rank}: {result['steps']} steps equal to the plain engine")


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
