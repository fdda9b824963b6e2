"""The bounds-checked build of the library (libretro_b200_checked.so): the same sources compiled with
-DRETRO_B200_CHECKED, in which every index a kernel reads from device memory is compared with its range before
use. The tiny CPU-runnable workload must run through it against the oracle without a single violation, and a
bad token id or block id planted AFTER the host's validation must be caught on the device, skipped and reported.

The library is chosen when the package loads, so the checks run in a child process; this file is its program."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _child() -> None:
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import numpy as np

    import retrograd_b200 as rb
    from conftest import C1_SPEC
    from helpers import ParityReport, check_step, expect_greedy
    from oracle import oracle as O

    lib = rb.load_library()
    assert lib.retro_b200_checked_build() == 1 and rb.LIB_PATH.name == "libretro_b200_checked.so"
    model = Path(sys.argv[2]) / "c1.gguf"
    rb.synth_gguf(model, **C1_SPEC)
    engine = rb.Engine(str(model), rb.EngineConfig(n_ctx=4096, n_seq_max=8, n_batch=1024, n_ubatch=1024))
    octx = O.Context(O.Model(str(model)), 8, 4096)
    out, rep, greedy = rb.StepOutput(), ParityReport(), rb.SamplingParamsV2.greedy()
    rng = np.random.default_rng(7)
    prefix = rng.integers(3, 4096, 32).tolist()
    prompts = [prefix + rng.integers(3, 4096, int(rng.integers(16, 129))).tolist() for _ in range(6)]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=greedy) for i, p in enumerate(prompts)]
    word = (lib.retro_b200_engine_check_word.argtypes[1]._type_ * 4)()
    for step in range(6):
        toks = check_step(rb, engine, octx, O, rows, out, rep)
        expect_greedy(O, toks, rep)
        assert lib.retro_b200_engine_check_word(engine._h, word) == 0 and list(word) == [0, 0, 0, 0]
        rows = [rb.StepRow.decode(i, i, out.row(i).token, len(prompts[i]) + step, greedy) for i in range(6)]
    engine.seq_cp(0, 6, 0, 40)           # a shared prefix with a copy-on-write boundary block, then more steps
    engine.step([rb.StepRow(6, 6, [7, 8, 9], 40, sample=True, sampling=greedy)], out)
    # planted after validation: a token id past the vocabulary ...
    os.environ["RB200_CHECK_INJECT"] = "token"
    try:
        engine.step([rb.StepRow(20, 7, [5, 6, 7], 0, sample=True, sampling=greedy)], out)
        raise SystemExit("the planted token id was not caught")
    except rb.EngineError as err:
        assert "bounds-checked build: a token id read on the device was 4103, outside [0, 4096)" in str(err), str(err)
    assert lib.retro_b200_engine_check_word(engine._h, word) == 0 and list(word)[:3] == [1, 4103, 4096] and word[3] >= 1
    # ... and a physical block id past the pool in the step's block-table patch
    engine.seq_rm(7)
    engine.seq_rm(5)
    os.environ["RB200_CHECK_INJECT"] = "block"
    try:
        engine.step([rb.StepRow(21, 5, [5, 6, 7], 0, sample=True, sampling=greedy)], out)
        raise SystemExit("the planted block id was not caught")
    except rb.EngineError as err:
        assert "a physical block id read on the device was" in str(err), str(err)
    del os.environ["RB200_CHECK_INJECT"]
    # the context is still usable: the other sequences continue and still follow the oracle
    engine.seq_rm(5)
    octx.seq_rm(5, -1, -1)
    rows = rows[:5]                      # the decode rows the loop above composed last and has not run yet
    toks = check_step(rb, engine, octx, O, rows, out, rep)
    expect_greedy(O, toks, rep)
    assert lib.retro_b200_engine_check_word(engine._h, word) == 0 and list(word) == [0, 0, 0, 0]
    engine.close()
    print(f"checked build: {rep.steps} steps clean, max|dlogit|={rep.max_logit_diff:.2e}, both planted indices caught")


@pytest.mark.gpu
def test_checked_build_runs_clean_and_catches_planted_indices(tmp_path):
    sys.path.insert(0, str(ROOT))
    from retrograd_b200 import build as B

    if not (ROOT / "retrograd_b200" / "libretro_b200_checked.so").exists():
        B.build(checked=True)
    env = dict(os.environ, RB200_CHECKED="1")
    env.pop("RB200_CHECK_INJECT", None)
    proc = subprocess.run([sys.executable, __file__, "child", str(tmp_path)], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    assert "both planted indices caught" in proc.stdout


def test_normal_build_reports_that_it_is_unchecked(rb):
    assert rb.load_library().retro_b200_checked_build() == 0


if __name__ == "__main__" and len(sys.argv) > 1 and sys.argv[1] == "child":
    _child()
