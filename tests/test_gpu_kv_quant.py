"""Quantised KV pools (engine kv_dtype Q8_0 / Q4_0, `crates/retrograd-ffi/runtime/src/retro_engine.cpp:84-90,251-266`):
the CUDA engine against the oracle whose cache returns ggml's quantise-then-dequantise of every stored row.

A quantiser is a step function: a K or V value that differs between the two sides by one f32 rounding can land on the
other side of a rounding boundary and come back one quantum apart (amax / 127 for Q8_0, amax / 8 for Q4_0). With the
few hundred thousand values of these cases that happens about once for Q8_0 and is invisible (a quantum is 0.8 % of
the block's largest value); for Q4_0 a single such event moves a logit by a few 1e-3, so its tolerance is wider.
"""
from __future__ import annotations

import numpy as np
import pytest

from helpers import ParityReport, check_step, expect_greedy
import helpers

pytestmark = pytest.mark.gpu

SPECS = {
    # head_dim 64, GQA 2: tiles of 64 tokens
    "hd64": dict(arch="llama", layers=3, d=256, heads=4, kv_heads=2, ff=512, vocab=1024, dtype="q8_0", seed=77),
    # head_dim 128, GQA 4: the 8B model's attention shape (tiles of 32 tokens)
    "hd128": dict(arch="llama", layers=2, d=512, heads=4, kv_heads=1, ff=1024, vocab=1024, dtype="q8_0", seed=78),
}
KV = {"q8_0": 2, "q4_0": 3}        # retro_engine_kv_dtype
TOL = {"q8_0": helpers.LOGIT_TOL, "q4_0": 5e-2}


def _prompt(seed, n, vocab=1024):
    return np.random.default_rng(seed).integers(3, vocab, n).tolist()


@pytest.mark.parametrize("shape", list(SPECS))
@pytest.mark.parametrize("dtype,native", [("q8_0", True), ("q8_0", False), ("q4_0", True), ("q4_0", False)])
def test_quantised_kv_pool_matches_the_oracle(rb, oracle, models, monkeypatch, shape, dtype, native):
    """Prefill chunks (tensor-core tiles), short rows, decode rows (split over several CTAs: the longest context is
    400 tokens), a shared prefix with its copy-on-write block and a second chunk over a resident context: every kernel
    that reads K / V, over a pool that holds quantised rows. Decode rows are read from the pool by their own kernel
    (`native`), or - like every other row - from the dequantised scratch."""
    path = models(f"kvq_{shape}", **SPECS[shape])
    monkeypatch.setattr(helpers, "LOGIT_TOL", TOL[dtype])
    monkeypatch.setenv("RB200_KV_Q8_NATIVE", "1" if native else "0")
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=2048, n_seq_max=5, n_batch=512, n_ubatch=512, kv_dtype=KV[dtype]))
    om = oracle.Model(str(path))
    octx = oracle.Context(om, 5, 2048, kv_dtype=KV[dtype])
    out = rb.StepOutput()
    rep = ParityReport()
    g = rb.SamplingParamsV2.greedy()
    prompts = [_prompt(500, 400), _prompt(501, 70), _prompt(502, 5)]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=g) for i, p in enumerate(prompts)]
    toks = check_step(rb, engine, octx, oracle, rows, out, rep)
    last = [toks[r][0].token for r in range(3)]
    length = [len(p) for p in prompts]
    for _ in range(3):                                   # decode rows
        rows = [rb.StepRow(i, i, [last[i]], length[i], sample=True, sampling=g) for i in range(3)]
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        last = [toks[r][0].token for r in range(3)]
        length = [n + 1 for n in length]
    # slot 3 shares slot 0's first 100 positions, then both go on: the boundary block is copied on write
    engine.seq_cp(0, 3, 0, 100)
    octx.seq_cp(0, 3, 0, 100)
    assert engine.seq_pos(3) == (0, 99)
    rows = [rb.StepRow(0, 0, [last[0]], length[0], sample=True, sampling=g),
            rb.StepRow(9, 3, _prompt(503, 90), 100, sample=True, sampling=g),       # a chunk over a resident, quantised context
            rb.StepRow(1, 1, [last[1]], length[1], sample=True, sampling=g)]
    toks = check_step(rb, engine, octx, oracle, rows, out, rep)
    rows = [rb.StepRow(9, 3, [toks[1][0].token], 190, sample=True, sampling=g),
            rb.StepRow(0, 0, [toks[0][0].token], length[0] + 1, sample=True, sampling=g)]
    toks = check_step(rb, engine, octx, oracle, rows, out, rep)
    print(f"kv {dtype} {shape} native={native}: max|dlogit|={rep.max_logit_diff:.3e} min margin={rep.min_margin:.3e} rows={rep.sampled}")
    engine.close()


def test_quantised_pool_is_smaller_and_its_snapshots_round_trip(rb, models):
    path = models("kvq_hd64", **SPECS["hd64"])
    g = rb.SamplingParamsV2.greedy()
    out = rb.StepOutput()
    sizes = {}
    for name, code in (("f16", 1), ("q8_0", 2), ("q4_0", 3)):
        engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=4096, n_seq_max=4, n_batch=256, n_ubatch=256, kv_dtype=code))
        sizes[name] = engine.memory().kv_bytes
        prompt = _prompt(600, 45)
        engine.step([rb.StepRow(0, 0, prompt, 0, sample=True, sampling=g)], out)
        tok = out.row(0).token
        snap = engine.seq_save(0)
        engine.seq_load(2, snap)
        assert engine.seq_pos(2) == (0, 44)
        # the restored sequence continues exactly as the original: the pool's bytes travelled, not rounded values
        engine.step([rb.StepRow(0, 0, [tok], 45, sample=True, sampling=g), rb.StepRow(1, 2, [tok], 45, sample=True, sampling=g)], out)
        assert out.row(0).token == out.row(1).token
        assert np.array_equal(engine.last_logits(0), engine.last_logits(1))
        if name == "q8_0":
            q8_snapshot = snap
        if name == "f16":
            f16_engine_snapshot_len = len(snap)
        engine.close()
    # 3 layers x 2 x 128 values per position: 2 bytes each, 8.5 bits, 4.5 bits (the quantised pools keep one layer of f16 scratch)
    assert sizes["q8_0"] < 0.90 * sizes["f16"] and sizes["q4_0"] < sizes["q8_0"]
    assert len(q8_snapshot) < f16_engine_snapshot_len
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=4096, n_seq_max=4, n_batch=256, n_ubatch=256))
    with pytest.raises(rb.EngineError, match="refused"):
        engine.seq_load(0, q8_snapshot)
    engine.close()


def test_f32_pool_is_refused_with_a_message(rb, models):
    path = models("kvq_hd64", **SPECS["hd64"])
    with pytest.raises(rb.EngineError, match="F32 is not supported"):
        rb.Engine(str(path), rb.EngineConfig(n_ctx=256, n_seq_max=2, n_batch=64, n_ubatch=64, kv_dtype=0))
