"""The prefill attention tile kernel on tcgen05 (TMA-staged K/V, scores and outputs in tensor memory) against the
mma.sync tile kernel it replaces (RB200_ATTN_TC5=0) and against the CPU oracle: ragged chunk lengths, chunks that
continue a resident sequence, contexts of many 64-key tiles, tiles whose last block is partly filled, GQA groups
of 1, 4 and 8, head widths 64 and 128."""
import numpy as np
import pytest

from helpers import ParityReport, check_step, expect_greedy

pytestmark = pytest.mark.gpu

SHAPES = {
    "hd128_g4": dict(arch="llama", layers=2, d=512, heads=4, kv_heads=1, head_dim=128, ff=1024, vocab=1024, dtype="q8_0", seed=61),
    "hd64_g8": dict(arch="qwen2", layers=2, d=512, heads=8, kv_heads=1, head_dim=64, ff=1024, vocab=1024, dtype="q8_0", seed=62),
    "hd64_g1": dict(arch="llama", layers=2, d=256, heads=4, kv_heads=4, head_dim=64, ff=512, vocab=1024, dtype="q8_0", seed=63),
}


def _steps(rb, rng):
    """Three steps: long ragged chunks from position 0; chunks continuing those sequences next to a fresh one and
    decode rows; then another round. Returns a list of row lists (request = slot)."""
    greedy = rb.SamplingParamsV2.greedy()
    lens = [333, 64, 129, 700, 17, 40]
    toks = [rng.integers(3, 1024, n + 400).tolist() for n in lens]
    first = [rb.StepRow(i, i, toks[i][:n], 0, sample=True, sampling=greedy) for i, n in enumerate(lens)]
    second = [rb.StepRow(i, i, toks[i][n:n + m], n, sample=True, sampling=greedy) for i, (n, m) in enumerate(zip(lens, [200, 65, 1, 31, 300, 1]))]
    second.append(rb.StepRow(6, 6, rng.integers(3, 1024, 257).tolist(), 0, sample=True, sampling=greedy))
    third = [rb.StepRow(i, i, toks[i][n + m:n + m + 33], n + m, sample=True, sampling=greedy) for i, (n, m) in enumerate(zip(lens, [200, 65, 1, 31, 300, 1]))]
    return [first, second, third]


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_tcgen05_prefill_attention_against_the_oracle_and_the_mma_sync_kernel(rb, oracle, models, monkeypatch, shape):
    path = models("attn_" + shape, **SHAPES[shape])
    cfg = rb.EngineConfig(n_ctx=16384, n_seq_max=8, n_batch=2048, n_ubatch=2048)
    results = {}
    for form in ("tcgen05", "mma_sync"):
        if form == "mma_sync":
            monkeypatch.setenv("RB200_ATTN_TC5", "0")
        else:
            monkeypatch.delenv("RB200_ATTN_TC5", raising=False)
        engine = rb.Engine(str(path), cfg)
        octx = oracle.Context(oracle.Model(str(path)), 8, 2048) if form == "tcgen05" else None
        out, rep = rb.StepOutput(2048, 0), ParityReport()
        rng = np.random.default_rng(9)
        trace = []
        for rows in _steps(rb, rng):
            if octx is not None:
                toks = check_step(rb, engine, octx, oracle, rows, out, rep)
                expect_greedy(oracle, toks, rep)
            else:
                engine.step(rows, out)
            trace.append(np.stack([engine.last_logits(i) for i in range(len(rows))]))
        if octx is not None:
            print(f"tcgen05 prefill attention {shape}: max|dlogit| vs oracle {rep.max_logit_diff:.3e}, tie events {rep.tie_events}")
        results[form] = trace
        engine.close()
    diff = max(float(np.abs(a - b).max()) for a, b in zip(results["tcgen05"], results["mma_sync"]))
    print(f"tcgen05 vs mma.sync prefill attention {shape}: max|dlogit| {diff:.3e}")
    assert diff < 2e-4
