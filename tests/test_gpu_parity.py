"""Parity of the CUDA decode step with the CPU oracle on the same seeded inputs, through the C ABI.

Bit-exact: packing maps, block-table resolution, greedy token streams. Logits: max abs <= 1e-2
in fp32 (helpers.LOGIT_TOL), measured and printed.
"""
import numpy as np
import pytest

from conftest import GOLDEN
from helpers import ParityReport, check_step, expect_greedy

pytestmark = pytest.mark.gpu


def _greedy_workload(rb, O, model_path, prompts, n_new, n_batch=256, n_ctx=4096, chunk=None, adapters=None):
    """Continuous-batching style plan: chunked prefill rows mixed with decode rows, greedy."""
    n = len(prompts)
    engine = rb.Engine(str(model_path), rb.EngineConfig(n_ctx=n_ctx, n_seq_max=max(n, 2), n_batch=n_batch, n_ubatch=n_batch))
    om = O.Model(str(model_path))
    octx = O.Context(om, max(n, 2), engine.context_size())
    out = rb.StepOutput()
    report = ParityReport()
    greedy = rb.SamplingParamsV2.greedy()
    pos = [0] * n          # next prompt position to prefill
    last = [None] * n      # last sampled token, to feed back
    done = [0] * n
    streams = [[] for _ in range(n)]
    chunk = chunk or n_batch
    while any(d < n_new for d in done):
        rows, kinds, budget = [], [], n_batch
        for i in range(n):          # decode rows first, as the scheduler composes them
            if last[i] is not None and done[i] < n_new and budget > 0:
                rows.append(rb.StepRow.decode(i, i, last[i], len(prompts[i]) + done[i] - 1, greedy))
                kinds.append("decode")
                budget -= 1
        for i in range(n):
            if last[i] is None and budget > 0:
                take = min(budget, chunk, len(prompts[i]) - pos[i])
                final = pos[i] + take == len(prompts[i])
                rows.append(rb.StepRow(i, i, prompts[i][pos[i] : pos[i] + take], pos[i], sample=final, sampling=greedy))
                kinds.append("prefill")
                budget -= take
        for r in rows:
            if adapters:
                r.adapter = adapters[r.slot]
        toks = check_step(rb, engine, octx, O, rows, out, report)
        expect_greedy(O, toks, report)
        for r, (row, kind) in enumerate(zip(rows, kinds)):
            i = row.slot
            if kind == "prefill":
                pos[i] += len(row.tokens)
            if row.sample:
                last[i] = out.row(r).token
                streams[i].append(last[i])
                done[i] += 1
    report.streams = streams
    engine.close()
    return report


def test_c1_tiny_llama_q8_0_greedy_streams(rb, oracle, c1_model):
    """The tiny CPU-runnable workload: 8 requests = shared 32-token prefix + 16..128 unique tokens, 32 greedy
    tokens each."""
    rng = np.random.default_rng(20261125)
    prefix = rng.integers(3, 4096, 32).tolist()
    prompts = [prefix + rng.integers(3, 4096, int(rng.integers(16, 129))).tolist() for _ in range(8)]
    rep = _greedy_workload(rb, oracle, c1_model, prompts, 32, n_batch=256, chunk=96)
    print(f"C1: steps={rep.steps} sampled={rep.sampled} max|dlogit|={rep.max_logit_diff:.3e} "
          f"min top-2 margin={rep.min_margin:.3e} tie events={rep.tie_events} max|dlogprob|={rep.max_logprob_diff:.2e}")
    assert rep.sampled == 8 * 32
    assert rep.tie_events == 0


@pytest.mark.parametrize(
    "name,spec",
    [
        ("q4k", dict(arch="llama", layers=2, d=512, heads=8, kv_heads=2, ff=1024, vocab=1024, dtype="q4_k", seed=11)),
        ("f16", dict(arch="llama", layers=2, d=256, heads=4, kv_heads=4, ff=512, vocab=512, dtype="f16", seed=12)),
        ("f32", dict(arch="qwen2", layers=2, d=128, heads=4, kv_heads=2, ff=256, vocab=300, dtype="f32", seed=13, bias=1)),
        ("mxfp4", dict(arch="llama", layers=2, d=256, heads=4, kv_heads=1, ff=512, vocab=512, dtype="mxfp4", seed=14)),
        ("hd128", dict(arch="llama", layers=1, d=512, heads=4, kv_heads=1, head_dim=128, ff=512, vocab=512, dtype="q8_0", seed=15)),
    ],
)
def test_storage_types_and_shapes(rb, oracle, models, name, spec):
    rng = np.random.default_rng(spec["seed"])
    prompts = [rng.integers(3, spec["vocab"], int(rng.integers(5, 60))).tolist() for _ in range(4)]
    rep = _greedy_workload(rb, oracle, models(name, **spec), prompts, 6, n_batch=64, chunk=23)
    print(f"{name}: max|dlogit|={rep.max_logit_diff:.3e} ties={rep.tie_events}")


@pytest.mark.parametrize("fixture", ["retrograd-tiny-qwen2-f32.gguf", "retrograd-tiny-qwen2-f16.gguf", "retrograd-tiny-qwen2-q8_0.gguf"])
def test_reference_tiny_qwen2_fixtures(rb, oracle, fixture):
    """The reference's own tiny models: qwen2 graph (q/k/v and output biases, half-split RoPE, GQA)."""
    rng = np.random.default_rng(5)
    prompts = [rng.integers(3, 260, int(rng.integers(4, 40))).tolist() for _ in range(3)]
    rep = _greedy_workload(rb, oracle, GOLDEN / fixture, prompts, 8, n_batch=32, n_ctx=512)
    print(f"{fixture}: max|dlogit|={rep.max_logit_diff:.3e} ties={rep.tie_events}")


def test_reference_tiny_olmoe_routing_is_bit_exact(rb, oracle):
    """Known answer (tests/expert_placement.rs:379-425): every token of the concentrated tiny
    OLMoE routes to experts {0, 1}; router ids equal the oracle's for every layer and token."""
    path = GOLDEN / "retrograd-tiny-olmoe-f32.gguf"
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=256, n_seq_max=2, n_batch=32, n_ubatch=32))
    engine.expert_route_enable(1)
    om = oracle.Model(str(path))
    octx = oracle.Context(om, 2, 256)
    out = rb.StepOutput()
    rep = ParityReport()
    greedy = rb.SamplingParamsV2.greedy()
    prompt = engine.tokenize_text("The quick brown fox")[:9]
    rows = [rb.StepRow(0, 0, prompt, 0, sample=True, sampling=greedy, n_top_logprobs=1)]
    n_tok = 0
    for step in range(4):
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        expect_greedy(oracle, toks, rep)
        n = len(rows[0].tokens)
        n_tok += n
        got = engine.last_routes().reshape(om.n_layer, n, om.n_expert_used)
        want = octx.last_routes().reshape(om.n_layer, n, om.n_expert_used)
        assert np.array_equal(got, want)
        assert np.array_equal(np.sort(got, axis=-1), np.broadcast_to([0, 1], got.shape))
        rows = [rb.StepRow.decode(0, 0, out.row(0).token, len(prompt) + step, greedy)]
    for layer in range(om.n_layer):
        assert list(engine.expert_route_counts(layer, 8)) == [n_tok, n_tok, 0, 0, 0, 0, 0, 0]
    engine.close()


def test_flat_router_moe_matches_oracle(rb, oracle, models):
    spec = dict(arch="olmoe", layers=2, d=128, heads=4, kv_heads=4, ff=64, vocab=512, experts=8, experts_used=2,
                dtype="q8_0", expert_dtype="mxfp4", seed=21)
    path = models("moe_flat", **spec)
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=512, n_seq_max=4, n_batch=64, n_ubatch=64))
    om = oracle.Model(str(path))
    octx = oracle.Context(om, 4, 512)
    out = rb.StepOutput()
    rep = ParityReport()
    rng = np.random.default_rng(3)
    greedy = rb.SamplingParamsV2.greedy()
    rows = [rb.StepRow(i, i, rng.integers(3, 512, 9 + 3 * i).tolist(), 0, sample=True, sampling=greedy) for i in range(3)]
    toks = check_step(rb, engine, octx, oracle, rows, out, rep)
    expect_greedy(oracle, toks, rep)
    T = sum(len(r.tokens) for r in rows)
    got = engine.last_routes().reshape(om.n_layer, T, 2)
    want = octx.last_routes().reshape(om.n_layer, T, 2)
    assert np.array_equal(got, want)
    assert len(np.unique(got)) > 2  # the flat router really spreads tokens
    print(f"moe flat: max|dlogit|={rep.max_logit_diff:.3e}")
    engine.close()


def test_tensor_core_gemm_path_wide_steps(rb, oracle, models):
    """Steps with hundreds of tokens take the tensor-core GEMM (f16 operands, f32 accumulate);
    the oracle stays f32 end to end, so this measures the path's real logit error."""
    spec = dict(arch="llama", layers=4, d=1024, heads=8, kv_heads=2, ff=2816, vocab=2048, dtype="q4_k", seed=31)
    rng = np.random.default_rng(31)
    prompts = [rng.integers(3, 2048, n).tolist() for n in (301, 77, 190, 12, 129)]
    rep = _greedy_workload(rb, oracle, models("q4k_wide", **spec), prompts, 4, n_batch=512, n_ctx=4096, chunk=256)
    print(f"q4k wide: max|dlogit|={rep.max_logit_diff:.3e} min margin={rep.min_margin:.3e} ties={rep.tie_events}")


def test_full_8b_shape_logits_within_tolerance(rb, oracle):
    """The headline workload's model at full size (32 layers, d 4096, Q4_K): a ragged prefill step on
    the tensor-core path and decode steps on the row path, logits against the f32 CPU oracle."""
    import bench

    path = bench.ensure_model("c2", 0)
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=4096, n_seq_max=4, n_batch=128, n_ubatch=128))
    om = oracle.Model(str(path), fast=True)
    octx = oracle.Context(om, 4, 4096)
    out = rb.StepOutput()
    rep = ParityReport()
    rng = np.random.default_rng(8)
    greedy = rb.SamplingParamsV2.greedy()
    prompts = [rng.integers(3, 128256, n).tolist() for n in (40, 9, 23)]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=greedy) for i, p in enumerate(prompts)]
    for step in range(3):
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        expect_greedy(oracle, toks, rep)
        rows = [rb.StepRow.decode(i, i, out.row(i).token, len(prompts[i]) + step, greedy) for i in range(3)]
    print(f"8B shape: max|dlogit|={rep.max_logit_diff:.3e} min margin={rep.min_margin:.3e} ties={rep.tie_events}")
    engine.close()


def test_moe_experts_on_the_tensor_cores_agree_with_the_row_kernel(rb, models, monkeypatch):
    """MXFP4 expert banks are decoded by the grouped tcgen05 GEMM straight from their 17-byte blocks (one launch
    per projection for all experts); RB200_MOE=rows keeps the CUDA-core row kernel on the same bytes. Same
    weights, two summation orders: routing equal, logits within 2e-4, greedy tokens equal."""
    spec = dict(arch="olmoe", layers=2, d=128, heads=4, kv_heads=4, ff=64, vocab=512, experts=8, experts_used=2,
                dtype="q8_0", expert_dtype="mxfp4", seed=21)
    path = models("moe_flat", **spec)
    rng = np.random.default_rng(9)
    prompts = [rng.integers(3, 512, 11 + 4 * i).tolist() for i in range(3)]
    greedy = rb.SamplingParamsV2.greedy()

    def run(rows_kernel: bool):
        if rows_kernel:
            monkeypatch.setenv("RB200_MOE", "rows")
        else:
            monkeypatch.delenv("RB200_MOE", raising=False)
        engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=512, n_seq_max=4, n_batch=64, n_ubatch=64))
        storage = engine.expert_storage(0)
        out = rb.StepOutput()
        engine.step([rb.StepRow(i, i, p, 0, sample=True, sampling=greedy) for i, p in enumerate(prompts)], out)
        toks = [out.row(i).token for i in range(3)]
        logits = np.stack([engine.last_logits(i) for i in range(3)])
        routes = engine.last_routes().copy()
        engine.step([rb.StepRow(i, i, [toks[i]], len(prompts[i]), sample=True, sampling=greedy) for i in range(3)], out)
        logits2 = np.stack([engine.last_logits(i) for i in range(3)])
        engine.close()
        return storage, toks, logits, logits2, routes

    s_tc, t_tc, l_tc, l2_tc, r_tc = run(False)
    s_rows, t_rows, l_rows, l2_rows, r_rows = run(True)
    assert s_tc == (39, 39, 39) and s_rows == (39, 39, 39)          # MXFP4 as stored, in both forms
    assert np.array_equal(r_tc, r_rows) and t_tc == t_rows
    err = max(float(np.abs(l_tc - l_rows).max()), float(np.abs(l2_tc - l2_rows).max()))
    print(f"moe tensor-core vs row kernel: max|dlogit|={err:.3e}")
    assert err < 2e-4


def test_tiny_workload_reproduces_the_committed_oracle_streams(rb):
    """The engine's greedy streams on the tiny CPU-runnable workload equal, token for token, the streams the CPU
    oracle wrote into tests/golden/c1_greedy_tokens.json (256 tokens; smallest oracle top-2 margin 1.4e-3)."""
    from retrograd_b200.golden_check import replay

    result = replay(rb)
    assert result["tokens"] == 256 and result["bit_exact"], result["first_mismatch"]


def test_tiny_workload_over_a_q8_0_kv_pool_reproduces_the_committed_oracle_streams(rb):
    """The same comparison with engine kv_dtype Q8_0 against the streams the oracle produced over a cache that returns
    ggml's quantise-then-dequantise of every stored row (256 tokens; smallest oracle top-2 margin 1.2e-3)."""
    from retrograd_b200.golden_check import replay

    result = replay(rb, kv="q8_0")
    assert result["tokens"] == 256 and result["bit_exact"], result["first_mismatch"]
