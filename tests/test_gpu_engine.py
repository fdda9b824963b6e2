"""Engine behaviour through the C ABI on the GPU: validation, sequence memory, sampling, adapters."""
import numpy as np
import pytest

from helpers import ParityReport, check_step, expect_greedy

pytestmark = pytest.mark.gpu


@pytest.fixture()
def pair(rb, oracle, c1_model):
    engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=1024, n_seq_max=8, n_batch=128, n_ubatch=128))
    om = oracle.Model(str(c1_model))
    octx = oracle.Context(om, 8, engine.context_size())
    yield engine, octx
    engine.close()


def _prompt(seed, n, vocab=4096):
    return np.random.default_rng(seed).integers(3, vocab, n).tolist()


def test_step_validation_messages(rb, pair):
    """Same checks, order and messages as the reference's step (retro_gen_core.cpp:2409-2516);
    nothing is decoded by a refused step."""
    engine, _ = pair
    out = rb.StepOutput()
    g = rb.SamplingParamsV2.greedy()
    cases = [
        ([rb.StepRow(0, 9, [5], 0)], "step row slot is outside the context's sequence range"),
        ([rb.StepRow(0, 0, [5], 1024)], "step row positions exceed the per-sequence context"),
        ([rb.StepRow(0, 0, [5, 6, 7], 0), rb.StepRow(1, 0, [8], 2)], "step rows overlap in the same sequence slot"),
        ([rb.StepRow(0, 0, [5], 0), rb.StepRow(1, 0, [8], 1, adapter=rb.ADAPTER_BASE)], "step rows of one sequence slot select different adapters"),
        ([rb.StepRow(0, 0, [4096], 0)], "token 4096 at index 0 is outside the vocabulary of size 4096"),
        ([rb.StepRow(0, 0, [5] * 129, 0)], "the step's tokens exceed the context's physical batch (n_batch)"),
        ([rb.StepRow(0, 0, [5], 0, adapter=77)], "step row adapter 77 is not a loaded per-row adapter"),
        ([rb.StepRow(0, 0, [5], 0, sample=True, sampling=rb.SamplingParamsV2(temperature=0.0))], "sampling temperature must be finite and greater than zero"),
        ([rb.StepRow(0, 0, [5], 0, sample=True, sampling=rb.SamplingParamsV2(top_p=0.0))], "sampling top_p must be in (0, 1]"),
        ([rb.StepRow(0, 0, [5], 0, sample=True, sampling=rb.SamplingParamsV2(min_p=2.0))], "sampling min_p must be in [0, 1]"),
        ([rb.StepRow(0, 0, [5], 0, sample=True, sampling=rb.SamplingParamsV2(logit_bias=[(5000, 1.0)]))], "token 5000 at index 0 is outside the vocabulary of size 4096"),
    ]
    for rows, message in cases:
        with pytest.raises(rb.InvalidArgument) as err:
            engine.step(rows, out)
        assert str(err.value) == message
        assert out.n_rows == 0
    assert engine.seq_pos(0) == (-1, -1) and engine.memory().cells_used == 0
    # a gap is a runtime condition, reported with -1
    engine.step([rb.StepRow(0, 0, [5, 6], 0)], out)
    with pytest.raises(rb.EngineError) as err:
        engine.step([rb.StepRow(0, 0, [7], 5)], out)
    assert not isinstance(err.value, rb.InvalidArgument) and "without a gap" in str(err.value)
    assert engine.seq_pos(0) == (0, 1)
    # v1 entry point: struct_size is the evolution key
    rows_out, _, _ = engine.step_v1([rb.StepRow(3, 1, [9, 10], 0, sample=True, sampling=g)])
    assert rows_out[0].sampled


def test_kv_full_is_a_capacity_condition(rb, c1_model):
    engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=64, n_seq_max=2, n_batch=64, n_ubatch=64))
    out = rb.StepOutput()
    engine.step([rb.StepRow(0, 0, _prompt(1, 64), 0)], out)
    used, total = engine.blocks()
    assert (used, total) == (4, 6)
    engine.step([rb.StepRow(1, 1, _prompt(2, 32), 0)], out)
    with pytest.raises(rb.EngineError) as err:
        engine.step([rb.StepRow(1, 1, _prompt(3, 16), 32)], out)   # would need a 7th block
    assert "KV cache is full" in str(err.value)
    assert engine.seq_pos(1) == (0, 31)                      # the refused step left nothing behind
    engine.seq_rm(0)
    engine.step([rb.StepRow(1, 1, _prompt(3, 16), 32)], out)
    assert engine.memory().cells_used == 48
    engine.close()


def test_prefix_copy_continuation_equals_cold_and_oracle(rb, oracle, pair):
    """seq_cp is metadata-only (shared blocks + copy-on-write of the boundary block) and a
    continuation after it is bit-identical to a cold prefill (tests/engine_runtime.rs:822-998)."""
    engine, octx = pair
    out = rb.StepOutput()
    rep = ParityReport()
    g = rb.SamplingParamsV2.greedy()
    prompt = _prompt(11, 53)
    check_step(rb, engine, octx, oracle, [rb.StepRow(0, 0, prompt[:37], 0)], out, rep)
    blocks_before = engine.blocks()[0]
    engine.seq_cp(0, 1, 0, 37)
    octx.seq_cp(0, 1, 0, 37)
    assert engine.blocks()[0] == blocks_before                       # nothing copied yet
    assert engine.seq_pos(1) == (0, 36) and engine.memory().cells_used == 74
    t0, _ = engine.block_table(0)
    t1, _ = engine.block_table(1)
    assert np.array_equal(t0, t1)
    toks = check_step(rb, engine, octx, oracle, [rb.StepRow(1, 1, prompt[37:], 37, sample=True, sampling=g)], out, rep)
    expect_greedy(oracle, toks, rep)
    warm = engine.last_logits(0)
    t1b, _ = engine.block_table(1)
    assert t1b[2] != t0[2] and np.array_equal(t1b[:2], t0[:2])        # boundary block copied, full blocks shared
    # the source continues independently with other tokens
    toks = check_step(rb, engine, octx, oracle, [rb.StepRow(2, 0, _prompt(12, 5), 37, sample=True, sampling=g)], out, rep)
    expect_greedy(oracle, toks, rep)
    # cold run in a fresh slot with the same step shapes: bit-identical logits (shared blocks + the
    # copied boundary block hold exactly what a cold prefill writes)
    check_step(rb, engine, octx, oracle, [rb.StepRow(3, 2, prompt[:37], 0)], out, rep)
    check_step(rb, engine, octx, oracle, [rb.StepRow(3, 2, prompt[37:], 37, sample=True, sampling=g)], out, rep)
    cold = engine.last_logits(0)
    assert np.array_equal(warm, cold)
    # one-shot prefill of the whole prompt: other kernels, other summation order - same greedy token
    check_step(rb, engine, octx, oracle, [rb.StepRow(4, 3, prompt, 0, sample=True, sampling=g)], out, rep)
    one_shot = engine.last_logits(0)
    assert int(np.argmax(one_shot)) == int(np.argmax(warm)) and np.abs(one_shot - warm).max() < 1e-3


def test_seq_rm_ranges_and_memory_accounting(rb, oracle, pair):
    engine, octx = pair
    out = rb.StepOutput()
    rep = ParityReport()
    g = rb.SamplingParamsV2.greedy()
    prompt = _prompt(21, 40)
    check_step(rb, engine, octx, oracle, [rb.StepRow(0, 0, prompt, 0)], out, rep)
    info = engine.memory()
    assert (info.n_slots, info.cells_total, info.cells_used, info.recurrent_bytes) == (8, 1024, 40, 0) and info.kv_bytes > 0
    engine.seq_rm(0, 30, -1)
    octx.seq_rm(0, 30, -1)
    assert engine.seq_pos(0) == (0, 29)
    with pytest.raises(rb.EngineError) as err:
        engine.seq_rm(0, 5, 9)
    assert str(err.value) == "the memory cannot remove that partial range; remove the whole sequence instead"
    # re-decode the tail: same logits as an uninterrupted run
    toks = check_step(rb, engine, octx, oracle, [rb.StepRow(0, 0, prompt[30:], 30, sample=True, sampling=g)], out, rep)
    expect_greedy(oracle, toks, rep)
    again = engine.last_logits(0)
    # the same two steps in a fresh slot give the same bits; a one-shot prefill the same token
    check_step(rb, engine, octx, oracle, [rb.StepRow(1, 1, prompt[:30], 0)], out, rep)
    check_step(rb, engine, octx, oracle, [rb.StepRow(1, 1, prompt[30:], 30, sample=True, sampling=g)], out, rep)
    assert np.array_equal(again, engine.last_logits(0))
    check_step(rb, engine, octx, oracle, [rb.StepRow(2, 2, prompt, 0, sample=True, sampling=g)], out, rep)
    assert int(np.argmax(engine.last_logits(0))) == int(np.argmax(again)) and np.abs(engine.last_logits(0) - again).max() < 1e-3
    engine.seq_rm(0)
    assert engine.seq_pos(0) == (-1, -1)
    engine.seq_rm(0)   # removing an empty slot is fine


def test_snapshot_round_trip(rb, oracle, pair):
    """seq_save / seq_load: two-call size contract, bit-identical continuation, corrupt or
    truncated data refused (tests/engine_runtime.rs:907-943)."""
    engine, octx = pair
    out = rb.StepOutput()
    g = rb.SamplingParamsV2.greedy()
    prompt = _prompt(31, 45)
    engine.step([rb.StepRow(0, 0, prompt[:33], 0)], out)
    blob = engine.seq_save(0)
    engine.step([rb.StepRow(0, 0, prompt[33:], 33, sample=True, sampling=g)], out)
    direct = engine.last_logits(0)
    assert engine.seq_load(5, blob) == len(blob)
    assert engine.seq_pos(5) == (0, 32)
    engine.step([rb.StepRow(1, 5, prompt[33:], 33, sample=True, sampling=g)], out)
    assert np.array_equal(direct, engine.last_logits(0))
    bad = bytearray(blob)
    bad[-1] ^= 0xFF
    for data in (bytes(bad), blob[: len(blob) // 2], b"junk"):
        with pytest.raises(rb.EngineError) as err:
            engine.seq_load(6, data)
        assert str(err.value) == "the snapshot was refused (wrong size, flags or corrupted data)"
    assert engine.seq_pos(6) == (-1, -1)
    with pytest.raises(rb.EngineError):
        engine.seq_save(0, flags=2)   # ON_DEVICE snapshots are refused


def test_logprobs_and_top_logprobs_match_the_oracle(rb, oracle, pair):
    """v1 rows report the raw temperature-1 top-k (logit desc, id asc); v2 rows report the top-k of
    the post-transformation distribution, truncated to the nucleus (retro_lora_train.h:1364-1369)."""
    engine, octx = pair
    sp = rb.SamplingParamsV2.from_v1(rb.SamplingParams(1e-4, 1e-6, 1, 0))
    rows = [rb.StepRow(i, i, _prompt(40 + i, 12 + i), 0, sample=True, sampling=sp, n_top_logprobs=5) for i in range(3)]
    outs, ids, lps = engine.step_v1(rows, out_stride=6)
    for r in range(3):
        logits = engine.last_logits(r)
        o = outs[r]
        assert o.token == int(np.argmax(logits)) and o.n_top == 5
        assert o.logprob == oracle.token_logprob(logits, o.token)
        want_ids, want_lps = oracle.top_token_logprobs(logits, 5)
        assert np.array_equal(ids[r, :5], want_ids)
        assert np.allclose(lps[r, :5], want_lps, rtol=0, atol=2e-6)
    for i in range(3):
        engine.seq_rm(i)
        engine.request_free(i)
    out = rb.StepOutput()
    engine.step(rows, out)
    for r in range(3):
        logits = engine.last_logits(r)
        tok, lp, slp, want_ids, want_lps = oracle.sample_token_v2(logits, oracle.Rng(0), temperature=1e-4, top_p=1e-6, k=5)
        o = out.row(r)
        got_ids, got_lps = out.top(r)
        assert o.token == tok and o.logprob == pytest.approx(lp, abs=2e-6)
        assert np.array_equal(got_ids, want_ids) and np.array_equal(got_lps, want_lps)


def test_seeded_sampling_is_reproducible_and_matches_its_restatement(rb, oracle, c1_model):
    """Seeded rows draw from a counter-based generator: same seed -> same stream; the token equals
    the CPU restatement of the same draw unless the draw sits on a rounding boundary."""
    def run(seed, temperature, top_p):
        engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=512, n_seq_max=4, n_batch=64, n_ubatch=64))
        out = rb.StepOutput()
        sp = rb.SamplingParamsV2(temperature=temperature, top_p=top_p, seed=seed)
        prompt = _prompt(50, 20)
        engine.step([rb.StepRow(0, 0, prompt, 0, sample=True, sampling=sp)], out)
        stream, checks = [], []
        for i in range(24):
            o = out.row(0)
            logits = engine.last_logits(0)
            want, margin = oracle.sample_philox(logits, temperature, top_p, seed, i)
            checks.append((o.token, want, margin))
            assert o.logprob == pytest.approx(float(oracle.token_logprob(logits, o.token)), abs=2e-6)
            stream.append(o.token)
            engine.step([rb.StepRow.decode(0, 0, o.token, len(prompt) + i, sp)], out)
        engine.close()
        return stream, checks

    for temperature, top_p in ((1.0, 1.0), (0.8, 0.9), (1.3, 0.5)):
        a, checks = run(7, temperature, top_p)
        b, _ = run(7, temperature, top_p)
        c, _ = run(8, temperature, top_p)
        assert a == b and a != c
        assert len(set(a)) > 4
        for got, want, margin in checks:
            assert got == want or margin < 1e-9, (got, want, margin)


def test_nucleus_and_top_k_restrict_the_support(rb, oracle, pair):
    engine, _ = pair
    out = rb.StepOutput()
    prompt = _prompt(60, 16)
    engine.step([rb.StepRow(0, 0, prompt, 0, sample=True, sampling=rb.SamplingParamsV2.greedy())], out)
    logits = engine.last_logits(0)
    order = np.argsort(-logits, kind="stable")
    p = np.exp((logits.astype(np.float64) - logits.max()))
    p /= p.sum()
    for trial in range(40):
        engine.seq_rm(0)
        sp = rb.SamplingParamsV2(temperature=1.0, top_p=0.02, seed=trial)
        engine.step([rb.StepRow(100 + trial, 0, prompt, 0, sample=True, sampling=sp, want_logprob=True, n_top_logprobs=3)], out)
        n_keep = int(np.searchsorted(np.cumsum(p[order]), 0.02 * (1 - 1e-12)) + 1)
        assert out.row(0).token in set(order[: n_keep + 1].tolist())
        ids, lps = out.top(0)
        assert ids[0] == order[0] and np.all(np.diff(lps) <= 0)
        engine.seq_rm(0)
        sp = rb.SamplingParamsV2(temperature=1.5, top_k=4, seed=trial)
        engine.step([rb.StepRow(200 + trial, 0, prompt, 0, sample=True, sampling=sp)], out)
        assert out.row(0).token in set(order[:4].tolist())


def test_v2_bias_and_penalties_match_the_oracle_when_greedy(rb, oracle, pair):
    """v2 order logit_bias -> penalties(window) -> top_k (retro_lora_train.h:1364-1369): with
    top_k = 1 the draw is deterministic, so token, policy logprob, post-transformation logprob
    and top ids must equal the reference's CPU oracle on the same raw logits."""
    engine, _ = pair
    out = rb.StepOutput()
    prompt = _prompt(70, 10)
    sp = rb.SamplingParamsV2(top_k=1, repeat_penalty=1.3, frequency_penalty=0.4, presence_penalty=0.2, penalty_window=6,
                             logit_bias=[(77, 3.0), (78, -2.0), (77, 1.5)])
    engine.step([rb.StepRow(0, 0, prompt, 0, sample=True, sampling=sp, want_logprob=True, n_top_logprobs=2)], out)
    history = []
    for i in range(12):
        o = out.row(0)
        logits = engine.last_logits(0)
        tok, lp, slp, ids, lps = oracle.sample_token_v2(logits, oracle.Rng(0), top_k=1, repeat_penalty=1.3, frequency_penalty=0.4,
                                                        presence_penalty=0.2, penalty_window=6, logit_bias=list(sp.logit_bias),
                                                        history=history, k=2)
        assert o.token == tok
        assert o.logprob == pytest.approx(lp, abs=2e-6)
        assert o.sampled_logprob == pytest.approx(slp, abs=1e-6)
        got_ids, got_lps = out.top(0)
        assert list(got_ids) == list(ids)
        assert got_lps[0] == pytest.approx(float(lps[0]), abs=1e-6) and got_lps[1] == -np.inf
        history.append(o.token)
        engine.step([rb.StepRow.decode(0, 0, o.token, len(prompt) + i, sp, ) if False else
                     rb.StepRow(0, 0, [o.token], len(prompt) + i, sample=True, sampling=sp, want_logprob=True, n_top_logprobs=2)], out)


def test_min_p_and_temperature_v2_rows_stay_inside_the_kept_set(rb, oracle, pair):
    engine, _ = pair
    out = rb.StepOutput()
    prompt = _prompt(71, 14)
    engine.step([rb.StepRow(0, 0, prompt, 0, sample=True, sampling=rb.SamplingParamsV2.greedy())], out)
    logits = engine.last_logits(0)
    keep = set(np.nonzero(logits >= logits.max() + np.log(np.float32(0.5)))[0].tolist())
    for trial in range(30):
        engine.seq_rm(0)
        sp = rb.SamplingParamsV2(temperature=2.0, min_p=0.5, seed=trial)
        engine.step([rb.StepRow(300 + trial, 0, prompt, 0, sample=True, sampling=sp, want_logprob=True)], out)
        assert out.row(0).token in keep
        assert out.row(0).sampled_logprob <= 0.0


def test_plain_greedy_rows_equal_the_general_sampler_and_the_oracle(rb, oracle, pair):
    """Greedy rows without logit edits are served by a separate chunked arg-max path. A zero logit
    bias sends the same row through the general sampler: both must report identical token,
    logprobs and top lists, and both must equal the oracle on the raw logits."""
    engine, _ = pair
    out = rb.StepOutput()
    plain = rb.SamplingParamsV2(top_k=1)
    general = rb.SamplingParamsV2(top_k=1, logit_bias=[(5, 0.0)])
    rows = []
    for i in range(3):
        prompt = _prompt(90 + i, 9 + 2 * i)
        rows.append(rb.StepRow(2 * i, 2 * i, prompt, 0, sample=True, sampling=plain, want_logprob=True, n_top_logprobs=3))
        rows.append(rb.StepRow(2 * i + 1, 2 * i + 1, prompt, 0, sample=True, sampling=general, want_logprob=True, n_top_logprobs=3))
    engine.step(rows, out)
    for i in range(3):
        a, b = out.row(2 * i), out.row(2 * i + 1)
        assert np.array_equal(engine.last_logits(2 * i), engine.last_logits(2 * i + 1))
        assert (a.token, a.logprob, a.sampled_logprob) == (b.token, b.logprob, b.sampled_logprob)
        ids_a, lps_a = out.top(2 * i)
        ids_b, lps_b = out.top(2 * i + 1)
        assert list(ids_a) == list(ids_b) and np.array_equal(np.asarray(lps_a), np.asarray(lps_b))
        logits = engine.last_logits(2 * i)
        assert a.token == int(np.argmax(logits))
        assert a.logprob == oracle.token_logprob(logits, a.token)
        assert a.sampled_logprob == 0.0 and lps_a[0] == 0.0 and lps_a[1] == -np.inf
    for sid in range(6):
        engine.seq_rm(sid)


def test_repeated_step_shapes_replay_as_cuda_graphs_with_identical_results(rb, oracle, c1_model, monkeypatch):
    """A decode loop repeats one step shape: from its third occurrence on, the step is a replayed CUDA
    graph. Tokens, logprobs and logits must equal the eager engine's bit for bit."""
    def run(graphs: bool):
        monkeypatch.setenv("RB200_GRAPHS", "1" if graphs else "0")
        engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=1024, n_seq_max=4, n_batch=64, n_ubatch=64))
        out = rb.StepOutput()
        g = rb.SamplingParamsV2.greedy()
        prompts = [_prompt(200 + i, 9 + i) for i in range(3)]
        engine.step([rb.StepRow(i, i, p, 0, sample=True, sampling=g, want_logprob=True) for i, p in enumerate(prompts)], out)
        last = [out.row(i).token for i in range(3)]
        trace = []
        for step in range(12):
            rows = [rb.StepRow(i, i, [last[i]], len(prompts[i]) + step, sample=True, sampling=g, want_logprob=True) for i in range(3)]
            engine.step(rows, out)
            last = [out.row(i).token for i in range(3)]
            trace.append(([out.row(i).token for i in range(3)], [out.row(i).logprob for i in range(3)], engine.last_logits(1).copy()))
        stats = engine.graph_stats()
        engine.close()
        return trace, stats
    eager, stats_eager = run(False)
    graphed, stats_graphed = run(True)
    assert stats_eager == (0, 0)
    assert stats_graphed[0] >= 8 and stats_graphed[1] >= 1
    for (t0, l0, x0), (t1, l1, x1) in zip(eager, graphed):
        assert t0 == t1 and l0 == l1 and np.array_equal(x0, x1)


def test_moe_decode_steps_replay_as_cuda_graphs_with_identical_results(rb, models, monkeypatch):
    """Expert routing changes from step to step while the step shape does not: the grouped expert
    launches size their grids from the step's token count, never from the routed counts, so one
    captured graph serves every routing. Tokens, logits and routes must equal the eager engine's."""
    spec = dict(arch="olmoe", layers=2, d=128, heads=4, kv_heads=4, ff=64, vocab=512, experts=8, experts_used=2,
                dtype="q8_0", expert_dtype="mxfp4", seed=21)
    path = models("moe_flat", **spec)

    def run(graphs: bool):
        monkeypatch.setenv("RB200_GRAPHS", "1" if graphs else "0")
        engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=512, n_seq_max=4, n_batch=64, n_ubatch=64))
        out = rb.StepOutput()
        g = rb.SamplingParamsV2.greedy()
        prompts = [_prompt(300 + i, 7 + 2 * i, vocab=512) for i in range(3)]
        engine.step([rb.StepRow(i, i, p, 0, sample=True, sampling=g) for i, p in enumerate(prompts)], out)
        last = [out.row(i).token for i in range(3)]
        trace = []
        for step in range(12):
            rows = [rb.StepRow(i, i, [last[i]], len(prompts[i]) + step, sample=True, sampling=g) for i in range(3)]
            engine.step(rows, out)
            last = [out.row(i).token for i in range(3)]
            trace.append((list(last), engine.last_logits(2).copy(), engine.last_routes().copy()))
        stats = engine.graph_stats()
        engine.close()
        return trace, stats
    eager, stats_eager = run(False)
    graphed, stats_graphed = run(True)
    assert stats_eager == (0, 0)
    assert stats_graphed[0] >= 8 and stats_graphed[1] >= 1
    assert len({r.tobytes() for _, _, r in eager}) > 1  # the routing really differs between steps
    for (t0, x0, r0), (t1, x1, r1) in zip(eager, graphed):
        assert t0 == t1 and np.array_equal(x0, x1) and np.array_equal(r0, r1)


@pytest.mark.parametrize("name,spec", [
    ("tails_q4k", dict(arch="llama", layers=3, d=512, heads=8, kv_heads=2, ff=1024, vocab=1024, dtype="q4_k", seed=41)),
    ("tails_q8", dict(arch="llama", layers=3, d=256, heads=4, kv_heads=2, ff=512, vocab=512, dtype="q8_0", seed=42)),
    # q / k / v biases go through the RoPE tail, the half-split rotation of this architecture too
    ("tails_q8_bias", dict(arch="qwen2", layers=2, d=256, heads=4, kv_heads=2, ff=512, vocab=512, dtype="q8_0", seed=43, bias=1)),
])
def test_finish_kernel_tails_equal_the_separate_kernels(rb, models, monkeypatch, name, spec):
    """For at most 16 tokens a step the streaming GEMMs' finish kernels also do the RMS norm or the SwiGLU
    that follows, and the attention merge writes the output projection's operand. The arithmetic and
    its order are those of the separate kernels: tokens, logprobs and logits are equal bit for bit.
    Steps of 3 tokens (one pass) and of 12 tokens (two passes of 8 and 4) cover both forms."""
    def run(fused: bool):
        monkeypatch.setenv("RB200_FUSED_FINISH", "1" if fused else "0")
        engine = rb.Engine(str(models(name, **spec)), rb.EngineConfig(n_ctx=1024, n_seq_max=4, n_batch=128, n_ubatch=128))
        out = rb.StepOutput()
        g = rb.SamplingParamsV2.greedy()
        prompts = [_prompt(300 + i, 20 + 3 * i, spec["vocab"]) for i in range(3)]
        engine.step([rb.StepRow(i, i, p, 0, sample=True, sampling=g, want_logprob=True) for i, p in enumerate(prompts)], out)
        last = [out.row(i).token for i in range(3)]
        pos = [len(p) for p in prompts]
        trace = []
        for step in range(6):
            n = 1 if step % 2 == 0 else 4          # 3 or 12 tokens in the step
            rows = [rb.StepRow(i, i, [last[i]] + _prompt(400 + 10 * step + i, n - 1, spec["vocab"]), pos[i], sample=True, sampling=g, want_logprob=True)
                    for i in range(3)]
            engine.step(rows, out)
            last = [out.row(i).token for i in range(3)]
            pos = [q + n for q in pos]
            trace.append(([out.row(i).token for i in range(3)], [out.row(i).logprob for i in range(3)], engine.last_logits(2).copy()))
        engine.close()
        return trace
    separate, fused = run(False), run(True)
    for (t0, l0, x0), (t1, l1, x1) in zip(separate, fused):
        assert t0 == t1 and l0 == l1 and np.array_equal(x0, x1)


def _greedy_v1(n_new, seed=0):
    # the serving layer's spelling of greedy for v1 rows: a nucleus that holds one token
    return dict(temperature=1e-4, top_p=1e-6, max_new_tokens=n_new, seed=seed)


def test_batched_generators_equal_the_step_loop_and_the_oracle(rb, oracle, pair):
    """retro_engine_generate_continuous_batch / _generate_batch run the same steps a caller would:
    greedy-equivalent rows must reproduce the oracle's arg-max chain, logprobs its temperature-1 policy
    values, and nothing stays resident afterwards."""
    engine, octx = pair
    prompts = [_prompt(300 + i, 5 + 7 * i) for i in range(3)]
    n_new = 6
    got, lps = engine.generate_continuous([(p, rb.SamplingParams(**_greedy_v1(n_new, seed=i))) for i, p in enumerate(prompts)], n_out_max=8)
    assert engine.memory().cells_used == 0
    for i, p in enumerate(prompts):
        seq = list(p)
        octx.seq_rm(i)
        logits = octx.step([(i, seq, 0, True, 0)])[0]
        want, want_lp = [], []
        for step in range(n_new):
            tok = int(np.argmax(logits))
            want.append(tok)
            want_lp.append(float(oracle.token_logprob(logits, tok)))
            if step + 1 < n_new:
                logits = octx.step([(i, [tok], len(p) + step, True, 0)])[0]
        assert got[i] == want
        assert np.allclose(lps[i], want_lp, rtol=0, atol=2e-4)      # the two sides differ in their logits by up to ~1e-4
        octx.seq_rm(i)
    # one prompt, three members: identical greedy streams, equal to the first sequence above
    members, _ = engine.generate_batch(prompts[0], [rb.SamplingParams(**_greedy_v1(n_new, seed=s)) for s in (1, 2, 3)], n_out_max=8)
    assert members[0] == members[1] == members[2] == got[0]
    assert engine.memory().cells_used == 0
    # n_out_max caps a row before max_new_tokens does
    short, _ = engine.generate_batch(prompts[1], [rb.SamplingParams(**_greedy_v1(n_new))], n_out_max=2)
    assert short[0] == got[1][:2]


def test_batched_generator_validation(rb, pair):
    engine, _ = pair
    good = rb.SamplingParams(temperature=1.0, top_p=1.0, max_new_tokens=2, seed=0)
    with pytest.raises(rb.EngineError, match="prompt tokens are required"):
        engine.generate_batch([], [good], 4)
    with pytest.raises(rb.EngineError, match="sampling params and output buffers are required"):
        engine.generate_batch([5, 6], [], 4)
    with pytest.raises(rb.EngineError, match="sequences but the context supports 8"):
        engine.generate_batch([5, 6], [good] * 9, 4)
    with pytest.raises(rb.EngineError, match="temperature must be finite"):
        engine.generate_batch([5, 6], [rb.SamplingParams(temperature=0.0, top_p=1.0, max_new_tokens=2)], 4)
    with pytest.raises(rb.EngineError, match="continuous generation inputs and output buffers are required"):
        engine.generate_continuous([], 4)
    with pytest.raises(rb.EngineError, match="invalid continuous generation prompt"):
        engine.generate_continuous([([], good)], 4)


def test_scheduler_composed_steps_reproduce_the_generators(rb, pair):
    """Plans composed the way the reference's scheduler does (retrograd_b200/scheduler.py): a merged group of
    three members (leader prefill of all but the last prompt token, prefix copied to the members, one terminal
    row each, then decode) beside two single requests, under continuous admission with a budget small
    enough that prefill is chunked, a token is kept for it, and the decode cursor rotates. Every request's
    greedy stream must equal what the engine's own generators produce for it."""
    from oracle.scheduler import CONTINUOUS, ComposeState, Group, Member, compose

    engine, _ = pair
    n_new = 5
    greedy = rb.SamplingParamsV2.greedy()
    shared = _prompt(500, 23)
    singles = [_prompt(501, 17), _prompt(502, 9)]
    want_shared, _ = engine.generate_batch(shared, [rb.SamplingParams(**_greedy_v1(n_new, seed=s)) for s in range(3)], n_out_max=n_new)
    want_single, _ = engine.generate_continuous([(p, rb.SamplingParams(**_greedy_v1(n_new))) for p in singles], n_out_max=n_new)

    live = [Group(prompt=shared, members=[Member(request_id=10 + i, slot=i, sampling=greedy) for i in range(3)], prefix_end=len(shared) - 1)]
    live += [Group(prompt=p, members=[Member(request_id=20 + i, slot=3 + i, sampling=greedy)], prefix_end=len(p)) for i, p in enumerate(singles)]
    streams = {m.request_id: [] for g in live for m in g.members}
    state, out = ComposeState(), rb.StepOutput()
    for _ in range(200):
        if all(not m.live for g in live for m in g.members):
            break
        rows, used = compose(live, 6, CONTINUOUS, state)
        assert 0 < used <= 6
        engine.step([rb.StepRow(r.request, r.slot, r.tokens, r.pos0, r.sample, r.sampling) for r in rows], out)
        for i, r in enumerate(rows):
            g = live[r.kind[1]]
            if r.kind[0] == "prefill":
                g.pos = r.kind[2]
                member = g.members[0] if r.kind[3] is not None else None
            else:
                member = g.members[r.kind[2]]
                if r.kind[0] == "terminal":
                    g.next_member = r.kind[2] + 1
            if member is not None:
                tok = out.row(i).token
                streams[member.request_id].append(tok)
                member.next_token, member.generated = tok, member.generated + 1
                if member.generated >= n_new:
                    member.live = False
                    engine.seq_rm(member.slot)
        # phase changes between steps: a finished prefix is copied to the other members; a finished terminal wave decodes
        for g in live:
            if g.phase == "prefill" and g.pos == g.prefix_end:
                if len(g.members) > 1:
                    for m in g.members[1:]:
                        engine.seq_cp(g.members[0].slot, m.slot, 0, g.prefix_end)
                    g.phase = "terminal"
                else:
                    g.phase = "decode"
            if g.phase == "terminal" and g.next_member >= len(g.members):
                g.phase = "decode"
    assert [streams[10 + i] for i in range(3)] == want_shared
    assert [streams[20 + i] for i in range(2)] == want_single
    assert engine.memory().cells_used == 0


def test_mixed_steps_with_the_attention_overlap_replay_as_graphs(rb, c1_model, monkeypatch):
    """A step with decode rows and a prefill chunk forks the decode-row attention onto a second stream. The
    same step shape repeated is captured (fork and join included) and replayed: results equal the eager run."""
    def run(graphs: bool):
        monkeypatch.setenv("RB200_GRAPHS", "1" if graphs else "0")
        engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=2048, n_seq_max=4, n_batch=128, n_ubatch=128))
        out = rb.StepOutput()
        g = rb.SamplingParamsV2.greedy()
        prompts = [_prompt(700 + i, 12 + i) for i in range(2)]
        engine.step([rb.StepRow(i, i, p, 0, sample=True, sampling=g) for i, p in enumerate(prompts)], out)
        last = [out.row(i).token for i in range(2)]
        trace = []
        for step in range(8):
            engine.seq_rm(2)
            rows = [rb.StepRow(i, i, [last[i]], len(prompts[i]) + step, sample=True, sampling=g, want_logprob=True) for i in range(2)]
            rows.append(rb.StepRow(2, 2, _prompt(800 + step, 40), 0, sample=True, sampling=g, want_logprob=True))
            engine.step(rows, out)
            last = [out.row(i).token for i in range(2)]
            trace.append(([out.row(i).token for i in range(3)], [out.row(i).logprob for i in range(3)], engine.last_logits(2).copy()))
        stats = engine.graph_stats()
        engine.close()
        return trace, stats
    eager, _ = run(False)
    graphed, stats = run(True)
    assert stats[0] >= 4
    for (t0, l0, x0), (t1, l1, x1) in zip(eager, graphed):
        assert t0 == t1 and l0 == l1 and np.array_equal(x0, x1)


def test_prefix_tree_hits_become_block_table_copies(rb, pair):
    """The caller's prefix index (retrograd_b200/prefix_tree.py) and the engine together: a finished request's
    slot stays dormant under its token path; a later prompt that shares a prefix gets `[0, hit)` by
    `seq_cp` - an exact boundary and a mid-sequence hit - prefills only the rest, and must produce the greedy
    stream of a cold run. The last prompt token is always prefilled (a hit is a strict prefix)."""
    from oracle.prefix_tree import PrefixTree

    engine, _ = pair
    g = rb.SamplingParamsV2.greedy()
    out = rb.StepOutput()
    tree = PrefixTree()

    def run(slot, prompt, n_new, hit=0):
        engine.step([rb.StepRow(slot, slot, prompt[hit:], hit, sample=True, sampling=g)], out)
        toks = [out.row(0).token]
        for step in range(1, n_new):
            engine.step([rb.StepRow(slot, slot, [toks[-1]], len(prompt) + step - 1, sample=True, sampling=g)], out)
            toks.append(out.row(0).token)
        return toks

    base = _prompt(900, 40)
    first = run(0, base, 4)
    # the finished sequence: prompt + generated tokens resident in slot 0 at depth len - 1 (the last token was never fed)
    path = base + first[:-1]
    engine.seq_rm(0, len(path), -1)
    node, attached = tree.insert(0, path, 0)
    assert attached and engine.seq_pos(0) == (0, len(path) - 1)

    usable = lambda n, hit: n.slot is not None and engine.seq_pos(n.slot) == (0, n.depth - 1)
    for slot, prompt in ((1, path + _prompt(901, 6)), (2, base[:25] + _prompt(902, 9))):
        cold = run(3, prompt, 4)
        engine.seq_rm(3)
        found = tree.longest_prefix(0, prompt[:-1], True, usable)       # strict prefix: the last prompt token is prefilled
        assert found is not None
        holder, hit = found
        assert hit == (len(path) if slot == 1 else 25)
        tree.touch(holder)
        engine.seq_cp(holder.slot, slot, 0, hit)
        assert run(slot, prompt, 4, hit=hit) == cold
        engine.seq_rm(slot)
    # eviction: the dormant slot is released and its node pruned
    victim = tree.eviction_candidate()
    engine.seq_rm(victim.slot)
    tree.remove(victim)
    assert tree.node_count() == 0 and engine.memory().cells_used == 0
