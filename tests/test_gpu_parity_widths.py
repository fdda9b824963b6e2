"""Parity with the CPU oracle at the WIDTHS of the large workloads (8B-class d 4096 / 32 query, 8 KV heads of 128 /
FFN 14336 / vocabulary 128 256; the 20B-class MoE's d 2880 / 64 x 8 heads of 64 / 32 experts top-4), with the
depth cut to two layers so that the oracle finishes in about a minute per test. The kernels a step picks depend
on widths and token counts, not on depth: these are the shapes the benchmark times.

Every test prints max |dlogit|, the smallest top-2 margin the oracle saw and the number of tie events."""
import numpy as np
import pytest

from helpers import ParityReport, check_step, expect_greedy

pytestmark = pytest.mark.gpu

WIDE = dict(arch="llama", layers=2, d=4096, heads=32, kv_heads=8, ff=14336, vocab=128256)


def _summary(name, rep):
    print(f"{name}: steps={rep.steps} sampled={rep.sampled} max|dlogit|={rep.max_logit_diff:.3e} min top-2 margin={rep.min_margin:.3e} "
          f"tie events={rep.tie_events}")


def _prefill_both(rb, engine, octx, out, plans, chunk=512, n_batch=2048):
    """Makes [0, n) of every (slot, tokens) resident on both sides without comparing (the comparison comes with
    the steps that follow): the engine in scheduler-like steps of up to n_batch tokens, the oracle row by row."""
    pending = [(slot, toks, 0) for slot, toks in plans]
    while pending:
        rows, rest, budget = [], [], n_batch
        for slot, toks, pos in pending:
            take = min(chunk, len(toks) - pos, budget)
            if take <= 0:
                rest.append((slot, toks, pos))
                continue
            rows.append(rb.StepRow(-1, slot, toks[pos : pos + take], pos, sample=False))
            budget -= take
            if pos + take < len(toks):
                rest.append((slot, toks, pos + take))
        engine.step(rows, out)
        octx.step([(r.slot, list(r.tokens), r.pos0, False) for r in rows])
        pending = rest


def test_mixed_step_shape_at_8b_widths_q4k(rb, oracle, models):
    """The step shape of the headline workload: 16 decode rows over resident contexts of 64..2048 tokens in the SAME
    step as a 512-token chunk continuing a sequence and a 100-token chunk (not a multiple of any tile), then decode
    steps of 18 rows. Runs the tcgen05 GEMM with a ragged last tile, the prefill attention tiles, the 9..16-vector
    and the eight-column decode attention on two streams, and afterwards the split-K / two-pass forms."""
    path = models("wide_q4k", **WIDE, dtype="q4_k", seed=2)
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=40000, n_seq_max=20, n_batch=2048, n_ubatch=2048))
    om = oracle.Model(str(path), fast=True)
    octx = oracle.Context(om, 20, 4096)
    out = rb.StepOutput(2048, 0)
    rep = ParityReport()
    rng = np.random.default_rng(42)
    greedy = rb.SamplingParamsV2.greedy()
    contexts = [64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536, 2047, 80, 150, 300, 600, 1200]
    seqs = {slot: rng.integers(3, 128256, n).tolist() for slot, n in enumerate(contexts)}
    seqs[16] = rng.integers(3, 128256, 1024).tolist()      # 512 resident, 512 more in the mixed step
    seqs[17] = rng.integers(3, 128256, 100).tolist()       # arrives whole in the mixed step
    _prefill_both(rb, engine, octx, out, [(s, seqs[s][:-1]) for s in range(16)] + [(16, seqs[16][:512])])
    rows = [rb.StepRow(s, s, [seqs[s][-1]], len(seqs[s]) - 1, sample=True, sampling=greedy) for s in range(16)]
    rows.append(rb.StepRow(16, 16, seqs[16][512:], 512, sample=True, sampling=greedy))
    rows.append(rb.StepRow(17, 17, seqs[17], 0, sample=True, sampling=greedy))
    # 628 tokens = five token tiles, the last one 116 tokens wide
    assert sum(len(r.tokens) for r in rows) == 16 + 512 + 100
    for step in range(3):
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        expect_greedy(oracle, toks, rep)
        rows = [rb.StepRow.decode(s, s, out.row(i).token, len(seqs[s]) + step, greedy) for i, s in enumerate(range(18))]
    _summary("8B widths Q4_K mixed step", rep)
    assert rep.sampled == 3 * 18
    engine.close()


def test_rollout_groups_at_8b_widths_q8_0(rb, oracle, models):
    """The GRPO-style rollout shape: three prompts, each decoded once and shared by a group of 8 through seq_cp,
    then steps of 24 rows - more than 16 tokens, so the Q8_0 tensor-core GEMM runs at row lengths 4096 and 14336 -
    and prefill chunks of 64 tokens through the same kernel. Greedy streams against the oracle's."""
    path = models("wide_q8", **WIDE, dtype="q8_0", seed=3)
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=16384, n_seq_max=24, n_batch=256, n_ubatch=256))
    om = oracle.Model(str(path), fast=True)
    octx = oracle.Context(om, 24, 2048)
    out = rb.StepOutput(256, 0)
    rep = ParityReport()
    rng = np.random.default_rng(43)
    greedy = rb.SamplingParamsV2.greedy()
    prompts = [rng.integers(3, 128256, n).tolist() for n in (200, 260, 310)]
    # each prompt but its last token into its leader's slot, in 64-token chunks of all three leaders per step
    pos = [0, 0, 0]
    while any(p < len(t) - 1 for p, t in zip(pos, prompts)):
        rows = []
        for g, toks in enumerate(prompts):
            take = min(64, len(toks) - 1 - pos[g])
            if take > 0:
                rows.append(rb.StepRow(-1, 8 * g, toks[pos[g] : pos[g] + take], pos[g], sample=False))
                pos[g] += take
        check_step(rb, engine, octx, oracle, rows, out, rep)
    for g in range(3):
        for m in range(1, 8):
            engine.seq_cp(8 * g, 8 * g + m)
            octx.seq_cp(8 * g, 8 * g + m, -1, -1)
    rows = [rb.StepRow(8 * g + m, 8 * g + m, [prompts[g][-1]], len(prompts[g]) - 1, sample=True, sampling=greedy) for g in range(3) for m in range(8)]
    for step in range(4):
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        expect_greedy(oracle, toks, rep)
        rows = [rb.StepRow.decode(r.slot, r.slot, out.row(i).token, r.pos0 + len(r.tokens), greedy) for i, r in enumerate(rows)]
    _summary("8B widths Q8_0 rollout groups", rep)
    assert rep.sampled == 4 * 24
    # members of a group see the same prefix and, greedy, produce the same stream
    engine.close()


def _write_wide_adapter(path, rank, alpha, seed, layers=2):
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(seed)
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_string("general.type", "adapter")
    w.add_string("adapter.type", "lora")
    w.add_float32("adapter.lora.alpha", float(alpha))
    d, dkv, ff = 4096, 1024, 14336
    shapes = {"attn_q": (d, d), "attn_k": (d, dkv), "attn_v": (d, dkv), "attn_output": (d, d), "ffn_gate": (d, ff), "ffn_up": (d, ff), "ffn_down": (ff, d)}
    for layer in range(layers):
        for target, (n_in, n_out) in shapes.items():
            w.add_tensor(f"blk.{layer}.{target}.weight.lora_a", rng.normal(0, 0.02, (rank, n_in)).astype(np.float32))
            w.add_tensor(f"blk.{layer}.{target}.weight.lora_b", rng.normal(0, 0.02, (n_out, rank)).astype(np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def test_sixteen_adapters_zipf_at_8b_widths(rb, oracle, models, tmp_path):
    """The multi-adapter workload's shape: the Q4_K base with 16 rank-16 adapters (alpha 32) on all seven targets,
    36 rows assigned to adapters by Zipf(1.1) in one step, then decode steps; against the oracle, and every row
    again ALONE in a fresh slot within 1e-3 of its logprob (the reference's own criterion, tests/lora_rows.rs:34-37)."""
    path = models("wide_q4k", **WIDE, dtype="q4_k", seed=2)
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=16384, n_seq_max=80, n_batch=2048, n_ubatch=2048))
    om = oracle.Model(str(path), fast=True)
    octx = oracle.Context(om, 80, 512)
    ids = []
    for a in range(16):
        apath = tmp_path / f"adapter{a}.gguf"
        _write_wide_adapter(apath, rank=16, alpha=32, seed=100 + a)
        ids.append(engine.adapter_load(str(apath)))
        assert om.lora_load(str(apath)) == ids[-1]
        apath.unlink()
    info = engine.adapter_rows_info()
    assert info["n_adapters"] == 16 and info["max_rank"] == 16 and info["stacked_bytes"] == info["unpadded_bytes"]
    rng = np.random.default_rng(44)
    weights = 1.0 / np.arange(1, 17) ** 1.1
    assigned = rng.choice(16, size=36, p=weights / weights.sum())
    assert len(set(assigned.tolist())) >= 6
    greedy = rb.SamplingParamsV2.greedy()
    out = rb.StepOutput(2048, 8)
    rep = ParityReport()
    prompts = [rng.integers(3, 128256, int(rng.integers(12, 40))).tolist() for _ in range(36)]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=greedy, n_top_logprobs=8, adapter=ids[a]) for i, (p, a) in enumerate(zip(prompts, assigned))]
    rows[5].adapter = rb.ADAPTER_BASE          # a base row in the mix
    toks = check_step(rb, engine, octx, oracle, rows, out, rep)
    expect_greedy(oracle, toks, rep)
    mixed = [(out.row(i).token, out.row(i).logprob, out.top(i)[0].copy()) for i in range(36)]
    for i in range(36):         # each row alone, in a fresh slot
        engine.step([rb.StepRow(100 + i, 40 + i, prompts[i], 0, sample=True, sampling=greedy, n_top_logprobs=8, adapter=rows[i].adapter)], out)
        assert out.row(0).token == mixed[i][0] and abs(out.row(0).logprob - mixed[i][1]) < 1e-3
        assert np.array_equal(out.top(0)[0], mixed[i][2])        # the same top-8 ids
    for step in range(2):       # decode steps of 36 rows under the mixed adapters
        rows = [rb.StepRow(i, i, [mixed[i][0]] if step == 0 else [last[i]], len(prompts[i]) + step, sample=True, sampling=greedy, adapter=rows[i].adapter)
                for i in range(36)]
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        expect_greedy(oracle, toks, rep)
        last = [out.row(i).token for i in range(36)]
    _summary("8B widths Q4_K + 16 adapters (Zipf 1.1)", rep)
    engine.close()


@pytest.mark.parametrize("experts", ["tensor_cores", "rows"])
def test_moe_20b_widths_mxfp4(rb, oracle, models, monkeypatch, experts):
    """The MoE workload's widths: d 2880 (not a multiple of 256: no tiled copies, no streaming or tcgen05 kernel),
    64 query / 8 KV heads of 64, 32 experts top-4 of FFN width 2880 in MXFP4, the rest Q8_0. Router choices bit
    for bit, logits within tolerance, with the expert FFNs on the tensor cores and (RB200_MOE=rows) on CUDA cores."""
    if experts == "rows":
        monkeypatch.setenv("RB200_MOE", "rows")
    else:
        monkeypatch.delenv("RB200_MOE", raising=False)
    spec = dict(arch="olmoe", layers=2, d=2880, heads=64, kv_heads=8, head_dim=64, ff=2880, vocab=201088, experts=32, experts_used=4,
                dtype="q8_0", expert_dtype="mxfp4", seed=5)
    path = models("moe_wide", **spec)
    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=8192, n_seq_max=24, n_batch=1024, n_ubatch=1024))
    om = oracle.Model(str(path), fast=True)
    octx = oracle.Context(om, 24, 1024)
    out = rb.StepOutput(1024, 0)
    rep = ParityReport()
    rng = np.random.default_rng(45)
    greedy = rb.SamplingParamsV2.greedy()
    prompts = [rng.integers(3, 201088, n).tolist() for n in (130, 64, 9, 33, 77, 21, 50, 18, 95, 40, 12, 27)]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=greedy) for i, p in enumerate(prompts)]
    route_ties = 0
    for step in range(3):
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        expect_greedy(oracle, toks, rep)
        T = sum(len(r.tokens) for r in rows)
        got = engine.last_routes().reshape(om.n_layer, T, 4)
        want = octx.last_routes().reshape(om.n_layer, T, 4)
        # Routing must agree bit for bit wherever the oracle's own probabilities decide it: a token whose deciding
        # gap is below 2e-6 in some layer is a tie that any reordering of an f32 sum may flip; it is counted, and
        # from that layer on the token is not compared. None of them may be a row's sampled (last) token.
        margins = octx.last_route_margins().reshape(om.n_layer, T)
        clear = np.logical_and.accumulate(margins > 2e-6, axis=0)
        route_ties += int((~clear).any(axis=0).sum())
        assert np.array_equal(got[clear], want[clear]), f"{int((got[clear] != want[clear]).sum())} routed expert ids differ away from ties"
        ends = np.cumsum([len(r.tokens) for r in rows]) - 1
        assert clear[:, ends].all(), "a sampled row's token sits on a routing tie: pick another seed"
        rows = [rb.StepRow.decode(i, i, out.row(i).token, len(prompts[i]) + step, greedy) for i in range(len(prompts))]
    assert len(np.unique(got)) > 8
    _summary(f"20B-MoE widths MXFP4 ({experts})", rep)
    print(f"routing: {route_ties} tokens on a tie (gap <= 2e-6)")
    assert route_ties <= 6
    engine.close()
