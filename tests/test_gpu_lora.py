"""Per-row LoRA adapters: one decode mixes rows of several adapters, the base model and the
context's own adapter set (retro_lora_train.h:1285-1306,2586-2605; tests/lora_rows.rs:150-240)."""
import numpy as np
import pytest

from helpers import ParityReport, check_step, expect_greedy

pytestmark = pytest.mark.gpu

SPEC = dict(arch="llama", layers=2, d=256, heads=4, kv_heads=2, ff=512, vocab=512, dtype="q8_0", seed=77)
TARGETS = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")


def _write_adapter(path, rank, alpha, seed):
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(seed)
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_string("general.type", "adapter")
    w.add_string("adapter.type", "lora")
    w.add_float32("adapter.lora.alpha", float(alpha))
    d, dkv, ff = 256, 128, 512
    shapes = {"attn_q": (d, d), "attn_k": (d, dkv), "attn_v": (d, dkv), "attn_output": (d, d), "ffn_gate": (d, ff), "ffn_up": (d, ff), "ffn_down": (ff, d)}
    for layer in range(2):
        for t in TARGETS:
            n_in, n_out = shapes[t]
            w.add_tensor(f"blk.{layer}.{t}.weight.lora_a", rng.normal(0, 0.05, (rank, n_in)).astype(np.float32))
            w.add_tensor(f"blk.{layer}.{t}.weight.lora_b", rng.normal(0, 0.05, (n_out, rank)).astype(np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def test_mixed_adapter_rows_match_the_oracle_and_each_adapter_alone(rb, oracle, models, tmp_path):
    model = models("lora_base", **SPEC)
    a_path, b_path = tmp_path / "a.gguf", tmp_path / "b.gguf"
    _write_adapter(a_path, rank=8, alpha=32, seed=1)
    _write_adapter(b_path, rank=16, alpha=32, seed=2)
    engine = rb.Engine(str(model), rb.EngineConfig(n_ctx=1024, n_seq_max=8, n_batch=128, n_ubatch=128))
    om = oracle.Model(str(model))
    octx = oracle.Context(om, 8, 1024)
    ida, idb = engine.adapter_load(str(a_path)), engine.adapter_load(str(b_path), 0.5)
    assert (ida, idb) == (om.lora_load(str(a_path)), om.lora_load(str(b_path), 0.5))
    info = engine.adapter_rows_info()
    assert info["n_adapters"] == 2 and info["max_rank"] == 16
    assert info["stacked_bytes"] > info["unpadded_bytes"] > 0          # the rank-8 adapter is padded to 16
    out = rb.StepOutput()
    rep = ParityReport()
    g = rb.SamplingParamsV2.greedy()
    rng = np.random.default_rng(5)
    prompts = [rng.integers(3, 512, n).tolist() for n in (21, 9, 14, 30)]
    adapters = [ida, idb, rb.ADAPTER_BASE, 0]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=g, n_top_logprobs=8, adapter=a) for i, (p, a) in enumerate(zip(prompts, adapters))]
    toks = check_step(rb, engine, octx, oracle, rows, out, rep)
    expect_greedy(oracle, toks, rep)
    mixed = [(out.row(i).token, out.row(i).logprob, engine.last_logits(i)) for i in range(4)]
    # each row alone, in a fresh slot: same token, logprob within 1e-3 (tests/lora_rows.rs:34-37)
    for i, (p, a) in enumerate(zip(prompts, adapters)):
        engine.step([rb.StepRow(10 + i, 4 + i, p, 0, sample=True, sampling=g, adapter=a)], out)
        assert out.row(0).token == mixed[i][0]
        assert abs(out.row(0).logprob - mixed[i][1]) < 1e-3
    # the adapters really change the output
    base_logits = mixed[2][2]
    engine.seq_rm(2)
    engine.step([rb.StepRow(21, 2, prompts[2], 0, sample=True, sampling=g, adapter=ida)], out)
    assert np.abs(engine.last_logits(0) - base_logits).max() > 1e-2
    # decode steps keep following the oracle under mixed adapters
    for step in range(3):
        rows = [rb.StepRow(i, i, [mixed[i][0]] if step == 0 else [last[i]], len(prompts[i]) + step, sample=True, sampling=g, adapter=adapters[i])
                for i in (0, 1, 3)]
        toks = check_step(rb, engine, octx, oracle, rows, out, rep)
        expect_greedy(oracle, toks, rep)
        last = {i: out.row(r).token for r, i in enumerate((0, 1, 3))}
    print(f"lora: max|dlogit|={rep.max_logit_diff:.3e} ties={rep.tie_events}")
    # unloading: the id stops being accepted, the others keep working
    engine.adapter_unload(ida)
    with pytest.raises(rb.InvalidArgument):
        engine.step([rb.StepRow(30, 7, [5], 0, adapter=ida)], out)
    engine.step([rb.StepRow(31, 7, [5, 6], 0, sample=True, sampling=g, adapter=idb)], out)
    assert engine.adapter_rows_info()["n_adapters"] == 1
    engine.close()


def test_tensor_core_and_cuda_core_lora_kernels_agree(rb, models, tmp_path, monkeypatch):
    """The segmented TF32 kernels (split operands, three MMAs per product) against the F32 CUDA-core kernels
    (RB200_LORA=rows) on the same mixed step: ranks 8, 16 and 24 (three rank tiles with padding), segments that
    end in partial 16-token tiles, base rows in between. Logits within 2e-4, the same greedy tokens."""
    model = models("lora_base", **SPEC)
    paths = []
    for i, rank in enumerate((8, 16, 24)):
        paths.append(tmp_path / f"r{rank}.gguf")
        _write_adapter(paths[-1], rank=rank, alpha=32, seed=10 + i)
    g = rb.SamplingParamsV2.greedy()
    rng = np.random.default_rng(6)
    prompts = [rng.integers(3, 512, n).tolist() for n in (37, 5, 18, 16, 1, 33, 9)]
    which = [0, 1, None, 2, 1, 0, 2]
    results = []
    for form in ("tensor_cores", "rows"):
        if form == "rows":
            monkeypatch.setenv("RB200_LORA", "rows")
        else:
            monkeypatch.delenv("RB200_LORA", raising=False)
        engine = rb.Engine(str(model), rb.EngineConfig(n_ctx=1024, n_seq_max=8, n_batch=128, n_ubatch=128))
        ids = [engine.adapter_load(str(p)) for p in paths]
        out = rb.StepOutput()
        rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=g, adapter=rb.ADAPTER_BASE if a is None else ids[a])
                for i, (p, a) in enumerate(zip(prompts, which))]
        engine.step(rows, out)
        results.append(([out.row(i).token for i in range(len(rows))], np.stack([engine.last_logits(i) for i in range(len(rows))])))
        engine.close()
    assert results[0][0] == results[1][0]
    diff = np.abs(results[0][1] - results[1][1]).max()
    print(f"lora tensor-core vs CUDA-core kernels: max|dlogit|={diff:.3e}")
    assert diff < 2e-4         # measured 6e-5: both forms are F32-accurate per product, the sums are ordered differently
