"""The rest of the reference's engine boundary on a GPU: the one-active-adapter family, the trainer-owned
generation context, counters, the expert bank inventory and the end-of-generation set."""
import ctypes as C

import numpy as np
import pytest

from test_gpu_lora import SPEC as LORA_SPEC, _write_adapter

pytestmark = pytest.mark.gpu


def _prompt(seed, n, vocab=512):
    return np.random.default_rng(seed).integers(3, vocab, n).tolist()


def test_active_adapter_rows_equal_the_same_adapter_selected_per_row(rb, models, tmp_path):
    """retro_engine.cpp:756-870: rows with adapter 0 decode under the active adapter; activating clears the KV and
    bumps the weights version; a per-row load of the same file gives the same logits bit for bit."""
    model = models("lora_base", **LORA_SPEC)
    a_path, b_path = tmp_path / "a.gguf", tmp_path / "b.gguf"
    _write_adapter(a_path, rank=8, alpha=32, seed=1)
    _write_adapter(b_path, rank=16, alpha=32, seed=2)
    engine = rb.Engine(str(model), rb.EngineConfig(n_ctx=1024, n_seq_max=8, n_batch=128, n_ubatch=128))
    g = rb.SamplingParamsV2.greedy()
    out = rb.StepOutput()
    p = _prompt(1, 19)
    assert engine.active_adapter() == ""
    engine.step([rb.StepRow(0, 0, p, 0, sample=True, sampling=g)], out)
    base = engine.last_logits(0).copy()
    v0 = engine.weights_version()

    engine.load_lora_named("a", a_path)             # registered, not applied: nothing changes
    assert engine.active_adapter() == "" and engine.weights_version() == v0 and engine.seq_pos(0) == (0, 18)
    with pytest.raises(rb.EngineError, match="no LoRA adapter registered under 'nope'"):
        engine.activate_lora("nope")
    with pytest.raises(rb.EngineError, match="cannot enable LoRA: no adapter is active"):
        engine.set_lora_enabled(True)

    engine.activate_lora("a")
    assert engine.active_adapter() == "a" and engine.weights_version() == v0 + 1
    assert engine.seq_pos(0) == (-1, -1) and engine.memory().cells_used == 0       # the KV was forgotten
    engine.step([rb.StepRow(1, 0, p, 0, sample=True, sampling=g)], out)
    under_a = engine.last_logits(0).copy()
    assert np.abs(under_a - base).max() > 1e-2
    # the registered adapters do not count as per-row adapters, and their ids are not selectable per row
    assert engine.adapter_rows_info()["n_adapters"] == 0
    ida = engine.adapter_load(str(a_path))
    engine.step([rb.StepRow(2, 1, p, 0, sample=True, sampling=g, adapter=ida), rb.StepRow(3, 2, p, 0, sample=True, sampling=g, adapter=rb.ADAPTER_BASE)], out)
    assert np.array_equal(engine.last_logits(0), under_a) and np.array_equal(engine.last_logits(1), base)
    assert engine.weights_version() == v0 + 1        # per-row loads leave the KV and the version alone

    # a second adapter beside the first; switching forgets the KV again
    engine.load_lora_named("b", b_path)
    engine.activate_lora("b")
    assert engine.active_adapter() == "b" and engine.weights_version() == v0 + 2 and engine.seq_pos(1) == (-1, -1)
    engine.step([rb.StepRow(4, 0, p, 0, sample=True, sampling=g)], out)
    under_b = engine.last_logits(0).copy()
    assert np.abs(under_b - under_a).max() > 1e-2
    # reloading the ACTIVE adapter re-applies it (KV forgotten); reloading another one does not
    engine.load_lora_named("a", a_path)
    assert engine.weights_version() == v0 + 2
    engine.load_lora_named("b", b_path)
    assert engine.weights_version() == v0 + 3
    # disabling is a weights change too
    engine.set_lora_enabled(False)
    assert engine.active_adapter() == "" and engine.weights_version() == v0 + 4
    engine.step([rb.StepRow(5, 0, p, 0, sample=True, sampling=g)], out)
    assert np.array_equal(engine.last_logits(0), base)
    # the historical single-adapter call: every registered adapter goes, the file becomes the active one
    engine.load_lora(a_path)
    assert engine.active_adapter() == str(a_path) and engine.weights_version() == v0 + 5
    with pytest.raises(rb.EngineError):
        engine.activate_lora("b")
    engine.step([rb.StepRow(6, 0, p, 0, sample=True, sampling=g)], out)
    assert np.array_equal(engine.last_logits(0), under_a)
    # two-call text contract of the name query
    lib = rb.load_library()
    n = C.c_size_t()
    small = C.create_string_buffer(3)
    assert lib.retro_engine_active_adapter(engine._h, small, 3, C.byref(n)) == -2 and n.value == len(str(a_path))
    engine.close()


def test_trainer_owned_generation_context_twins(rb, models, tmp_path):
    """retro_lora_train.h:1906-1945: the same step and sequence operations on a trainer's generation context. A
    weight update forgets the KV and bumps the version; a snapshot freezes the trained adapter as a per-row one."""
    model = models("lora_base", **LORA_SPEC)
    a_path, b_path = tmp_path / "a.gguf", tmp_path / "b.gguf"
    _write_adapter(a_path, rank=8, alpha=32, seed=1)
    _write_adapter(b_path, rank=8, alpha=32, seed=3)
    cfg = rb.EngineConfig(n_ctx=1024, n_seq_max=8, n_batch=128, n_ubatch=128)
    engine = rb.Engine(str(model), cfg)
    engine.load_lora(a_path)
    trainer = rb.TrainerGeneration(str(model), cfg, adapter_path=a_path)
    g = rb.SamplingParamsV2.greedy()
    out_e, out_t = rb.StepOutput(), rb.StepOutput()
    prompts = [_prompt(10 + i, 9 + 4 * i) for i in range(3)]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=g, want_logprob=True) for i, p in enumerate(prompts)]
    engine.step(rows, out_e)
    trainer.step(rows, out_t)
    for step in range(4):
        assert [(r.token, r.logprob) for r in out_e.rows()] == [(r.token, r.logprob) for r in out_t.rows()]
        rows = [rb.StepRow(i, i, [out_e.row(i).token], len(prompts[i]) + step, sample=True, sampling=g, want_logprob=True) for i in range(3)]
        engine.step(rows, out_e)
        trainer.step(rows, out_t)
    assert trainer.seq_pos(0) == engine.seq_pos(0) and trainer.memory().cells_used == engine.memory().cells_used
    assert trainer.kv_unified() and trainer.seq_save(1) == engine.seq_save(1)
    v1_rows, _, _ = trainer.step_v1([rb.StepRow(7, 5, prompts[0], 0, sample=True, sampling=rb.SamplingParams(temperature=1e-4, top_p=1e-6))])
    assert v1_rows[0].sampled
    # the policy is frozen as a per-row adapter, then the weights move on
    v = trainer.weights_version()
    snap = trainer.adapter_snapshot()
    assert trainer.adapter_rows_info()["n_adapters"] == 1 and trainer.weights_version() == v
    trainer.seq_rm(0)
    trainer.step([rb.StepRow(20, 0, prompts[0], 0, sample=True, sampling=g, want_logprob=True)], out_t)
    before = (out_t.row(0).token, out_t.row(0).logprob)
    trainer.weights_updated(b_path)                  # the optimizer stepped: new adapter weights
    assert trainer.weights_version() == v + 1 and trainer.seq_pos(0) == (-1, -1)
    trainer.step([rb.StepRow(21, 0, prompts[0], 0, sample=True, sampling=g, want_logprob=True),
                  rb.StepRow(22, 1, prompts[0], 0, sample=True, sampling=g, want_logprob=True, adapter=snap)], out_t)
    # the snapshot still decodes like the old policy (another batch position: within the reference's 1e-3, tests/lora_rows.rs:34-37)
    assert out_t.row(1).token == before[0] and abs(out_t.row(1).logprob - before[1]) < 1e-3
    assert abs(out_t.row(0).logprob - before[1]) > 1e-3                   # the live policy moved
    trainer.weights_updated()                        # a weight import without a file: forget and bump
    assert trainer.weights_version() == v + 2
    snap2 = trainer.adapter_snapshot(replace=snap)
    assert snap2 != snap and trainer.adapter_rows_info()["n_adapters"] == 1
    trainer.request_free(21)
    assert trainer.generation_stats()["calls"] == 0
    trainer.close()
    engine.close()
    lib = rb.load_library()
    assert lib.retro_trainer_generation_seq_rm(None, 0, -1, -1) == -1 and lib.retro_last_error() == b"trainer handle is null"


def test_counters_memory_report_and_generation_stats(rb, c1_model):
    engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=2048, n_seq_max=8, n_batch=256, n_ubatch=256))
    rep = engine.memory_report()
    assert rep["has_generation_context"] and rep["optimizer_state_bytes"] == 0 and rep["trainable_gradient_bytes"] == 0
    assert rep["model_weight_bytes"] > 2_000_000 and rep["generation_kv_bytes"] == engine.memory().kv_bytes
    assert rep["device_bytes"] == rep["model_weight_bytes"] + rep["generation_kv_bytes"] + rep["generation_compute_bytes"] + rep["trainable_parameter_bytes"]
    assert rep["device_memory_samples"] == 1 and rep["device_total_bytes"] > rep["device_used_bytes"] >= rep["device_bytes"] // 2
    assert engine.generation_stats() == dict(calls=0, sequences=0, prompt_tokens=0, prefilled_tokens=0, reused_tokens=0, hits=0, evictions=0)
    greedy = rb.SamplingParams(temperature=1e-4, top_p=1e-6, max_new_tokens=3)
    prompt = _prompt(5, 40, 4096)
    engine.generate_batch(prompt, [greedy] * 4, n_out_max=4)
    st = engine.generation_stats()
    # the prompt is decoded once (39 tokens into slot 0) and attached to three more sequences; every member then
    # decodes the last prompt token itself
    assert st == dict(calls=1, sequences=4, prompt_tokens=160, prefilled_tokens=39 + 4, reused_tokens=3 * 39, hits=3, evictions=0)
    engine.generate_continuous([(prompt[:10], greedy), (prompt[:7], greedy)], n_out_max=4)
    st = engine.generation_stats()
    assert st["calls"] == 2 and st["sequences"] == 6 and st["prompt_tokens"] == 177 and st["prefilled_tokens"] == 43 + 17 and st["hits"] == 3
    engine.close()


def test_shared_prompt_generator_on_a_partitioned_pool(rb, c1_model):
    """kv_unified = 0 only takes whole-sequence copies: the shared prompt must still reach every member."""
    greedy = rb.SamplingParams(temperature=1e-4, top_p=1e-6, max_new_tokens=5)
    prompt = _prompt(6, 23, 4096)
    results = []
    for unified in (1, 0):
        engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=2048, n_seq_max=4, n_batch=128, n_ubatch=128, kv_unified=unified))
        assert engine.kv_unified() == bool(unified)
        results.append(engine.generate_batch(prompt, [greedy] * 3, n_out_max=6))
        engine.close()
    (tok_u, lp_u), (tok_p, lp_p) = results
    assert tok_u == tok_p and lp_u == lp_p and len(tok_p) == 3 and all(1 <= len(t) <= 5 for t in tok_p)


def test_end_of_generation_is_more_than_eos(rb, models):
    """retro_gen_core.cpp:1168, retro_engine.cpp:665 stop on the vocabulary's end-of-generation set: EOS, the
    end-of-turn id the file names, and control pieces spelled like a turn end."""
    spec = dict(arch="llama", layers=1, d=256, heads=4, kv_heads=4, ff=512, vocab=512, dtype="q8_0", seed=9, eot=300, turn_end=301)
    engine = rb.Engine(str(models("eog", **spec)), rb.EngineConfig(n_ctx=512, n_seq_max=2, n_batch=64, n_ubatch=64))
    assert engine.eos_token() == 2
    assert [engine.is_eog_token(t) for t in (2, 300, 301, 302, 5)] == [True, True, True, False, False]
    lib = rb.load_library()
    flag = C.c_bool()
    assert lib.retro_engine_is_eog_token(engine._h, 9999, C.byref(flag)) == -1
    engine.close()


def test_expert_bank_inventory_stats_and_route_paths(rb, models):
    spec = dict(arch="olmoe", layers=2, d=256, heads=4, kv_heads=4, ff=128, vocab=512, experts=8, experts_used=2, dtype="f16", expert_dtype="mxfp4", seed=21)
    engine = rb.Engine(str(models("moe_banks", **spec)), rb.EngineConfig(n_ctx=512, n_seq_max=4, n_batch=64, n_ubatch=64))
    banks = engine.expert_banks()
    assert [b["name"] for b in banks] == sorted(f"blk.{l}.ffn_{r}_exps.weight" for l in range(2) for r in ("down", "gate", "up"))
    gate0 = next(b for b in banks if b["name"] == "blk.0.ffn_gate_exps.weight")
    assert gate0["layer"] == 0 and gate0["role"] == "gate" and gate0["ne"] == [256, 128, 8, 1] and gate0["type_name"] == "MXFP4"
    assert gate0["n_elements"] == 256 * 128 * 8 and gate0["n_bytes"] == 256 * 128 * 8 // 32 * 17
    down1 = next(b for b in banks if b["name"] == "blk.1.ffn_down_exps.weight")
    assert down1["layer"] == 1 and down1["role"] == "down" and down1["ne"] == [128, 256, 8, 1]
    lib = rb.load_library()
    n = C.c_size_t()
    from retrograd_b200 import _ffi

    short = (_ffi.ExpertBankDescC * 2)()
    assert lib.retro_engine_expert_banks(engine._h, short, 2, C.byref(n)) == -2 and n.value == 6
    st = engine.expert_stats()
    assert st.n_groups == 0 and st.small.hits == st.large.misses == st.copy.bytes == 0
    assert engine.expert_route_paths() == (0, 0, 0)
    engine.expert_route_enable(1)
    out = rb.StepOutput()
    engine.step([rb.StepRow(0, 0, _prompt(3, 11), 0, sample=True, sampling=rb.SamplingParamsV2.greedy())], out)
    assert engine.expert_route_paths() == (2 * 11 * 2, 0, 0)        # layers x tokens x experts per token, all from resident banks
    engine.close()
    dense = rb.Engine(str(models("eog", arch="llama", layers=1, d=256, heads=4, kv_heads=4, ff=512, vocab=512, dtype="q8_0", seed=9, eot=300, turn_end=301)),
                      rb.EngineConfig(n_ctx=512, n_seq_max=2, n_batch=64, n_ubatch=64))
    assert dense.expert_banks() == []
    dense.close()
