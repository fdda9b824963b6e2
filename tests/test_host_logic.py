"""Host-side logic that needs no GPU: the C-ABI surface, config validation, the KV bookkeeping."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(rb):
    header = (ROOT / "include" / "retro_b200.h").read_text()
    declared = set(re.findall(r"\b(retro_(?:b200_)?[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 42
    lib = rb.load_library()
    from retrograd_b200 import _ffi

    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _ffi.SYMBOLS, f"{name} has no ctypes binding"


def test_library_exports_the_reference_bindings_step_path_symbols(rb):
    """`nm -D` of the built library against the committed list of names the reference's `extern "C"` block
    declares for this path: a missing one would keep the reference's crate from linking."""
    wanted = [l.strip() for l in (ROOT / "tests" / "golden" / "abi_symbols.txt").read_text().splitlines() if l.strip() and not l.startswith("#")]
    assert len(wanted) >= 60
    out = subprocess.run(["nm", "-D", "--defined-only", str(rb.LIB_PATH)], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    missing = [name for name in wanted if name not in exported]
    assert not missing, f"not exported: {missing}"


def test_grammar_handles_own_their_text(rb):
    """retro_grammar.cpp:1-76: an owned GBNF string; empty text and a null handle are refused with a message."""
    lib = rb.load_library()
    g = lib.retro_grammar_from_gbnf(b'root ::= "a" | "b"')
    assert g and lib.retro_grammar_gbnf(g) == b'root ::= "a" | "b"'
    lib.retro_grammar_free(g)
    assert not lib.retro_grammar_from_gbnf(b"") and lib.retro_last_error() == b"gbnf is required and must not be empty"
    assert not lib.retro_grammar_from_gbnf(None)
    assert lib.retro_grammar_gbnf(None) is None and lib.retro_last_error() == b"grammar is null"
    j = lib.retro_grammar_json_object()
    assert j and lib.retro_grammar_gbnf(j).startswith(b"root ::= object")
    lib.retro_grammar_free(j)
    assert not lib.retro_grammar_from_json_schema(b"") and lib.retro_last_error() == b"json_schema is required and must not be empty"
    assert not lib.retro_grammar_from_json_schema(b'{"type": "object"}') and b"pass GBNF" in lib.retro_last_error()
    lib.retro_grammar_free(None)


def test_struct_layouts_match_the_published_header(rb):
    """Sizes pinned by crates/retrograd-ffi/src/lib.rs:2899-3052."""
    from retrograd_b200 import _ffi as F

    assert C.sizeof(F.EngineConfigC) == 64 and F.EngineConfigC.kv_unified.offset == 40 and F.EngineConfigC.expert_device_cache_bytes.offset == 56
    assert C.sizeof(F.SamplingParamsC) == 16
    assert C.sizeof(F.StepRowC) == 64 and F.StepRowC.sampling.offset == 36 and F.StepRowC.adapter.offset == 56
    assert C.sizeof(F.StepOutRowC) == 20 and F.StepOutRowC.sampled.offset == 17
    assert C.sizeof(F.SamplingParamsV2C) == 72 and F.SamplingParamsV2C.grammar.offset == 64
    assert C.sizeof(F.StepRowV2C) == 128 and F.StepRowV2C.sampling.offset == 40 and F.StepRowV2C.adapter.offset == 120
    assert C.sizeof(F.StepOutRowV2C) == 24 and F.StepOutRowV2C.sampled_logprob.offset == 20
    assert C.sizeof(F.MemoryInfoC) == 40
    assert C.sizeof(F.AdapterRowsInfoC) == 32
    # lib.rs:2958-2969 (memory report), retro_lora_train.h:788-795, 827-840, 1113-1131
    assert C.sizeof(F.MemoryReportC) == 216 and F.MemoryReportC.trainable_parameter_bytes.offset == 48
    assert F.MemoryReportC.base_trainable_on_host.offset == 74 and F.MemoryReportC.device_bytes.offset == 80
    assert F.MemoryReportC.device_memory_samples.offset == 136
    assert C.sizeof(F.GenerationStatsC) == 56
    assert C.sizeof(F.ExpertBankDescC) == 272 and F.ExpertBankDescC.role.offset == 4 and F.ExpertBankDescC.tensor.offset == 24
    assert C.sizeof(F.ExpertCacheStatsC) == 464 and F.ExpertCacheStatsC.n_groups.offset == 72 and F.ExpertCacheStatsC.groups.offset == 80


def _new(rb, path, **over):
    cfg = rb.EngineConfig(**over).to_c()
    lib = rb.load_library()
    h = lib.retro_engine_new(path, C.byref(cfg))
    return h, (lib.retro_last_error() or b"").decode()


def test_engine_config_is_validated_before_anything_loads(rb):
    """Messages of crates/retrograd-ffi/runtime/src/retro_engine.cpp:112-153,469-483."""
    lib = rb.load_library()
    assert not lib.retro_engine_new(None, None)
    assert lib.retro_last_error().decode() == "model_path is required"
    h, msg = _new(rb, b"/nonexistent.gguf", n_ctx=0)
    assert not h and msg == "engine n_ctx and n_seq_max must be greater than zero"
    h, msg = _new(rb, b"/nonexistent.gguf", n_ubatch=1024, n_batch=512)
    assert not h and msg == "engine n_ubatch must be in (0, n_batch]"
    h, msg = _new(rb, b"/nonexistent.gguf", n_seq_max=600, n_batch=512)
    assert not h and msg == "engine n_seq_max must not exceed LLAMA_MAX_SEQ, n_batch or n_ctx"
    h, msg = _new(rb, b"/nonexistent.gguf", kv_dtype=9)
    assert not h and msg == "engine kv_dtype must be one of retro_engine_kv_dtype"
    h, msg = _new(rb, b"/nonexistent.gguf", kv_dtype=2, flash_attn=False)
    assert not h and msg == "a quantized engine kv_dtype requires flash_attn"
    h, msg = _new(rb, b"/nonexistent.gguf", device=7)
    assert not h and msg == "engine device must be one of retro_device"
    # the pool is F16, Q8_0 or Q4_0 here; the reference's fourth type is refused in words before anything loads
    h, msg = _new(rb, b"/nonexistent.gguf", kv_dtype=0)
    assert not h and msg == "this backend stores the KV cache as F16, Q8_0 or Q4_0: engine kv_dtype F32 is not supported"
    cfg = rb.EngineConfig().to_c()
    cfg.struct_size = 8
    assert not lib.retro_engine_new(b"/nonexistent.gguf", C.byref(cfg))
    assert lib.retro_last_error().decode() == "retro_engine_config.struct_size is too small for this build"


def test_there_is_no_cpu_path(rb, c1_model):
    """device=cpu is refused, and without a CUDA device the constructor fails loudly."""
    h, msg = _new(rb, str(c1_model).encode(), device=1)
    assert not h and "only runs on a CUDA GPU" in msg
    import torch

    if not torch.cuda.is_available():
        with pytest.raises(rb.EngineError):
            rb.Engine(str(c1_model))


def test_null_handles_are_refused(rb):
    lib = rb.load_library()
    v = C.c_uint32()
    assert lib.retro_engine_vocab_size(None, C.byref(v)) == -1
    assert lib.retro_last_error().decode() == "engine handle is null"
    lib.retro_engine_free(None)


def test_synth_rejects_unknown_keys(rb, tmp_path):
    with pytest.raises(rb.EngineError):
        rb.synth_gguf(tmp_path / "x.gguf", bogus=1)


def test_synth_models_are_deterministic_and_readable(rb, tmp_path, oracle):
    a, b = tmp_path / "a.gguf", tmp_path / "b.gguf"
    spec = dict(arch="llama", layers=1, d=256, heads=4, kv_heads=2, ff=512, vocab=512, dtype="q4_k", seed=5)
    rb.synth_gguf(a, **spec)
    rb.synth_gguf(b, **spec)
    assert a.read_bytes() == b.read_bytes()
    rb.synth_gguf(b, **{**spec, "seed": 6})
    assert a.read_bytes() != b.read_bytes()
    m = oracle.Model(str(a))
    assert (m.n_layer, m.d, m.n_head, m.n_head_kv, m.head_dim, m.ff, m.vocab) == (1, 256, 4, 2, 64, 512, 512)


def test_the_oracle_folders_model_writer_gives_the_same_bytes(rb, oracle, tmp_path):
    """The benchmark's CPU arm writes its model without loading the GPU library; both arms must run the same file."""
    for i, spec in enumerate((dict(arch="llama", layers=1, d=256, heads=4, kv_heads=2, ff=512, vocab=512, dtype="q4_k", seed=5),
                              dict(arch="olmoe", layers=1, d=256, heads=4, kv_heads=4, ff=128, vocab=512, experts=8, experts_used=2, dtype="q8_0",
                                   expert_dtype="mxfp4", seed=21))):
        a, b = tmp_path / f"a{i}.gguf", tmp_path / f"b{i}.gguf"
        rb.synth_gguf(a, **spec)
        oracle.synth_gguf(b, **spec)
        assert a.read_bytes() == b.read_bytes()
    assert oracle.threads(2) == 2 and oracle.threads() == 2


@pytest.mark.parametrize("ggml_type,rel", [(8, 0.01), (12, 0.12), (39, 0.3)])
def test_encoders_round_trip_within_their_step(rb, oracle, ggml_type, rel):
    import numpy as np

    x = np.random.default_rng(ggml_type).normal(0, 0.02, 1024).astype(np.float32)
    raw = rb.quantize_row(ggml_type, x)
    y = oracle.dequantize_row(ggml_type, raw, x.size)
    assert np.abs(x - y).max() <= rel * np.abs(x).max()


def test_kv_bookkeeping(tmp_path):
    exe = tmp_path / "kv_manager_test"
    subprocess.run(["g++", "-std=c++17", "-O1", "-o", str(exe), str(ROOT / "tests" / "cpp" / "kv_manager_test.cpp")], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr


def test_mxfp4_expert_blocks_recode_exactly_as_q8_0(rb, oracle):
    """The engine holds MXFP4 expert banks as Q8_0 for the tensor cores: the doubled E2M1 value as the int8,
    half the E8M0 scale as the f16 d. Every value must decode to the same f32; a scale an f16 cannot hold
    (below 2^-24 or above 2^15) refuses the whole tensor."""
    rng = np.random.default_rng(17)
    n_blocks = 4096
    blocks = rng.integers(0, 256, (n_blocks, 17), dtype=np.uint8)
    blocks[:, 0] = rng.integers(104, 144, n_blocks)          # scales 2^-24 .. 2^15 after halving, subnormal f16 included
    blocks[:40, 0] = np.arange(104, 144)                       # every admissible scale at least once
    raw = blocks.tobytes()
    recoded = rb.recode_mxfp4_as_q8_0(raw)
    assert recoded is not None and len(recoded) == n_blocks * 34
    want = oracle.dequantize_row(oracle.T_MXFP4, raw, n_blocks * 32)
    got = oracle.dequantize_row(oracle.T_Q8_0, recoded, n_blocks * 32)
    assert np.array_equal(want, got)
    for bad in (0, 1, 103, 144, 255):
        blocks[7, 0] = bad
        assert rb.recode_mxfp4_as_q8_0(blocks.tobytes()) is None
