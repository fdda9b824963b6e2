"""Golden files produced by the reference's own fixture generators (tests/golden/make_golden.py).

The digests below are the ones the reference pins in tests/fixtures/TINY_FIXTURE.toml,
TINY_F16_FIXTURE.toml, TINY_Q8_FIXTURE.toml and TINY_MOE_FIXTURE.toml.
"""
import hashlib
import json

import numpy as np
import pytest

from conftest import GOLDEN

PINNED = {
    "retrograd-tiny-qwen2-f32.gguf": ("218570a8f7793864c8c1b4a6eb6d132c5ecff9e2432b8c0b41270a6901971f07", 737952),
    "retrograd-tiny-qwen2-f16.gguf": ("f2abf21a1f4ffd7fe6cf433d2186027f3be9b7469c8cd0e3f8fa50dced4cf052", 376480),
    "retrograd-tiny-qwen2-q8_0.gguf": ("f48a0e831ab1c16b07aa98b645205fb08e5c390ada539fa36052fc9e93463890", 207072),
    "retrograd-tiny-olmoe-f32.gguf": ("951939411c8fcfb8ededc826c4dd558674f04abfb9d751b53c62033436957a03", 1065440),
}


@pytest.mark.parametrize("name", sorted(PINNED))
def test_golden_files_carry_the_reference_digests(name):
    data = (GOLDEN / name).read_bytes()
    assert (hashlib.sha256(data).hexdigest(), len(data)) == PINNED[name]
    recorded = json.loads((GOLDEN / "fixtures.json").read_text())[name]
    assert recorded["sha256"] == PINNED[name][0]


def test_oracle_reads_the_reference_fixtures(oracle):
    m = oracle.Model(str(GOLDEN / "retrograd-tiny-qwen2-q8_0.gguf"))
    assert (m.n_layer, m.d, m.n_head, m.n_head_kv, m.head_dim, m.ff, m.vocab, m.neox) == (4, 64, 4, 2, 16, 128, 260, 1)
    moe = oracle.Model(str(GOLDEN / "retrograd-tiny-olmoe-f32.gguf"))
    assert (moe.n_layer, moe.d, moe.n_head, moe.n_head_kv, moe.ff, moe.n_expert, moe.n_expert_used) == (2, 64, 4, 4, 64, 8, 2)


def test_q8_0_encoder_reproduces_the_reference_file(rb):
    """The F32 and Q8_0 fixtures hold the same numbers at two precisions
    (tests/fixtures/TINY_Q8_FIXTURE.toml): encoding the F32 tensors with this project's Q8_0
    encoder must give the reference's bytes (scripts/gen-tiny-fixture.py:173-198)."""
    gguf = pytest.importorskip("gguf")
    f32 = {t.name: t for t in gguf.GGUFReader(str(GOLDEN / "retrograd-tiny-qwen2-f32.gguf")).tensors}
    q8 = {t.name: t for t in gguf.GGUFReader(str(GOLDEN / "retrograd-tiny-qwen2-q8_0.gguf")).tensors}
    checked = 0
    for name, t in q8.items():
        if t.tensor_type.name != "Q8_0":
            continue
        values = np.asarray(f32[name].data, dtype=np.float32).reshape(-1)
        want = np.asarray(t.data, dtype=np.uint8).reshape(-1).tobytes()
        assert rb.quantize_row(8, values) == want, name
        checked += 1
    assert checked >= 4 * 7 + 2


def test_f16_fixture_decodes_to_the_f32_fixture(oracle):
    """Every weight was snapped to the F16 grid before storage, so both files decode to the same
    values (scripts/gen-tiny-fixture.py:159-170)."""
    gguf = pytest.importorskip("gguf")
    f32 = {t.name: t for t in gguf.GGUFReader(str(GOLDEN / "retrograd-tiny-qwen2-f32.gguf")).tensors}
    f16 = {t.name: t for t in gguf.GGUFReader(str(GOLDEN / "retrograd-tiny-qwen2-f16.gguf")).tensors}
    for name, t in f16.items():
        if t.tensor_type.name != "F16":
            continue
        raw = np.asarray(t.data).view(np.uint8).reshape(-1)
        got = oracle.dequantize_row(oracle.T_F16, raw, raw.size // 2)
        assert np.array_equal(got, np.asarray(f32[name].data, dtype=np.float32).reshape(-1)), name


def test_committed_greedy_streams_are_what_the_oracle_produces():
    """tests/golden/c1_greedy_tokens.json is the output of tests/golden/make_c1_tokens.py: regenerated here from the
    oracle and compared with the committed file."""
    import importlib.util
    import json
    import tempfile
    from pathlib import Path

    import numpy as np

    from oracle import oracle as O

    here = Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_c1_tokens", here / "make_c1_tokens.py")
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    golden = json.loads((here / "c1_greedy_tokens.json").read_text())
    assert golden["spec"] == mk.SPEC and golden["prompt_seed"] == mk.SEED and golden["min_top2_margin"] > 1e-3
    q8 = golden["kv_q8_0"]
    assert q8["prompt_seed"] == mk.SEED_KV_Q8_0 and q8["min_top2_margin"] > 1e-3
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "c1.gguf"
        O.synth_gguf(path, **mk.SPEC)
        ctx = O.Context(O.Model(str(path)), mk.N_REQUESTS, 4096)
        ps = mk.prompts()
        rows = [(i, list(p), 0, True, 0) for i, p in enumerate(ps)]
        streams = [[] for _ in ps]
        for step in range(mk.N_NEW):
            logits = ctx.step(rows)
            toks = [int(np.argsort(-row, kind="stable")[0]) for row in logits]
            for i, t in enumerate(toks):
                streams[i].append(t)
            rows = [(i, [t], len(ps[i]) + step, True, 0) for i, t in enumerate(toks)]
        q8_streams, q8_margin = mk.run(path, 2, mk.SEED_KV_Q8_0)
    assert streams == golden["streams"]
    # the streams over a Q8_0 cache: other prompts, and a cache that changes the tokens
    assert q8_streams == q8["streams"] and abs(q8_margin - q8["min_top2_margin"]) < 1e-6
