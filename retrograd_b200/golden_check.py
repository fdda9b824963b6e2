"""Replays the tiny CPU-runnable workload through the engine and compares its greedy token streams with the
streams the CPU oracle produced for the same requests (tests/golden/c1_greedy_tokens.json, written by
tests/golden/make_c1_tokens.py). Reads the committed file only: nothing of the oracle is loaded here."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent.parent / "tests" / "golden" / "c1_greedy_tokens.json"


def golden_prompts(golden: dict, seed: int | None = None) -> list[list[int]]:
    rng = np.random.default_rng(golden["prompt_seed"] if seed is None else seed)
    prefix = rng.integers(3, 4096, 32).tolist()
    return [prefix + rng.integers(3, 4096, int(rng.integers(16, 129))).tolist() for _ in range(golden["n_requests"])]


def replay(rb, model_path: str | None = None, kv: str = "f16") -> dict:
    """Returns {"workload", "tokens", "bit_exact", "first_mismatch"}; synthesises the model when no path is given.
    kv: "f16", or "q8_0" for the streams the oracle produced over a Q8_0 KV cache (their own prompts)."""
    golden = json.loads(GOLDEN.read_text())
    want_streams = golden["streams"] if kv == "f16" else golden["kv_" + kv]["streams"]
    prompts = golden_prompts(golden, None if kv == "f16" else golden["kv_" + kv]["prompt_seed"])
    kv_dtype = {"f16": rb.KV_DTYPE_F16, "q8_0": rb.KV_DTYPE_Q8_0}[kv]
    with tempfile.TemporaryDirectory() as tmp:
        if model_path is None:
            model_path = str(Path(tmp) / "c1.gguf")
            rb.synth_gguf(model_path, **golden["spec"])
        engine = rb.Engine(model_path, rb.EngineConfig(n_ctx=4096, n_seq_max=len(prompts), n_batch=1024, n_ubatch=1024, kv_dtype=kv_dtype))
        greedy = rb.SamplingParamsV2.greedy()
        out = rb.StepOutput(1024, 0)
        rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=greedy) for i, p in enumerate(prompts)]
        streams = [[] for _ in prompts]
        for step in range(golden["n_new"]):
            engine.step(rows, out)
            for i in range(len(prompts)):
                streams[i].append(out.row(i).token)
            rows = [rb.StepRow.decode(i, i, streams[i][-1], len(prompts[i]) + step, greedy) for i in range(len(prompts))]
        engine.close()
    mismatch = None
    for i, (got, want) in enumerate(zip(streams, want_streams)):
        for j, (a, b) in enumerate(zip(got, want)):
            if a != b and mismatch is None:
                mismatch = {"request": i, "position": j, "engine": a, "oracle": b}
    return {"workload": "tiny llama-style Q8_0 (2 layers, d 256), 8 requests with a shared 32-token prefix, 32 greedy tokens each",
            "tokens": sum(len(s) for s in streams), "bit_exact": mismatch is None, "first_mismatch": mismatch}
