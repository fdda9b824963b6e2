"""Writes tests/golden/c1_greedy_tokens.json: the greedy token streams of the CPU oracle on the tiny CPU-runnable
workload (seeded llama-style Q8_0 model of 2 layers, d 256; 8 requests = a shared 32-token prefix + 16..128 unique
tokens; 32 new tokens each), over an F16 and over a Q8_0 KV cache, with the smallest top-2 logit margin the oracle met.
No GPU needed:

    python tests/golden/make_c1_tokens.py

The GPU test and the benchmark's `golden_check` replay the same requests through the engine and compare the streams
bit for bit with this file (they read the file, not the oracle)."""
import json
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import oracle as O  # noqa: E402

SPEC = dict(arch="llama", layers=2, d=256, heads=4, kv_heads=4, ff=688, vocab=4096, dtype="q8_0", seed=20261125)
SEED, N_REQUESTS, N_NEW = 37, 8, 32          # the seed with the widest smallest margin among 31..44
SEED_KV_Q8_0 = 59                            # the same choice for the Q8_0 cache, among 31..60


def prompts(seed: int = SEED):
    rng = np.random.default_rng(seed)
    prefix = rng.integers(3, 4096, 32).tolist()
    return [prefix + rng.integers(3, 4096, int(rng.integers(16, 129))).tolist() for _ in range(N_REQUESTS)]


def run(model_path: Path, kv_dtype: int, seed: int = SEED):
    """The oracle's greedy streams over a cache of `kv_dtype` (retro_engine_kv_dtype: 1 F16, 2 Q8_0) and the smallest
    top-2 logit margin it met."""
    ctx = O.Context(O.Model(str(model_path)), N_REQUESTS, 4096, kv_dtype=kv_dtype)
    ps = prompts(seed)
    streams = [[] for _ in ps]
    margin = float("inf")
    rows = [(i, list(p), 0, True, 0) for i, p in enumerate(ps)]
    for step in range(N_NEW):
        logits = ctx.step(rows)
        nxt = []
        for i, row in enumerate(logits):
            order = np.argsort(-row, kind="stable")
            margin = min(margin, float(row[order[0]] - row[order[1]]))
            tok = int(order[0])
            streams[i].append(tok)
            nxt.append((i, [tok], len(ps[i]) + step, True, 0))
        rows = nxt
    return streams, margin


def main() -> None:
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "c1.gguf"
        O.synth_gguf(path, **SPEC)
        streams, margin = run(path, 1)
        q8_streams, q8_margin = run(path, 2, SEED_KV_Q8_0)
    out = {"spec": SPEC, "prompt_seed": SEED, "n_requests": N_REQUESTS, "n_new": N_NEW, "min_top2_margin": margin, "streams": streams,
           # the same requests over a Q8_0 KV pool (engine kv_dtype 2)
           "kv_q8_0": {"prompt_seed": SEED_KV_Q8_0, "min_top2_margin": q8_margin, "streams": q8_streams}}
    (Path(__file__).resolve().parent / "c1_greedy_tokens.json").write_text(json.dumps(out) + "\n")
    print(f"wrote {N_REQUESTS} streams of {N_NEW} tokens; smallest top-2 margin {margin:.4f} (F16 cache), {q8_margin:.4f} (Q8_0 cache)")


if __name__ == "__main__":
    main()
