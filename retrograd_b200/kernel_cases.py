"""Runs one kernel of the decode step in isolation on seeded random data, for timing and for
profiler captures of a small case.

    python -m retrograd_b200.kernel_cases gemm --n-out 28672 --n-in 4096 --tokens 2048 --path 3 --iters 5

    python -m retrograd_b200.kernel_cases attention --mode decode --seqs 256 --ctx 1024 --iters 4

    python -m retrograd_b200.kernel_cases moe --experts 32 --n-out 2880 --n-in 2880 --tokens 2048 --iters 5

`--path`: 0 engine's choice, 1 f32 row kernel, 3 exact
tensor-core kernel (mma.sync), 4 exact tcgen05 kernel, 5 exact weight-streaming kernel (at most 8 tokens).
Operands smaller than 256 MB are timed with a write of a buffer larger than L2 before every launch. Weights are random Q4_K blocks (scales pinned to small f16 values), the
activations N(0, 1). `--type q8_0` runs the Q8_0 kernels (paths 1, 3, 4 and 5). Prints the mean device time per launch and the rates derived from it.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import op_gemm, op_gemm_mxfp4_grouped


def random_q4k(rng: np.random.Generator, n_out: int, n_in: int) -> np.ndarray:
    blocks = n_out * n_in // 256
    raw = rng.integers(0, 256, (blocks, 144), dtype=np.uint8)
    raw[:, 0:2] = np.frombuffer(np.float16(2.0 ** -9).tobytes(), dtype=np.uint8)
    raw[:, 2:4] = np.frombuffer(np.float16(2.0 ** -7).tobytes(), dtype=np.uint8)
    return raw.reshape(-1)


def random_q8_0(rng: np.random.Generator, n_out: int, n_in: int) -> np.ndarray:
    blocks = n_out * n_in // 32
    raw = rng.integers(0, 256, (blocks, 34), dtype=np.uint8)
    raw[:, 0:2] = np.frombuffer(np.float16(2.0 ** -9).tobytes(), dtype=np.uint8)
    return raw.reshape(-1)


def random_mxfp4(rng: np.random.Generator, n_rows: int, n_in: int) -> np.ndarray:
    blocks = n_rows * n_in // 32
    raw = rng.integers(0, 256, (blocks, 17), dtype=np.uint8)
    raw[:, 0] = rng.integers(116, 124, blocks, dtype=np.uint8)       # block scales 2^-11 .. 2^-4
    return raw.reshape(-1)


def moe_case(args) -> None:
    """The grouped MXFP4 expert GEMM alone: `--experts` banks of n_out x n_in, `--tokens` (token, expert) pairs spread
    over the experts as a routed step would (multinomial with unequal shares)."""
    rng = np.random.default_rng(args.seed)
    banks = random_mxfp4(rng, args.experts * args.n_out, args.n_in)
    shares = rng.dirichlet(np.full(args.experts, 4.0))
    counts = rng.multinomial(args.tokens, shares)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    x = rng.normal(0, 1, (args.tokens, args.n_in)).astype(np.float32)
    _, ms = op_gemm_mxfp4_grouped(banks, args.experts, args.n_out, args.n_in, x, offsets, iters=args.iters)
    flops = 2.0 * args.tokens * args.n_in * args.n_out
    weight_bytes = args.experts * args.n_out * args.n_in * 17 // 32
    print(json.dumps({
        "kernel": "gemm_mxfp4_grouped", "experts": args.experts, "n_out": args.n_out, "n_in": args.n_in, "pairs": args.tokens,
        "pairs_per_expert": [int(c) for c in counts], "ms_per_launch": ms, "tflops": flops / ms / 1e9, "weight_gbs": weight_bytes / ms / 1e6,
    }))


def attention_case(args) -> None:
    """The attention kernels at the 8B shape (32 query / 8 KV heads of 128) inside a ONE-layer model, so the
    whole case holds well under 2 GB on the device: `--seqs` sequences are prefilled to `--ctx` tokens
    through the normal step path, then `--iters` measured steps run and the attention class's device time
    per step is reported with the K/V bytes those steps had to read."""
    import os
    import tempfile

    from . import Engine, EngineConfig, SamplingParamsV2, StepOutput, StepRow, synth_gguf

    path = os.path.join(tempfile.gettempdir(), "retrograd_b200_attention_case.gguf")
    synth_gguf(path, arch="llama", layers=1, d=4096, heads=32, kv_heads=8, ff=1024, vocab=1024, dtype="q4_k", seed=5)
    n_ctx = args.seqs * (args.ctx + 1024 + 64)
    kv_code = {"f16": 1, "q8_0": 2, "q4_0": 3}[args.kv_dtype]
    engine = Engine(path, EngineConfig(n_ctx=n_ctx, n_seq_max=args.seqs, n_batch=2048, n_ubatch=2048, kv_dtype=kv_code))
    out = StepOutput(2048, 0)
    rng = np.random.default_rng(args.seed)
    greedy = SamplingParamsV2.greedy()
    pos = [0] * args.seqs
    # prefill in steps of up to four 512-token chunks
    pending = [(s, args.ctx) for s in range(args.seqs)]
    while pending:
        rows, rest = [], []
        for s, left in pending:
            if len(rows) < 4:
                take = min(512, left)
                rows.append(StepRow(s, s, rng.integers(3, 1024, take).tolist(), pos[s], False))
                pos[s] += take
                if left > take:
                    rest.append((s, left - take))
            else:
                rest.append((s, left))
        engine.step(rows, out)
        pending = rest
    kv_tok_bytes = 2 * 8 * 128 * {"f16": 2.0, "q8_0": 34 / 32, "q4_0": 18 / 32}[args.kv_dtype]          # one layer
    engine.profile(True, reset=True)
    kv_bytes = 0
    for it in range(args.iters):
        if args.mode == "decode":
            rows = [StepRow(s, s, [int(rng.integers(3, 1024))], pos[s], True, greedy) for s in range(args.seqs)]
            for s in range(args.seqs):
                pos[s] += 1
                kv_bytes += pos[s] * kv_tok_bytes
        else:
            rows = []
            for s in (2 * it % args.seqs, (2 * it + 1) % args.seqs):
                rows.append(StepRow(s, s, rng.integers(3, 1024, 512).tolist(), pos[s], False))
                pos[s] += 512
                kv_bytes += pos[s] * kv_tok_bytes
        engine.step(rows, out)
    prof = engine.profile_read()
    ms = prof["attention"]["ms"] / args.iters
    print(json.dumps({
        "kernel": "attention", "mode": args.mode, "kv_dtype": args.kv_dtype, "seqs": args.seqs, "ctx": args.ctx, "ms_per_step": ms,
        "kv_gb_per_step": kv_bytes / args.iters / 1e9, "kv_gbs": kv_bytes / args.iters / ms / 1e6,
        "launches_per_step": prof["attention"]["launches"] / args.iters,
    }))
    engine.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attention", "moe"])
    ap.add_argument("--experts", type=int, default=32, help="moe: expert banks")
    ap.add_argument("--seqs", type=int, default=64, help="attention: sequences resident")
    ap.add_argument("--ctx", type=int, default=2048, help="attention: tokens resident per sequence before the measured steps")
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill"],
                    help="attention: measured steps are one-token rows of every sequence, or 512-token chunks of two sequences")
    ap.add_argument("--kv-dtype", default="f16", choices=["f16", "q8_0", "q4_0"], help="attention: storage type of the KV pool")
    ap.add_argument("--n-out", type=int, default=28672)
    ap.add_argument("--n-in", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--path", type=int, default=0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--type", default="q4_k", choices=["q4_k", "q8_0"])
    args = ap.parse_args()
    if args.kernel == "attention":
        attention_case(args)
        return
    if args.kernel == "moe":
        moe_case(args)
        return
    rng = np.random.default_rng(args.seed)
    w = random_q4k(rng, args.n_out, args.n_in) if args.type == "q4_k" else random_q8_0(rng, args.n_out, args.n_in)
    ggml_type, bytes_per_block, block = (12, 144, 256) if args.type == "q4_k" else (8, 34, 32)
    x = rng.normal(0, 1, (args.tokens, args.n_in)).astype(np.float32)
    _, ms = op_gemm(ggml_type, w, args.n_out, args.n_in, x, path=args.path, iters=args.iters)
    flops = 2.0 * args.tokens * args.n_in * args.n_out
    weight_bytes = args.n_out * args.n_in * bytes_per_block // block
    print(json.dumps({
        "kernel": "gemm_" + args.type, "path": args.path, "n_out": args.n_out, "n_in": args.n_in, "tokens": args.tokens,
        "ms_per_launch": ms, "tflops": flops / ms / 1e9, "weight_gbs": weight_bytes / ms / 1e6,
    }))


if __name__ == "__main__":
    main()
