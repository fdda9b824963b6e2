"""Runs one kernel of the decode step in isolation on seeded random data, for timing and for
profiler captures of a small case.

    python -m retrograd_b200.kernel_cases gemm --n-out 28672 --n-in 4096 --tokens 2048 --path 3 --iters 5

`--path`: 0 engine's choice, 1 f32 row kernel, 2 single-term f16 tensor-core kernel, 3 exact
tensor-core kernel (mma.sync), 4 exact tcgen05 kernel, 5 exact weight-streaming kernel (at most 8 tokens).
Operands smaller than 256 MB are timed with a write of a buffer larger than L2 before every launch. Weights are random Q4_K blocks (scales pinned to small f16 values), the
activations N(0, 1). `--type q8_0` runs the Q8_0 kernels (paths 1 and 5). Prints the mean device time per launch and the rates derived from it.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import op_gemm


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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm"])
    ap.add_argument("--n-out", type=int, default=28672)
    ap.add_argument("--n-in", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--path", type=int, default=0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--type", default="q4_k", choices=["q4_k", "q8_0"])
    args = ap.parse_args()
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
