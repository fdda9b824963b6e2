#!/usr/bin/env python3
"""Benchmark of the batched decode step: decode tokens/s on the Llama-3-8B-shape Q4_K ragged workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c2|c1]

One "step" is one scheduler step of continuous batching: every live request's decode row plus
chunked-prefill rows (512-token chunks) of newly admitted requests, through `retro_engine_step_v2`
of libretro_b200 with HOST buffers. Model weights and prompts are synthetic: a seeded random
8B-shape GGUF quantised to Q4_K, prompts of uniform-random token ids with log-uniform lengths
64..4096, output lengths uniform 64..512 (no data set is involved).

Printed keys beyond the base contract:
  value        decode tokens / device time of the K timed steps (CUDA events around each step's
               kernels; the few-KB plan is already in HBM when the timed region starts)
  e2e          the same tokens / wall time of the K `retro_engine_step_v2` calls, host plan in,
               sampled rows out (host<->device copies inside the timed region)
  roofline     the dominant kernel class of the timed region, timed live with CUDA events on the
               launching stream, against the measured peak of MEASURED_PEAKS.json
  cpu_baseline the CPU oracle timed on this host's cores on a bounded sample (N=1, rank 0)
  unprofiled   the K steps that follow the timed region, with the engine's profiler off (N=1): what a caller gets when
               no events separate the kernel classes - repeated step shapes replay as CUDA graphs

`--impl reference` times the reference's CPU path for the same metric. The reference itself cannot
be built in this image (no Rust toolchain, and its compute library is an un-vendored submodule), so
the arm runs the CPU restatement under oracle/ with every host thread on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # the headline workload: 8B-shape Q4_K, 256 concurrent ragged requests, 512-token prefill chunks
    "c2": dict(
        name="llama3-8b-shape Q4_K, 256 ragged requests, continuous batching, 512-token prefill chunks",
        spec=dict(arch="llama", layers=32, d=4096, heads=32, kv_heads=8, ff=14336, vocab=128256, dtype="q4_k", seed=2),
        n_requests=256, prompt=(64, 4096), output=(64, 512), chunk=512, n_batch=2048, n_ctx=420_000,
    ),
    # the same model with eight long-running requests: every timed step is a pure decode step of eight
    # tokens, the regime where the weight stream from HBM bounds the step
    "c2_decode8": dict(
        name="llama3-8b-shape Q4_K, 8 requests, decode-only steps of 8 tokens",
        model="c2",
        spec=dict(arch="llama", layers=32, d=4096, heads=32, kv_heads=8, ff=14336, vocab=128256, dtype="q4_k", seed=2),
        n_requests=8, prompt=(64, 512), output=(2048, 4096), chunk=512, n_batch=512, n_ctx=65536,
    ),
    "c2_decode16": dict(
        name="llama3-8b-shape Q4_K, 16 requests, decode-only steps of 16 tokens",
        model="c2",
        spec=dict(arch="llama", layers=32, d=4096, heads=32, kv_heads=8, ff=14336, vocab=128256, dtype="q4_k", seed=2),
        n_requests=16, prompt=(64, 512), output=(2048, 4096), chunk=512, n_batch=512, n_ctx=131072,
    ),
    # the 8B shape in Q8_0 (the rollout workload's weights), again eight long-running requests
    "c3_decode8": dict(
        name="llama3-8b-shape Q8_0, 8 requests, decode-only steps of 8 tokens",
        model="c3",
        spec=dict(arch="llama", layers=32, d=4096, heads=32, kv_heads=8, ff=14336, vocab=128256, dtype="q8_0", seed=3),
        n_requests=8, prompt=(64, 512), output=(2048, 4096), chunk=512, n_batch=512, n_ctx=65536,
    ),
    # the rollout workload: the 8B shape in Q8_0, 64 prompts each sampled as a group of 8 whose members share the
    # prompt's KV blocks (one prefill per group, then whole-sequence copies), temperature 1.0, top-p 1.0, seeded.
    # All 512 samples start together, as a rollout batch does: the timed steps are decode steps of 512 rows.
    "c3": dict(
        name="llama3-8b-shape Q8_0 rollout, 64 prompts x groups of 8 sharing the prompt KV, temperature 1.0 seeded",
        spec=dict(arch="llama", layers=32, d=4096, heads=32, kv_heads=8, ff=14336, vocab=128256, dtype="q8_0", seed=3),
        n_requests=512, group=8, prompt=(256, 1024), output=(512, 512), chunk=512, n_batch=2048, n_ctx=340_000, temperature=1.0,
    ),
    # multi-adapter decode: the Q4_K base with 16 rank-16 adapters (alpha 32) on all seven projections, 128
    # requests assigned to adapters by Zipf(1.1)
    "c4": dict(
        name="llama3-8b-shape Q4_K + 16 rank-16 LoRA adapters on q/k/v/o/gate/up/down, 128 requests assigned by Zipf(1.1)",
        model="c2",
        spec=dict(arch="llama", layers=32, d=4096, heads=32, kv_heads=8, ff=14336, vocab=128256, dtype="q4_k", seed=2),
        n_requests=128, prompt=(128, 2048), output=(256, 256), chunk=512, n_batch=2048, n_ctx=300_000,
        adapters=dict(n=16, rank=16, alpha=32.0, zipf=1.1),
    ),
    # the gpt-oss-20b-like MoE shape at its own size: 24 layers, 512 ragged requests
    "c5": dict(
        name="gpt-oss-20b-shape MoE (24 layers, 32 experts top-4, MXFP4 experts), 512 ragged requests per GPU",
        spec=dict(arch="olmoe", layers=24, d=2880, heads=64, kv_heads=8, head_dim=64, ff=2880, vocab=201088, experts=32, experts_used=4,
                  dtype="q8_0", expert_dtype="mxfp4", seed=5),
        n_requests=512, prompt=(64, 2048), output=(128, 512), chunk=512, n_batch=2048, n_ctx=720_000, ep=True,
    ),
    # the gpt-oss-20b-like MoE shape cut to 6 of its 24 layers (a full-depth model costs a quarter of an hour of
    # GPU time per run): experts MXFP4, the rest Q8_0. With more than one GPU the ranks form an expert-parallel
    # group: each serves 32 / N experts and its own requests.
    "c5_ep": dict(
        name="gpt-oss-20b-shape MoE cut to 6 layers (32 experts top-4, MXFP4), 128 requests per GPU, expert parallel",
        spec=dict(arch="olmoe", layers=6, d=2880, heads=64, kv_heads=8, head_dim=64, ff=2880, vocab=201088, experts=32, experts_used=4,
                  dtype="q8_0", expert_dtype="mxfp4", seed=5),
        n_requests=128, prompt=(64, 1024), output=(128, 512), chunk=512, n_batch=1024, n_ctx=200_000, ep=True,
    ),
    # the tiny CPU-runnable shape (used to exercise this script quickly)
    "c1": dict(
        name="tiny llama-style Q8_0, 8 requests",
        spec=dict(arch="llama", layers=2, d=256, heads=4, kv_heads=4, ff=688, vocab=4096, dtype="q8_0", seed=20261125),
        n_requests=8, prompt=(48, 160), output=(32, 64), chunk=64, n_batch=128, n_ctx=4096,
    ),
}


def gemm_step_bytes(sp, hd, w_elems_layer, tokens, sampled) -> float:
    """Algorithmic bytes of one step's weight GEMMs: every weight once, each GEMM's activations in (the hi + lo
    split, 4 bytes per element) and results out (f32), for the four projections of a layer and the head."""
    bpw = {"q4_k": 144 / 256, "q8_0": 34 / 32, "f16": 2.0, "f32": 4.0}.get(sp["dtype"], 1.0)
    dq, dkv = sp["heads"] * hd, sp["kv_heads"] * hd
    in_sum = sp["d"] + dq + sp["d"] + sp["ff"]
    out_sum = (dq + 2 * dkv) + sp["d"] + 2 * sp["ff"] + sp["d"]
    layer = w_elems_layer * bpw + tokens * 4 * (in_sum + out_sum)
    head = sp["d"] * sp["vocab"] * bpw + sampled * 4 * (sp["d"] + sp["vocab"])
    return sp["layers"] * layer + head


def model_path(workload: str) -> Path:
    base = Path(os.environ.get("RB200_MODEL_DIR", "/dev/shm" if Path("/dev/shm").is_dir() else "/tmp"))
    return base / f"retrograd_b200_{WORKLOADS[workload].get('model', workload)}.gguf"


def ensure_model(workload: str, rank: int, host_only: bool = False) -> Path:
    """The workload's seeded GGUF, written once per box. `host_only`: through the oracle folder's copy of the
    writer, so that the CPU arm never loads the GPU library (the two writers give the same bytes)."""
    path = model_path(workload)
    done = path.with_suffix(".done")
    if rank == 0 and not done.exists():
        if host_only:
            from oracle import oracle as O

            O.synth_gguf(path, **WORKLOADS[workload]["spec"])
        else:
            import retrograd_b200 as rb

            rb.synth_gguf(path, **WORKLOADS[workload]["spec"])
        done.write_text("ok")
    while not done.exists():
        time.sleep(0.5)
    return path


def write_adapter(path: Path, sp: dict, rank: int, alpha: float, seed: int) -> None:
    """A seeded LoRA adapter GGUF (general.type = adapter) with A [rank, in] and B [out, rank] ~ N(0, 0.02) on the
    seven projections of every layer, written with the gguf package of the image."""
    import gguf

    rng = np.random.default_rng(seed)
    hd = sp.get("head_dim") or sp["d"] // sp["heads"]
    d, dq, dkv, ff = sp["d"], sp["heads"] * hd, sp["kv_heads"] * hd, sp["ff"]
    shapes = {"attn_q": (d, dq), "attn_k": (d, dkv), "attn_v": (d, dkv), "attn_output": (dq, d), "ffn_gate": (d, ff), "ffn_up": (d, ff), "ffn_down": (ff, d)}
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_string("general.type", "adapter")
    w.add_string("adapter.type", "lora")
    w.add_float32("adapter.lora.alpha", float(alpha))
    for layer in range(sp["layers"]):
        for target, (n_in, n_out) in shapes.items():
            w.add_tensor(f"blk.{layer}.{target}.weight.lora_a", rng.standard_normal((rank, n_in), dtype=np.float32) * np.float32(0.02))
            w.add_tensor(f"blk.{layer}.{target}.weight.lora_b", rng.standard_normal((n_out, rank), dtype=np.float32) * np.float32(0.02))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


class Request:
    __slots__ = ("rid", "prompt", "n_out", "slot", "pos", "done", "last", "times", "adapter", "members", "waiting", "need", "sampling")

    def __init__(self, rid, prompt, n_out):
        self.rid, self.prompt, self.n_out = rid, prompt, n_out
        self.slot, self.pos, self.done, self.last, self.times = -1, 0, 0, None, []
        self.adapter = 0            # index into the loaded adapters + 1; 0 = none
        self.members = None         # a group leader's other members, until the prompt's blocks are shared with them
        self.waiting = False        # a group member whose leader is still prefilling the shared prompt
        self.need = len(prompt) + n_out
        self.sampling = None


class Workload:
    """Seeded open-loop request source: a new request is ready whenever a slot frees."""

    def __init__(self, cfg, seed):
        self.cfg = cfg
        self.rng = np.random.default_rng(seed)
        self.next_id = 0
        self.vocab = cfg["spec"]["vocab"]
        zipf = cfg.get("adapters")
        self.adapter_p = None
        if zipf:
            w = 1.0 / np.arange(1, zipf["n"] + 1) ** zipf["zipf"]
            self.adapter_p = w / w.sum()

    def request(self, midflight: bool = False) -> Request:
        lo, hi = self.cfg["prompt"]
        n_prompt = int(round(math.exp(self.rng.uniform(math.log(lo), math.log(hi)))))
        n_out = int(self.rng.integers(self.cfg["output"][0], self.cfg["output"][1] + 1))
        if midflight:
            # a request caught in the middle of its generation: the tokens it already produced
            # are part of what has to be resident
            produced = int(self.rng.integers(0, n_out))
            n_prompt += produced
            n_out -= produced
        prompt = self.rng.integers(3, self.vocab, n_prompt, dtype=np.int32)
        r = Request(self.next_id, prompt, max(n_out, 1))
        if self.adapter_p is not None:
            r.adapter = 1 + int(self.rng.choice(len(self.adapter_p), p=self.adapter_p))
        self.next_id += 1
        return r

    def group(self, size: int) -> list:
        """A prompt sampled `size` times: the leader carries the prompt, the members wait for its blocks."""
        leader = self.request()
        members = []
        for _ in range(size - 1):
            m = Request(self.next_id, leader.prompt, leader.n_out)
            m.waiting, m.need = True, leader.n_out
            self.next_id += 1
            members.append(m)
        leader.members = members
        return [leader] + members


class Driver:
    """Continuous batching as the reference's scheduler composes a step
    (crates/retrograd-infer/src/scheduler.rs:933-1089): decode rows first, then prefill chunks of
    at most `chunk` tokens per request while the step's token budget lasts."""

    def __init__(self, rb, engine, cfg, workload, sampling):
        self.rb, self.engine, self.cfg, self.wl, self.sampling = rb, engine, cfg, workload, sampling
        self.free_slots = list(range(cfg["n_requests"]))[::-1]
        self.live: list[Request] = []
        self.out = rb.StepOutput(cfg["n_batch"], 0)
        self.reserved = 0
        self.expert_parallel = False      # set when the engine joined an expert-parallel group: every rank steps in lock-step
        self.adapter_ids = []             # engine ids of the loaded adapters, in the order Request.adapter counts them

    def sampling_of(self, r):
        if self.cfg.get("temperature") is None:
            return self.sampling
        if r.sampling is None:
            r.sampling = self.rb.SamplingParamsV2(temperature=self.cfg["temperature"], top_p=1.0, seed=20261125 + r.rid)
        return r.sampling

    def admit(self, midflight=False):
        size = self.cfg.get("group")
        while size and len(self.free_slots) >= size:
            group = self.wl.group(size)
            need = sum(r.need for r in group)
            if self.reserved + need > self.cfg["n_ctx"]:
                break
            self.reserved += need
            for r in group:
                r.slot = self.free_slots.pop()
                self.live.append(r)
        if size:
            return
        while self.free_slots:
            r = self.wl.request(midflight)
            need = len(r.prompt) + r.n_out
            if self.reserved + need > self.cfg["n_ctx"]:
                break
            self.reserved += need
            r.slot = self.free_slots.pop()
            self.live.append(r)

    def compose(self, prefill_only=False, decode_only=0):
        """`decode_only` = n > 0: only the first n decoding requests' rows (the decode-only measurement)."""
        rb = self.rb
        rows, kinds, budget = [], [], self.cfg["n_batch"]
        for r in self.live:
            if prefill_only or (decode_only and len(rows) >= decode_only):
                break
            if r.last is not None and budget > 0:
                rows.append(rb.StepRow(r.rid, r.slot, [r.last], len(r.prompt) + r.done - 1, True, self.sampling_of(r), adapter=self.adapter_of(r)))
                kinds.append(r)
                budget -= 1
        for r in self.live:
            if r.last is None and budget > 0 and not decode_only and not r.waiting:
                # a group leader stops one token short: the last prompt token is every member's first own row
                end = len(r.prompt) - (1 if r.members else 0)
                take = min(budget, self.cfg["chunk"], end - r.pos)
                if take <= 0:
                    continue
                final = r.pos + take == len(r.prompt)
                rows.append(rb.StepRow(r.rid, r.slot, r.prompt[r.pos : r.pos + take], r.pos, final, self.sampling_of(r), adapter=self.adapter_of(r)))
                kinds.append(r)
                budget -= take
        return rows, kinds

    def adapter_of(self, r):
        return self.adapter_ids[r.adapter - 1] if r.adapter and self.adapter_ids else 0

    def share_prompts(self):
        """Group leaders whose prompt is resident but for its last token hand its blocks to their members."""
        for r in self.live:
            if r.members and r.pos == len(r.prompt) - 1:
                for m in r.members:
                    self.engine.seq_cp(r.slot, m.slot)
                    m.pos, m.waiting = r.pos, False
                r.members = None

    def step(self, prefill_only=False, decode_only=0):
        rows, reqs = self.compose(prefill_only, decode_only)
        if not rows:
            if self.expert_parallel:
                self.engine.ep_idle_step()      # this rank's experts still serve the other ranks' tokens
            return dict(decode=0, prefill=0, sampled=0, rows=rows, wall=0.0, tokens=0, ctx_tokens=0, finished=[])
        self.engine.step(rows, self.out)
        wall = self.engine.last_call_s
        stamp = time.perf_counter()
        n_decode = n_prefill = sampled = 0
        ctx_tokens = 0
        for i, (row, r) in enumerate(zip(rows, reqs)):
            n = len(row.tokens)
            if r.last is None:
                r.pos += n
                n_prefill += n
            else:
                n_decode += 1
            ctx_tokens += row.pos0 + n      # every resident KV entry of the row's sequence is read at least once
            if row.sample:
                r.last = self.out.row(i).token
                r.done += 1
                r.times.append(stamp)
                sampled += 1
        self.share_prompts()
        finished = [] if decode_only else [r for r in self.live if r.done >= r.n_out]
        for r in finished:
            self.engine.seq_rm(r.slot)
            self.engine.request_free(r.rid)
            self.free_slots.append(r.slot)
            self.reserved -= r.need
            self.live.remove(r)
        return dict(decode=n_decode, prefill=n_prefill, sampled=sampled, wall=wall, tokens=n_decode + n_prefill,
                    ctx_tokens=ctx_tokens, finished=finished, rows=rows)


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self):
        mhz = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        reasons = set()
        for s in self.samples:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        max_mhz = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(max_mhz) if max_mhz else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, "fallback"


def host_cores() -> int:
    """The host cores this process may run on (a launcher may have narrowed the affinity mask)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_baseline(path: Path, cfg, steps: int = 2, rows: int = 8, prompt: int = 4):
    """The CPU oracle (all host threads; activations re-quantised to 8-bit blocks and integer dot products, the
    arithmetic of the reference's CPU backend and the faster of the oracle's two modes) on a bounded sample: `rows`
    concurrent requests, a `prompt`-token prefill each, then `steps` decode steps."""
    from oracle import oracle as O

    cores = O.threads(host_cores())
    m = O.Model(str(path), fast=True, act_q8=True)
    ctx = O.Context(m, rows, 64)
    rng = np.random.default_rng(1)
    vocab = cfg["spec"]["vocab"]
    logits = ctx.step([(i, rng.integers(3, vocab, prompt).tolist(), 0, True) for i in range(rows)])
    times = []
    for s in range(steps):
        t0 = time.perf_counter()
        logits = ctx.step([(i, [int(np.argmax(logits[i]))], prompt + s, True) for i in range(rows)])
        times.append(time.perf_counter() - t0)
    ctx.close()
    m.close()
    return rows / statistics.median(times), times, cores


def run_reference(args, cfg, rank, world):
    """The reference's CPU path for the same metric: the CPU restatement with every host thread,
    one bounded decode step per timed step."""
    if rank != 0:
        return
    path = ensure_model(args.workload, 0, host_only=True)
    from oracle import oracle as O

    # the thread count is set here, not inherited: torchrun exports OMP_NUM_THREADS=1 to its children
    cores = O.threads(host_cores())
    rows, prompt = 8, 4
    m = O.Model(str(path), fast=True, act_q8=True)
    ctx = O.Context(m, rows, 64 + args.steps + args.warmup)
    rng = np.random.default_rng(1)
    vocab = cfg["spec"]["vocab"]
    logits = ctx.step([(i, rng.integers(3, vocab, prompt).tolist(), 0, True) for i in range(rows)])
    times = []
    for s in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        logits = ctx.step([(i, [int(np.argmax(logits[i]))], prompt + s, True) for i in range(rows)])
        if s >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = rows * len(times) / total
    sample = (f"{rows} concurrent requests, {prompt}-token prompts, {len(times)} decode steps of the same GGUF on {cores} OpenMP threads: the CPU "
              "restatement of the path (the reference itself cannot be built here) with activations re-quantised to 8-bit blocks and integer dot "
              "products as the reference's CPU backend computes, a bounded decode-only sample, not the GPU arm's 256-request mix")
    print(json.dumps({
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": cfg["name"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kv-dtype", default="f16", choices=["f16", "q8_0", "q4_0"],
                    help="storage type of the KV pool (engine kv_dtype); the headline workload is defined on f16")
    ap.add_argument("--graphs", action="store_true",
                    help="time the steps with the engine's profiler off, so repeated step shapes replay as CUDA graphs; the per-class "
                         "times and the roofline then come from a second, profiled pass of the same number of steps")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return

    if world > 1:
        # the two-rank expert-parallel check below runs on plain NCCL paths (read when the library first
        # initialises in this process, so before the process group exists)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import retrograd_b200 as rb
    from retrograd_b200 import build as B

    if rank == 0 and not rb.LIB_PATH.exists():
        B.build()
    if dist:
        dist.barrier()
    path = ensure_model(args.workload, local_rank if world > 1 else 0)
    if dist:
        dist.barrier()

    # ---- two GPUs or more: ranks 0 and 1 first compare an expert-parallel pair of engines with plain engines on
    # the same rows (a tiny MoE model, every rank of the pair stepping the same number of times); the outcome
    # travels in the line as "ep_parity"
    ep_parity = None
    if world > 1:
        from retrograd_b200.ep_check import plain_vs_expert_parallel

        holder = [rb.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(holder, src=0)
        mine = None
        if rank < 2:
            try:
                result = plain_vs_expert_parallel(rb, rank, 2, holder[0], path.parent)
                result["engine"].close()
                mine = {"steps": result["steps"], "bit_exact": result["bit_exact"], "footprint_split": result["footprint_split"]}
            except Exception as err:      # reported, not fatal: the replica measurement below does not depend on it
                mine = {"steps": 0, "bit_exact": False, "error": str(err)[:200]}
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        pair = [g for g in gathered[:2] if g]
        ep_parity = {"ranks": 2, "steps": min(g["steps"] for g in pair), "bit_exact": all(g["bit_exact"] for g in pair),
                     "footprint_split": all(g.get("footprint_split", False) for g in pair)}
        errors = [g["error"] for g in pair if "error" in g]
        if errors:
            ep_parity["error"] = errors[0]
        dist.barrier()

    engine = rb.Engine(str(path), rb.EngineConfig(n_ctx=cfg["n_ctx"], n_seq_max=cfg["n_requests"], n_batch=cfg["n_batch"], n_ubatch=cfg["n_batch"],
                                                  kv_dtype={"f16": rb.KV_DTYPE_F16, "q8_0": rb.KV_DTYPE_Q8_0, "q4_0": rb.KV_DTYPE_Q4_0}[args.kv_dtype]))
    sampling = rb.SamplingParamsV2.greedy()
    driver = Driver(rb, engine, cfg, Workload(cfg, seed=1000 + rank), sampling)
    if cfg.get("adapters"):
        ad = cfg["adapters"]
        for a in range(ad["n"]):
            apath = path.parent / f"retrograd_b200_adapter_rank{rank}_{a}.gguf"
            write_adapter(apath, cfg["spec"], ad["rank"], ad["alpha"], seed=7000 + a)
            driver.adapter_ids.append(engine.adapter_load(str(apath)))
            apath.unlink()
    expert_parallel = bool(cfg.get("ep")) and world > 1
    if expert_parallel:
        holder = [rb.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(holder, src=0)
        weights_before = engine.memory_report()["model_weight_bytes"]
        engine.ep_init(rank, world, holder[0])
        driver.expert_parallel = True
        ep_block = {"world": world, "experts_per_rank": cfg["spec"]["experts"] // world, "exchange": "NCCL send/recv of f32 rows, per MoE layer",
                    "weight_bytes_per_rank_before": weights_before, "weight_bytes_per_rank": engine.memory_report()["model_weight_bytes"]}

    # ---- ramp (untimed): a steady-state snapshot - every slot holds a request caught mid-flight
    driver.admit(midflight=True)
    ramp_steps = 0
    while True:
        busy = any(r.last is None for r in driver.live)
        if expert_parallel:
            # every rank joins every step's exchange: ramp until the slowest rank is done
            flag = torch.tensor([1 if busy else 0], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            if not int(flag.item()):
                break
            if busy:
                driver.step(prefill_only=True)
            else:
                engine.ep_idle_step()
        else:
            if not busy:
                break
            driver.step(prefill_only=True)     # no request advances its generation during the ramp
        ramp_steps += 1
    for _ in range(args.warmup):
        driver.step()
        driver.admit()

    # ---- timed region: exactly K steps
    engine.profile(not args.graphs, reset=True)
    clocks = ClockSampler(local_rank)
    clocks.start()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_push("timed")
    dev_ms, wall_s, decode_tokens, prefill_tokens, rows_per_step, launches, h2d, d2h = 0.0, 0.0, 0, 0, [], 0, 0, 0
    attn_bytes = 0
    gemm_flops = 0
    gemm_bytes = 0      # algorithmic bytes of the weight GEMMs: weights once per step, activations in (hi + lo, 4 B per element) and out (f32)
    step_tokens = 0
    # bytes of K and V one resident token holds over all layers: 2 per value in f16, 34 / 32 in Q8_0, 18 / 32 in Q4_0
    kv_value_bytes = {"f16": 2.0, "q8_0": 34.0 / 32.0, "q4_0": 18.0 / 32.0}[args.kv_dtype]
    kv_tok_bytes = 2 * cfg["spec"]["layers"] * cfg["spec"]["kv_heads"] * (cfg["spec"].get("head_dim") or cfg["spec"]["d"] // cfg["spec"]["heads"]) * kv_value_bytes
    sp = cfg["spec"]
    hd = sp.get("head_dim") or sp["d"] // sp["heads"]
    w_elems_layer = sp["d"] * (sp["heads"] * hd + 2 * sp["kv_heads"] * hd) + sp["heads"] * hd * sp["d"] + 3 * sp["d"] * sp["ff"]
    if sp.get("experts"):      # per token: the router and the experts it uses
        w_elems_layer += sp["d"] * sp["experts"] + (sp["experts_used"] - 1) * 3 * sp["d"] * sp["ff"]
    for _ in range(args.steps):
        info = driver.step()
        ms, n_launch = engine.last_step_stats()
        a, b = engine.last_step_io()
        dev_ms += ms
        wall_s += info["wall"]
        decode_tokens += info["sampled"]
        prefill_tokens += info["prefill"]
        rows_per_step.append(len(info["rows"]))
        launches += n_launch
        h2d += a
        d2h += b
        attn_bytes += info["ctx_tokens"] * kv_tok_bytes
        step_tokens += info["tokens"]
        gemm_flops += 2 * (info["tokens"] * w_elems_layer * sp["layers"] + info["sampled"] * sp["d"] * sp["vocab"])
        gemm_bytes += gemm_step_bytes(sp, hd, w_elems_layer, info["tokens"], info["sampled"])
        driver.admit()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    if dist:
        dist.barrier()
    clocks.stop_flag.set()
    clocks.join()
    if args.graphs:
        # second pass, profiled (eager launches): per-class device times and the roofline's kernel time
        engine.profile(True, reset=True)
        attn_bytes = gemm_flops = gemm_bytes = step_tokens = 0
        for _ in range(args.steps):
            info = driver.step()
            attn_bytes += info["ctx_tokens"] * kv_tok_bytes
            step_tokens += info["tokens"]
            gemm_flops += 2 * (info["tokens"] * w_elems_layer * sp["layers"] + info["sampled"] * sp["d"] * sp["vocab"])
            gemm_bytes += gemm_step_bytes(sp, hd, w_elems_layer, info["tokens"], info["sampled"])
            driver.admit()
        torch.cuda.synchronize()
    profile = engine.profile_read()
    engine.profile(False)

    # ---- decode-only steps on the same engine and model (untimed for `value`): the weight stream of a whole
    # step against the measured HBM rate. No admissions, no prefill rows; repeated shapes replay as CUDA graphs.
    decode_only = []
    weight_bytes_step = None
    if not expert_parallel:
        bpw_of = {"q4_k": 144 / 256, "q8_0": 34 / 32, "mxfp4": 17 / 32, "f16": 2.0, "f32": 4.0}
        bpw = bpw_of.get(sp["dtype"], 1.0)
        if sp.get("experts"):
            # a decode step of hundreds of rows touches every expert: all banks once, the dense matrices once
            dense = sp["d"] * (sp["heads"] * hd + 2 * sp["kv_heads"] * hd) + sp["heads"] * hd * sp["d"]
            banks = sp["experts"] * 3 * sp["d"] * sp["ff"] * bpw_of.get(sp.get("expert_dtype", sp["dtype"]), 1.0)
            weight_bytes_step = sp["layers"] * (dense * bpw + sp["d"] * sp["experts"] * 4 + banks) + sp["d"] * sp["vocab"] * bpw
        else:
            weight_bytes_step = (sp["layers"] * w_elems_layer + sp["d"] * sp["vocab"]) * bpw
        decoders = sum(1 for r in driver.live if r.last is not None)
        for want in ((cfg["n_requests"],) if sp.get("experts") else (8, cfg["n_requests"])):
            n_rows = min(want, decoders)
            if n_rows == 0 or any(d["rows"] == n_rows for d in decode_only):
                continue
            times = []
            for i in range(3 + 10):
                driver.step(decode_only=n_rows)
                if i >= 3:
                    times.append(engine.last_step_stats()[0])
            ms = statistics.mean(times)
            decode_only.append({"rows": n_rows, "ms_per_step": ms, "tok_s": n_rows / (ms * 1e-3)})

    # inter-token gaps of every request that sampled more than once in the timed region
    gaps = []
    for r in driver.live:
        t = r.times[-(args.steps + 1):]
        gaps += [1e3 * (b - a) for a, b in zip(t, t[1:])]

    # ---- the same workload going on for K more steps without the profiler's events between kernel classes (untimed for
    # `value`): repeated step shapes replay as CUDA graphs and dependent launches overlap, as they do for a caller
    unprofiled = None
    if not args.graphs and world == 1:
        u_ms, u_sampled, u_tokens = 0.0, 0, 0
        for _ in range(args.steps):
            info = driver.step()
            u_ms += engine.last_step_stats()[0]
            u_sampled += info["sampled"]
            u_tokens += info["tokens"]
            driver.admit()
        torch.cuda.synchronize()
        unprofiled = {"steps": args.steps, "tok_s": u_sampled / (u_ms * 1e-3), "ms_per_step": u_ms / args.steps,
                      "tokens_per_step": u_tokens / args.steps,
                      "note": "K later steps of the same request stream with the engine's profiler off (their own token mix)"}

    from retrograd_b200.replicas import aggregate

    # every rank's own step time, so that a slow whole-job step can be attributed (imbalance of the seeded
    # request streams, or one GPU's clocks)
    rank_ms = [dev_ms / args.steps]
    if dist:
        gathered = [None] * world
        dist.all_gather_object(gathered, dev_ms / args.steps)
        rank_ms = [float(x) for x in gathered]
    # whole job: the slowest rank's time, every rank's tokens (replicas, no data-path collective)
    (dev_ms, wall_s), (decode_tokens, prefill_tokens, launches, step_tokens_all) = aggregate(
        [dev_ms, wall_s], [decode_tokens, prefill_tokens, launches, step_tokens], dist, torch.device("cuda", local_rank))
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        engine.close()
        return

    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    top = max(("gemm", "attention"), key=lambda k: profile[k]["ms"])
    bytes_per_weight = {"q4_k": 144 / 256, "q8_0": 34 / 32, "f16": 2.0, "f32": 4.0}.get(sp["dtype"], 1.0)
    if top == "gemm" and step_tokens / args.steps <= 16:
        # few tokens per step: the launches are bound by streaming every weight byte once per step
        weight_bytes = (sp["layers"] * w_elems_layer + sp["d"] * sp["vocab"]) * bytes_per_weight * args.steps
        achieved = weight_bytes / (profile["gemm"]["ms"] * 1e-3) / 1e9
        # DRAM traffic per launch: the capture of the streaming kernel on a 295 MB matrix read 295.7 MB and wrote
        # 9.4 MB for 295.5 MB of weights (profiles/gemm_q4k_stream_128256x4096.md); traffic grows with the bytes
        roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": weight_bytes / max(profile["gemm"]["launches"], 1) * (295.7 + 9.4) / 295.5,
                "traffic_source": "algorithmic bytes per launch x the DRAM/algorithmic ratio of the one-launch ncu capture in profiles/",
                "kernel": "dequant-fused weight-streaming GEMM (all launches of the timed region)"}
    elif top == "gemm":
        achieved = gemm_flops / (profile["gemm"]["ms"] * 1e-3) / 1e12
        # DRAM traffic per launch: the capture of the tcgen05 kernel at 2048 tokens moved 314 MB for 335 MB of
        # algorithmic bytes (profiles/gemm_q4k_tc5_28672x4096_2048tok.md); traffic grows with the tokens and rows
        roof = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                "traffic": gemm_bytes / max(profile["gemm"]["launches"], 1) * 314.0 / 334.6,
                "traffic_source": "algorithmic bytes per launch x the DRAM/algorithmic ratio of the one-launch ncu capture in profiles/",
                "kernel": "dequant-fused weight GEMM (all launches of the timed region)"}
    else:
        achieved = attn_bytes / (profile["attention"]["ms"] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": None, "kernel": "paged ragged attention (all launches of the timed region)"}
    # the paged attention kernels beside it: KV bytes the step's rows had to read / their device time
    if profile["attention"]["ms"] > 0:
        a_gbs = attn_bytes / (profile["attention"]["ms"] * 1e-3) / 1e9
        roof["attention"] = {"bound": "hbm", "achieved": a_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": a_gbs / hbm_peak,
                             "kv_bytes_per_step": attn_bytes / args.steps}
    roof["peak_source"] = f"of {peak_kind}"
    roof["launches"] = profile[top]["launches"]
    roof["avg_launch_ms"] = profile[top]["ms"] / max(profile[top]["launches"], 1)

    line = {
        "metric": "decode_tokens_per_s", "value": decode_tokens / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "n_batch": cfg["n_batch"], "n_ctx": cfg["n_ctx"], "parallelism": f"expert parallel x{world}" if expert_parallel else f"replicas x{world}",
                   "arrivals": "closed loop: a new request is admitted the moment a slot frees (the saturated steady state of the arrival process)",
                   "rows_per_step": statistics.mean(rows_per_step), "decode_tokens_per_step": decode_tokens / args.steps / world,
                   "prefill_tokens_per_step": prefill_tokens / args.steps / world, "tokens_per_step": step_tokens_all / args.steps / world,
                   "ramp_steps": ramp_steps, "cuda_graphs": bool(args.graphs), "kv_dtype": args.kv_dtype,
                   "l2": "inputs larger than L2: every step streams >4 GB of weights and the ragged KV"},
        "e2e": {"value": decode_tokens / wall_s, "unit": "tok/s", "h2d_bytes_per_step": h2d / args.steps, "d2h_bytes_per_step": d2h / args.steps},
        "gpu_launches": int(launches),
        "p50_inter_token_ms": statistics.median(gaps) if gaps else None,
        "clocks": clocks.summary(),
        "rank_ms_per_step": {"min": min(rank_ms), "median": statistics.median(rank_ms), "max": max(rank_ms)},
        "roofline": roof,
        "kernel_classes_ms": {k: round(v["ms"], 3) for k, v in profile.items()},
    }
    if decode_only:
        for d in decode_only:
            d["weight_gbs"] = weight_bytes_step / (d["ms_per_step"] * 1e-3) / 1e9
            d["frac"] = d["weight_gbs"] / hbm_peak
        line["decode_only"] = decode_only
    if unprofiled is not None:
        line["unprofiled"] = unprofiled
    if ep_parity is not None:
        line["ep_parity"] = ep_parity
    if expert_parallel:
        line["expert_parallel"] = ep_block
    engine.close()
    # a correctness record beside the timing: the tiny CPU-runnable workload replayed through the same library, its
    # greedy streams compared token for token with the streams the CPU oracle committed under tests/golden/
    from retrograd_b200.golden_check import replay

    line["golden_check"] = replay(rb)
    if world == 1 and not args.no_cpu_baseline:
        value, times, cores = cpu_baseline(path, cfg)
        line["cpu_baseline"] = {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                                "sample": f"8 concurrent requests, 4-token prompts, {len(times)} decode steps of the same GGUF (CPU restatement, activations re-quantised to 8-bit blocks, integer dot products)"}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
