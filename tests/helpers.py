"""Drives the CUDA engine (through the C ABI) and the CPU oracle with one step plan."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

LOGIT_TOL = 1e-2  # max abs difference of fp32 logits after the dequant-GEMM chain (the stated tolerance)


@dataclass
class ParityReport:
    steps: int = 0
    sampled: int = 0
    max_logit_diff: float = 0.0
    max_logprob_diff: float = 0.0
    min_margin: float = float("inf")
    tie_events: int = 0
    streams: dict = field(default_factory=dict)


def check_step(rb, engine, octx, O, rows, out, report: ParityReport, check_maps: bool = True):
    """rows: list of rb.StepRow. Runs the step on both sides and compares everything visible."""
    engine.step(rows, out)
    ologits = octx.step([(r.slot, list(r.tokens), r.pos0, r.sample, r.adapter) for r in rows])
    report.steps += 1
    if check_maps:
        want = O.pack([(r.slot, len(r.tokens), r.pos0, r.sample) for r in rows])
        got = engine.last_pack()
        for key in ("tok_slot", "tok_pos", "tok_row", "out_index"):
            assert np.array_equal(got[key], want[key]), key
        assert np.array_equal(got["cu_rows"][: len(rows) + 1], want["cu_rows"])
        # block tables resolve every token to the cell its slot's table names
        for slot in {r.slot for r in rows}:
            table, B = engine.block_table(slot)
            sel = got["tok_slot"] == slot
            pos = got["tok_pos"][sel]
            assert np.array_equal(got["tok_cell"][sel], table[pos // B] * B + pos % B)
    s = 0
    tokens = {}
    for r, row in enumerate(rows):
        o = out.row(r)
        assert o.sampled == row.sample
        if not row.sample:
            continue
        glogits = engine.last_logits(s)
        diff = float(np.abs(glogits - ologits[s]).max())
        report.max_logit_diff = max(report.max_logit_diff, diff)
        assert diff <= LOGIT_TOL, f"logits differ by {diff} at row {r}"
        top2 = np.partition(ologits[s], -2)[-2:]
        margin = float(top2[1] - top2[0])
        report.min_margin = min(report.min_margin, margin)
        tokens[r] = (o, glogits, ologits[s], margin, diff)
        report.sampled += 1
        s += 1
    return tokens


def expect_greedy(O, tokens, report: ParityReport):
    """Greedy rows: the engine's token is the oracle's arg-max (lowest id on ties); a flip is only
    tolerated, and counted, when the oracle's top-2 margin is inside the measured logit error."""
    for r, (o, glogits, ologits, margin, diff) in tokens.items():
        want = int(np.argmax(ologits))
        assert o.token == int(np.argmax(glogits)), "the sampler did not return the arg-max of its own logits"
        if o.token != want:
            assert margin <= 2 * diff, f"greedy token {o.token} != oracle {want} with margin {margin} > 2 x {diff}"
            report.tie_events += 1
        lp = float(O.token_logprob(glogits, o.token))
        report.max_logprob_diff = max(report.max_logprob_diff, abs(lp - o.logprob))
        assert abs(lp - o.logprob) <= 2e-6 * max(1.0, abs(lp)), (lp, o.logprob)
