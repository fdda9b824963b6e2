"""Host-side mirror of how the reference's scheduler turns its live request groups into one step plan
(`Scheduler::compose`, crates/retrograd-infer/src/scheduler.rs:933-1089). The scheduler itself stays with
the caller; this restatement exists so that workloads driven from Python (tests, the bench) hand the
engine the same kind of plans the Rust caller would: decode rows first, then prefill chunks and
terminal rows with what is left of the `n_batch` token budget.

Rules restated (line numbers in scheduler.rs):
  * Lockstep never mixes decode rows with prefill / terminal rows: while any group is not decoding, no
    decode row is planned (:945-950).
  * Continuous keeps one token of the budget for prefill progress while a prefill is active; with a
    budget of a single token, decode and prefill take turns (:966-977).
  * When more members decode than the budget allows, a cursor rotates over them so every member
    advances in turn (:978-984).
  * A group prefills its shared prefix `[0, prefix_end)` through its leader in chunks of at most the
    remaining budget; the row samples only when the group has a single member and the chunk ends the
    prompt (:1020-1055).
  * After the prefix was copied to the members, each live member gets a terminal row: the last prompt
    token at position `len(prompt) - 1`, sampled (:1056-1083).

Test infrastructure, like the rest of this folder: the shipped library never imports it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

CONTINUOUS = "continuous"
LOCKSTEP = "lockstep"


@dataclass
class Member:
    request_id: int
    slot: int
    live: bool = True
    next_token: int = 0          # the token its next decode row feeds
    generated: int = 0           # tokens sampled so far
    sampling: Any = None
    n_top_logprobs: int = 0
    want_logprob: bool = False


@dataclass
class Group:
    """Requests that share one prompt (a GRPO group, `n > 1`, or identical prompts merged on admission)."""
    prompt: Sequence[int]
    members: list[Member]
    prefix_end: int = 0          # the leader prefills [0, prefix_end); len(prompt) for a single member, len - 1 for several
    phase: str = "prefill"       # "prefill" | "terminal" | "decode"
    pos: int = 0                 # prefill progress
    next_member: int = 0         # terminal progress
    leader: int = 0
    adapter: int = 0


@dataclass
class PlannedRow:
    request: int
    slot: int
    tokens: list[int]
    pos0: int
    sample: bool
    sampling: Any
    n_top_logprobs: int
    want_logprob: bool
    adapter: int
    kind: tuple = field(default_factory=tuple)     # ("decode", group, member) | ("prefill", group, end, sampled_member) | ("terminal", group, member)


@dataclass
class ComposeState:
    decode_cursor: int = 0
    prefill_turn: bool = False


def compose(live: Sequence[Group], n_batch: int, mode: str, state: ComposeState) -> tuple[list[PlannedRow], int]:
    """One step's rows and their token count. `state` carries the rotation cursor and the turn flag between steps."""
    n_batch = max(int(n_batch), 1)
    rows: list[PlannedRow] = []
    used = 0
    prefill_active = any(g.phase != "decode" for g in live)
    allow_decode = mode == CONTINUOUS or not prefill_active

    decode_list: list[tuple[int, int]] = []
    if allow_decode:
        for gi, g in enumerate(live):
            if g.phase != "decode":
                continue
            decode_list += [(gi, mi) for mi, m in enumerate(g.members) if m.live]
    if mode == CONTINUOUS and prefill_active:
        if n_batch == 1:
            state.prefill_turn = not state.prefill_turn
            decode_budget = 0 if state.prefill_turn else 1
        else:
            decode_budget = n_batch - 1
    else:
        decode_budget = n_batch
    if decode_list:
        start = state.decode_cursor % len(decode_list)
        decode_list = decode_list[start:] + decode_list[:start]
        count = min(decode_budget, len(decode_list))
        state.decode_cursor = (start + count) % len(decode_list)
        decode_list = decode_list[:count]
    for gi, mi in decode_list:
        g, m = live[gi], live[gi].members[mi]
        rows.append(PlannedRow(m.request_id, m.slot, [m.next_token], len(g.prompt) + m.generated - 1, True, m.sampling, m.n_top_logprobs,
                               m.want_logprob, g.adapter, ("decode", gi, mi)))
    used += len(decode_list)

    for gi, g in enumerate(live):
        if used >= n_batch:
            break
        if g.phase == "prefill":
            chunk = min(n_batch - used, g.prefix_end - g.pos)
            if chunk == 0:
                continue
            end = g.pos + chunk
            sampled = 0 if (len(g.members) == 1 and end == len(g.prompt)) else None
            leader = g.members[g.leader]
            rows.append(PlannedRow(leader.request_id, leader.slot, list(g.prompt[g.pos:end]), g.pos, sampled is not None, leader.sampling,
                                   leader.n_top_logprobs if sampled is not None else 0, sampled is not None and leader.want_logprob, g.adapter,
                                   ("prefill", gi, end, sampled)))
            used += chunk
        elif g.phase == "terminal":
            last = len(g.prompt) - 1
            mi = g.next_member
            while mi < len(g.members) and used < n_batch:
                m = g.members[mi]
                if m.live:
                    rows.append(PlannedRow(m.request_id, m.slot, [g.prompt[last]], last, True, m.sampling, m.n_top_logprobs, m.want_logprob,
                                           g.adapter, ("terminal", gi, mi)))
                    used += 1
                mi += 1
    return rows, used
