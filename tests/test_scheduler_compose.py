"""The step-composition rules of the reference's scheduler (crates/retrograd-infer/src/scheduler.rs:933-1089)
as restated in retrograd_b200/scheduler.py: which rows a step carries, in which order, within `n_batch`."""
from oracle.scheduler import CONTINUOUS, LOCKSTEP, ComposeState, Group, Member, compose


def _decoding(gid, n_members, prompt_len=6, generated=3):
    members = [Member(request_id=100 * gid + i, slot=10 * gid + i, next_token=1000 + 100 * gid + i, generated=generated) for i in range(n_members)]
    return Group(prompt=list(range(prompt_len)), members=members, prefix_end=prompt_len, phase="decode")


def _prefilling(gid, prompt_len, n_members=1, pos=0):
    members = [Member(request_id=100 * gid + i, slot=10 * gid + i, n_top_logprobs=3, want_logprob=True) for i in range(n_members)]
    prefix_end = prompt_len if n_members == 1 else prompt_len - 1
    return Group(prompt=list(range(50, 50 + prompt_len)), members=members, prefix_end=prefix_end, phase="prefill", pos=pos)


def test_decode_rows_come_first_then_prefill_chunks_take_the_rest_of_the_budget():
    live = [_decoding(0, 2), _prefilling(1, 40), _decoding(2, 1), _prefilling(3, 9)]
    rows, used = compose(live, 16, CONTINUOUS, ComposeState())
    assert [r.kind[0] for r in rows] == ["decode", "decode", "decode", "prefill"]
    assert [r.request for r in rows[:3]] == [0, 1, 200]
    # a decode row feeds the member's pending token at position len(prompt) + generated - 1
    assert rows[0].tokens == [1000] and rows[0].pos0 == 6 + 3 - 1 and rows[0].sample
    # the first prefilling group takes everything that is left; the second gets nothing this step
    assert rows[3].tokens == list(range(50, 63)) and rows[3].pos0 == 0 and not rows[3].sample
    assert rows[3].n_top_logprobs == 0 and not rows[3].want_logprob
    assert used == 16


def test_a_single_member_samples_on_the_chunk_that_ends_its_prompt():
    g = _prefilling(1, 10, pos=6)
    rows, used = compose([g], 64, CONTINUOUS, ComposeState())
    assert len(rows) == 1 and rows[0].tokens == [56, 57, 58, 59] and rows[0].pos0 == 6
    assert rows[0].sample and rows[0].n_top_logprobs == 3 and rows[0].want_logprob
    assert rows[0].kind == ("prefill", 0, 10, 0) and used == 4


def test_a_merged_group_prefills_all_but_the_last_token_unsampled_then_one_terminal_row_per_live_member():
    g = _prefilling(2, 10, n_members=3)
    rows, used = compose([g], 64, CONTINUOUS, ComposeState())
    assert len(rows) == 1 and len(rows[0].tokens) == 9 and not rows[0].sample and rows[0].kind == ("prefill", 0, 9, None)
    assert rows[0].slot == g.members[0].slot
    g.phase, g.members[1].live = "terminal", False
    rows, used = compose([g], 64, CONTINUOUS, ComposeState())
    assert [r.kind for r in rows] == [("terminal", 0, 0), ("terminal", 0, 2)]
    assert all(r.tokens == [59] and r.pos0 == 9 and r.sample for r in rows) and used == 2
    # a terminal wave that does not fit continues from `next_member` in the next step
    g.members[1].live, g.next_member = True, 1
    rows, used = compose([g], 1, CONTINUOUS, ComposeState())
    assert [r.kind for r in rows] == [("terminal", 0, 1)]


def test_lockstep_never_mixes_decode_with_prefill():
    live = [_decoding(0, 2), _prefilling(1, 5)]
    rows, _ = compose(live, 16, LOCKSTEP, ComposeState())
    assert [r.kind[0] for r in rows] == ["prefill"]
    live[1].phase = "decode"
    live[1].members[0].generated = 1
    rows, _ = compose(live, 16, LOCKSTEP, ComposeState())
    assert [r.kind[0] for r in rows] == ["decode", "decode", "decode"]


def test_continuous_keeps_one_token_for_prefill_and_rotates_the_decoding_members():
    live = [_decoding(0, 5), _prefilling(1, 100)]
    state = ComposeState()
    seen = []
    for _ in range(5):
        rows, used = compose(live, 4, CONTINUOUS, state)
        assert used == 4 and [r.kind[0] for r in rows] == ["decode"] * 3 + ["prefill"]
        assert len(rows[3].tokens) == 1
        seen.append([r.kind[2] for r in rows[:3]])
        live[1].pos += 1
    assert seen == [[0, 1, 2], [3, 4, 0], [1, 2, 3], [4, 0, 1], [2, 3, 4]]
    # without an active prefill the whole budget decodes
    live[1].phase = "decode"
    rows, used = compose(live, 4, CONTINUOUS, state)
    assert used == 4 and all(r.kind[0] == "decode" for r in rows)


def test_a_budget_of_one_token_alternates_between_prefill_and_decode():
    live = [_decoding(0, 1), _prefilling(1, 10)]
    state = ComposeState()
    kinds = []
    for _ in range(4):
        rows, used = compose(live, 1, CONTINUOUS, state)
        assert used == 1 and len(rows) == 1
        kinds.append(rows[0].kind[0])
    assert kinds == ["prefill", "decode", "prefill", "decode"]
