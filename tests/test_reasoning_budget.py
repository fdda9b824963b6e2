"""Reasoning-budget forcing (reference: budget_machine, retro_gen_core.cpp:890-1007; driven from the step at
:2609-2680, 2727-2760; retro_engine_set_reasoning_budget, retro_lora_train.h:2622-2627).

The host logic runs without a GPU against a straight restatement of the machine in this file; the GPU test runs
requests through the engine and checks the forced rows' flags, tokens and log-probabilities."""
import numpy as np
import pytest

START, END, ALT_END = [10, 11], [20, 21, 22], [30]


def _machine(start, ends, budget, n_tail, prompt, sampled, incomplete=()):
    """IDLE -> COUNTING -> (WAITING) -> FORCING -> DONE, written the slow way: tag matches are looked up in the
    accepted history instead of being tracked incrementally."""
    state, remaining, pos, seen = "idle", 0, 0, []
    forced_seq = ends[0]

    def closes(tags, history, since):
        # a tag goes by when the history ends with it and the whole tag was accepted after `since`
        return any(len(history) - since >= len(t) and history[-len(t):] == t for t in tags)

    since = 0

    def accept(tok):
        nonlocal state, remaining, pos, since
        seen.append(tok)
        if state == "idle":
            if closes([start], seen, since):
                state, remaining, since = "counting", budget, len(seen)
                if remaining <= 0:
                    state, pos = "forcing", 0
        elif state in ("counting", "waiting"):
            if closes(ends, seen, since):
                state = "done"
                return
            whole = tok not in incomplete
            if state == "waiting":
                if whole:
                    state, pos, since = "forcing", 0, len(seen)
            else:
                remaining -= 1
                if remaining <= 0:
                    if whole:
                        state, pos, since = "forcing", 0, len(seen)
                    else:
                        state = "waiting"
        elif state == "forcing":
            pos += 1
            if pos >= len(forced_seq):
                state = "done"

    tail = prompt[len(prompt) - min(n_tail, len(prompt)):]
    i = 0
    while i < len(tail):
        accept(tail[i])
        i += 1
        if state != "forcing":
            continue
        rest = tail[i:]
        hits = [(k, k + len(t)) for t in ends for k in range(len(rest) - len(t) + 1) if rest[k:k + len(t)] == t]
        if not hits:
            break
        for tok in forced_seq:
            accept(tok)
        i += min(hits)[1]
    out, flags = [], []
    for tok in sampled:
        forced = state == "forcing" and pos < len(forced_seq)
        emit = forced_seq[pos] if forced else tok
        accept(emit)
        out.append(emit)
        flags.append(forced)
    return out, flags


CASES = [
    # (budget, n_tail, prompt, sampled, incomplete)
    (3, 4, [1, 2, 10, 11], [5, 6, 7, 8, 9, 5, 6], ()),                 # three free tokens, then the end tag, then free again
    (3, 4, [1, 2, 10, 11], [5, 20, 21, 22, 9, 5, 6, 7], ()),           # the model closes the block itself
    (0, 2, [10, 11], [5, 6, 7, 8, 9], ()),                             # nothing to spend: forced from the first token
    (2, 8, [10, 11, 4, 20, 21, 22, 3], [5, 6, 7, 8], ()),              # opened and closed inside the prompt
    (2, 2, [7, 7, 7, 10, 11, 3], [5, 6, 7, 8, 9], ()),                 # the tag lies outside the replayed tail: idle
    (5, 6, [9, 9, 9], [1, 10, 11, 2, 3, 30, 4, 10, 11, 5], ()),        # opened by the model, closed by the alternative tag
    (2, 3, [3, 10, 11], [5, 40, 41, 6, 7, 8, 9, 1], (40, 41)),         # budget spent inside a UTF-8 sequence: waits
    (0, 6, [10, 11, 20, 21, 22, 4], [5, 6, 7], ()),                    # budget 0 and an empty block written by the template
    (0, 3, [10, 11, 4], [5, 6, 7, 8], ()),                             # forcing starts on a prompt token, the prompt goes on
    (4, 4, [10, 10, 11, 10], [10, 11, 5, 6, 7, 8, 9, 9], ()),          # a broken partial match restarts
    (1, 2, [10, 11], [20, 5, 6, 7, 8], ()),                            # a partial end tag does not close the block
]


@pytest.mark.parametrize("budget,n_tail,prompt,sampled,incomplete", CASES)
def test_budget_machine_matches_its_restatement(rb, budget, n_tail, prompt, sampled, incomplete):
    ends = [END, ALT_END]
    want = _machine(START, ends, budget, n_tail, prompt, sampled, incomplete)
    got = rb.reasoning_check(START, ends, budget, n_tail, prompt, sampled, incomplete)
    assert got == want
    inactive = rb.reasoning_check(START, ends, -1, n_tail, prompt, sampled, incomplete)
    assert inactive == (list(sampled), [False] * len(sampled))


def test_known_sequences(rb):
    """Spelled out, so that the machine is not only compared with the restatement above."""
    ends = [END, ALT_END]
    assert rb.reasoning_check(START, ends, 3, 4, [1, 2, 10, 11], [5, 6, 7, 8, 9, 5, 6]) == (
        [5, 6, 7, 20, 21, 22, 6], [False, False, False, True, True, True, False])
    assert rb.reasoning_check(START, ends, 0, 2, [10, 11], [5, 6, 7, 8, 9]) == ([20, 21, 22, 8, 9], [True, True, True, False, False])
    assert rb.reasoning_check(START, ends, 2, 3, [3, 10, 11], [5, 40, 41, 6, 7, 8, 9, 1], (40, 41)) == (
        [5, 40, 41, 6, 20, 21, 22, 1], [False, False, False, False, True, True, True, False])


@pytest.mark.gpu
def test_step_rows_report_forced_tokens(rb, c1_model):
    engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=2048, n_seq_max=8, n_batch=128, n_ubatch=128))
    with pytest.raises(rb.EngineError, match="declares no reasoning block"):
        engine.set_reasoning_budget(4)
    with pytest.raises(rb.EngineError, match="must be -1"):
        engine.set_reasoning_budget(-2)
    with pytest.raises(rb.EngineError, match="outside the vocabulary"):
        engine.set_reasoning_tags([5, 10 ** 6], [[7]], 4)
    start, end = [100, 101], [200, 201, 202]
    greedy = rb.SamplingParamsV2.greedy()
    sampled = rb.SamplingParamsV2(temperature=0.9, top_p=0.95, seed=11)
    rng = np.random.default_rng(3)
    body = rng.integers(300, 4000, 40).tolist()
    prompt = body + start                        # the template's generation prompt opened the block
    out = rb.StepOutput(128, 4)

    def run(prompt, slot, request, sampling, n, chunks=None, want_logprob=False):
        """Prefills the prompt in `chunks`, then decodes n tokens; returns the rows' (token, forced, logprob, logits)."""
        pos, rows_out = 0, []
        chunks = chunks or (len(prompt),)
        for c, size in enumerate(chunks):
            last = c == len(chunks) - 1
            engine.step([rb.StepRow(request, slot, prompt[pos:pos + size], pos, sample=last, sampling=sampling, want_logprob=want_logprob)], out)
            pos += size
        for i in range(n):
            r = out.row(0)
            rows_out.append((r.token, r.forced, r.logprob, r.sampled_logprob, engine.last_logits(0).copy()))
            if i + 1 < n:
                engine.step([rb.StepRow(request, slot, [r.token], pos, sample=True, sampling=sampling, want_logprob=want_logprob)], out)
                pos += 1
        return rows_out

    free = run(prompt, 0, 0, greedy, 10)
    assert not any(r[1] for r in free)
    engine.set_reasoning_tags(start, [end], len(start))
    engine.set_reasoning_budget(4)
    # the same request again, its prompt arriving in three chunks: four free tokens, then the end tag, then free again
    limited = run(prompt, 1, 1, greedy, 10, chunks=(17, 24, len(prompt) - 41))      # the opening tag straddles the last two chunks
    assert [r[0] for r in limited[:4]] == [r[0] for r in free[:4]]
    assert [r[0] for r in limited[4:7]] == end and [r[1] for r in limited] == [False] * 4 + [True] * 3 + [False] * 3
    for token, forced, logprob, _, logits in limited:
        lp = logits.astype(np.float64)
        want = lp[token] - lp.max() - np.log(np.exp(lp - lp.max()).sum())
        assert abs(logprob - want) < 1e-4          # the forced token's own log-probability, not the arg-max's
    assert limited[4][0] != int(np.argmax(limited[4][4]))
    # a sampled (non-greedy) request: the draw still happens, the forced rows report the forced token's
    # post-transformation log-probability (minus infinity when the nucleus excluded it)
    drawn = run(prompt, 2, 2, sampled, 8, want_logprob=True)
    assert [r[0] for r in drawn[4:7]] == end and [r[1] for r in drawn] == [False] * 4 + [True] * 3 + [False]
    assert all(r[3] <= 0.0 for r in drawn)
    # a request whose prompt did not open the block is left alone, and budget -1 switches forcing off
    assert not any(r[1] for r in run(body, 3, 3, greedy, 6))
    engine.set_reasoning_budget(-1)
    assert [r[0] for r in run(prompt, 4, 4, greedy, 10)] == [r[0] for r in free]
    engine.close()
