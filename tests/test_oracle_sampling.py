"""Behaviour of the restated CPU sampling oracle
(crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:41-51,103-225,718-875,2942-2985)."""
import numpy as np


def _logits(seed=0, n=4096):
    return np.random.default_rng(seed).normal(0, 1.5, n).astype(np.float32)


def test_log_softmax_terms_match_a_double_precision_restatement(oracle):
    l = _logits(1)
    mx, ls = oracle.log_softmax_terms(l)
    assert mx == l.max()
    acc = 0.0
    for v in l:
        acc += np.exp(np.float64(v) - np.float64(mx))
    assert ls == np.log(acc)


def test_tiny_nucleus_is_the_arg_max(oracle):
    # the serving layer spells greedy as temperature 1e-4 / top_p 1e-6
    # (crates/retrograd-openai/src/chat/convert.rs:24-30)
    for seed in range(8):
        l = _logits(seed)
        tok, lp = oracle.sample_token(l, 1e-4, 1e-6, oracle.Rng(seed))
        assert tok == int(np.argmax(l))
        assert lp == oracle.token_logprob(l, tok)


def test_top_p_one_draw_is_reproducible_and_follows_the_distribution(oracle):
    l = np.array([0.0, 1.0, 2.0, -1.0], dtype=np.float32)
    rng = oracle.Rng(1234)
    draws = np.array([oracle.sample_token(l, 1.0, 1.0, rng)[0] for _ in range(4000)])
    again = oracle.Rng(1234)
    assert draws[0] == oracle.sample_token(l, 1.0, 1.0, again)[0]
    p = np.exp(l - l.max())
    p /= p.sum()
    freq = np.bincount(draws, minlength=4) / draws.size
    assert np.abs(freq - p).max() < 0.03


def test_nucleus_keeps_the_smallest_prefix_reaching_top_p(oracle):
    l = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float64)).astype(np.float32)
    rng = oracle.Rng(7)
    seen = {oracle.sample_token(l, 1.0, 0.75, rng)[0] for _ in range(500)}
    assert seen == {0, 1}


def test_top_token_logprobs_order_and_ties(oracle):
    l = _logits(3, 512)
    l[10] = l[400] = l.max() + 1.0  # a tie at the top: the lower id first
    ids, lps = oracle.top_token_logprobs(l, 5)
    assert list(ids[:2]) == [10, 400]
    order = sorted(range(512), key=lambda i: (-l[i], i))[:5]
    assert list(ids) == order
    assert lps[0] == oracle.token_logprob(l, 10)


def test_v2_top_k_one_is_greedy_over_the_transformed_logits(oracle):
    l = _logits(5, 300)
    best = int(np.argmax(l))
    tok, lp, slp, ids, lps = oracle.sample_token_v2(l, oracle.Rng(0), top_k=1, k=2)
    assert tok == best and slp == 0.0 and ids[0] == best
    assert lp == oracle.token_logprob(l, best)
    # a bias moves the arg-max; the reported policy logprob stays the raw one
    other = (best + 7) % 300
    tok2, lp2, *_ = oracle.sample_token_v2(l, oracle.Rng(0), top_k=1, logit_bias=[(other, 100.0)])
    assert tok2 == other and lp2 == oracle.token_logprob(l, other)


def test_v2_penalties_follow_the_window(oracle):
    l = np.zeros(16, dtype=np.float32)
    l[3] = 2.0
    l[5] = 1.9
    # token 3 was emitted twice inside the window: frequency 2 * 0.5 pushes it below token 5
    tok, *_ = oracle.sample_token_v2(l, oracle.Rng(0), top_k=1, frequency_penalty=0.5, history=[3, 3], penalty_window=2)
    assert tok == 5
    # outside the window the penalty does not apply
    tok, *_ = oracle.sample_token_v2(l, oracle.Rng(0), top_k=1, frequency_penalty=0.5, history=[3, 3, 7], penalty_window=1)
    assert tok == 3


def test_philox_draw_restatement(oracle):
    u = [oracle.philox_uniform(42, i) for i in range(2000)]
    assert all(0.0 <= x < 1.0 for x in u)
    assert abs(np.mean(u) - 0.5) < 0.03
    assert oracle.philox_uniform(42, 5) == u[5] and oracle.philox_uniform(43, 5) != u[5]
    l = _logits(9, 1000)
    tok, margin = oracle.sample_philox(l, 1.0, 1.0, 42, 0)
    assert 0 <= tok < 1000 and margin >= 0.0
    # a one-token nucleus is the arg-max whatever the draw
    assert oracle.sample_philox(l, 1e-4, 1e-6, 1, 0)[0] == int(np.argmax(l))
