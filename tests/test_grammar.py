"""The GBNF engine behind grammar-constrained rows (host only: `retro_b200_grammar_check`), then constrained
sampling on the GPU: every sampled token must keep the text inside the grammar."""
import re

import numpy as np
import pytest

JSON_GBNF = None


def test_literals_classes_groups_and_repetitions(rb):
    check = rb.grammar_check
    g = 'root ::= "yes" | "no"'
    assert [check(g, t) for t in ("", "y", "yes", "no", "n", "yesx", "maybe")] == [1, 1, 2, 2, 1, 0, 0]
    g = 'root ::= [a-c]+ "-" [0-9]{2,3}'
    assert [check(g, t) for t in ("a", "abc-", "abc-1", "abc-12", "abc-123", "abc-1234", "-12", "abd-12")] == [1, 1, 1, 2, 2, 0, 0, 0]
    g = 'root ::= ("ab" | "c")* "."'
    assert [check(g, t) for t in (".", "ab.", "abcab.", "a", "ac.", "abab")] == [2, 2, 2, 1, 0, 1]
    g = 'root ::= item ("," ws item)*\nitem ::= [^,\\n]+   # anything but a comma\nws ::= " "?'
    assert [check(g, t) for t in ("x", "x, y", "x,y,z", "x,", ",x")] == [2, 2, 2, 1, 0]
    g = 'root ::= "a"? "b"{3} . "\\n"'
    assert [check(g, t) for t in ("abbbZ\n", "bbb?\n", "bbb\n", "abb")] == [2, 2, 1, 1]
    g = 'root ::= "\\u00e9t\\xe9" [\\U0001F600-\\U0001F64F]'
    assert check(g, "été😀") == 2 and check(g, "ét") == 1 and check(g, "ete") == 0


def test_nested_rules_and_the_json_object_grammar(rb):
    lib = rb.load_library()
    h = lib.retro_grammar_json_object()
    gbnf = lib.retro_grammar_gbnf(h).decode()
    lib.retro_grammar_free(h)
    check = rb.grammar_check
    assert check(gbnf, '{"a": [1, 2.5e3, {"b": null}], "c": "x\\n\\u00e9", "d": true}') == 2
    assert check(gbnf, '{"a": [1, 2') == 1
    assert check(gbnf, '{"a" 1}') == 0 and check(gbnf, "[1]") == 0 and check(gbnf, '{"a": 01}') == 0
    g = "root ::= expr\nexpr ::= term ([-+] term)*\nterm ::= num | \"(\" expr \")\"\nnum ::= [0-9]+"
    assert [check(g, t) for t in ("1+2", "(1+2)-3", "((4))", "(1+", "1+)", "()")] == [2, 2, 2, 1, 0, 0]


def test_invalid_grammars_are_refused_with_a_reason(rb):
    for gbnf, why in (("rot ::= \"a\"", "no root rule"), ("root ::= missing", "undefined rule"), ("root ::= \"a", "unterminated literal"),
                      ("root ::= [a-", "unterminated character class"), ("root ::= root \"a\" | \"b\"", "left-recursive"), ("root ::= *", "needs something to repeat"),
                      ("root ::= (\"a\"", "expected )"), ("root \"a\"", "expected ::="), ("root ::= \"a\"{3,2}", "below its lower bound")):
        with pytest.raises(rb.InvalidArgument, match=re.escape(why)):
            rb.grammar_check(gbnf, "a")


@pytest.mark.gpu
def test_grammar_rows_only_sample_what_the_grammar_allows(rb, c1_model):
    """v2 rows with a grammar (retro_gen_core.cpp:773-798, 2738-2745): the mask comes after bias and penalties and
    before top_k; the request keeps its place in the grammar across steps; an end-of-generation token is only
    allowed once the grammar is complete; a row without the grammar drops the request's state."""
    engine = rb.Engine(str(c1_model), rb.EngineConfig(n_ctx=1024, n_seq_max=8, n_batch=128, n_ubatch=128))
    out = rb.StepOutput()
    rng = np.random.default_rng(3)
    digits = rb.Grammar('root ::= [0-9]{3} "-" [a-f]+ "."')
    words = rb.Grammar('root ::= ("yes" | "no") "!"')
    prompts = [rng.integers(3, 4096, n).tolist() for n in (9, 14, 11)]
    sampled = lambda g, seed, **kw: rb.SamplingParamsV2(temperature=1.0, top_p=1.0, seed=seed, grammar=g, **kw)
    params = [sampled(digits, 1), sampled(words, 2, top_k=3), rb.SamplingParamsV2(top_k=1, grammar=digits)]
    rows = [rb.StepRow(i, i, p, 0, sample=True, sampling=params[i], want_logprob=True) for i, p in enumerate(prompts)]
    text = ["", "", ""]
    done = [False] * 3
    for step in range(14):
        engine.step(rows, out)
        nxt = []
        for r, row in enumerate(rows):
            i = row.slot
            tok = out.row(r).token
            if engine.is_eog_token(tok):
                done[i] = True
                continue
            text[i] += engine.detokenize([tok]).decode()
            gbnf = params[i].grammar.gbnf()
            assert rb.grammar_check(gbnf, text[i]) >= 1, (i, text[i])
            assert np.isfinite(out.row(r).sampled_logprob)
            nxt.append(rb.StepRow(i, i, [tok], len(prompts[i]) + step, sample=True, sampling=params[i], want_logprob=True))
        rows = nxt
        if not rows:
            break
    # the grammars are finite or end in a closed tail: every sequence finished with an end-of-generation token
    # right after completing its grammar, or is still inside the open [a-f]+ tail
    assert re.fullmatch(r"(yes|no)!", text[1]) and done[1]
    assert re.fullmatch(r"[0-9]{3}-[a-f]+\.?", text[0]) and re.fullmatch(r"[0-9]{3}-[a-f]+\.?", text[2])
    for i in (0, 2):
        assert done[i] == text[i].endswith(".") or not done[i]
    # a grammar that can never be continued with this vocabulary, an invalid grammar, and a changed grammar text
    impossible = rb.Grammar("root ::= [b-a]")        # an empty range: nothing can ever match
    engine.seq_rm(5)
    with pytest.raises(rb.EngineError, match="grammar allows no token at this position"):
        engine.step([rb.StepRow(40, 5, [7, 8], 0, sample=True, sampling=sampled(impossible, 5))], out)
    engine.seq_rm(5)
    with pytest.raises(rb.InvalidArgument, match="failed to compile the request's grammar"):
        engine.step([rb.StepRow(41, 5, [7, 8], 0, sample=True, sampling=sampled(rb.Grammar("root ::= oops"), 5))], out)
    assert engine.seq_pos(5) == (-1, -1)          # refused before anything was decoded
    only_x = rb.Grammar('root ::= "x"+')
    only_y = rb.Grammar('root ::= "y"+')
    engine.step([rb.StepRow(42, 5, [7, 8], 0, sample=True, sampling=sampled(only_x, 6))], out)
    assert engine.detokenize([out.row(0).token]) == b"x"
    engine.step([rb.StepRow(42, 5, [out.row(0).token], 2, sample=True, sampling=sampled(only_y, 6))], out)     # another text: compiled anew
    assert engine.detokenize([out.row(0).token]) == b"y"
    engine.step([rb.StepRow(42, 5, [out.row(0).token], 3, sample=True, sampling=rb.SamplingParamsV2(top_k=1))], out)  # no grammar: unconstrained
    engine.close()
