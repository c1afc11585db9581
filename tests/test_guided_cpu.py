"""Guided decoding: regex compiler against Python's ``re``, token-level automaton, engine output."""
import json
import re

import numpy as np
import pytest
import torch

from vllm_ascend_b200.sample.guided import (GuidedDecodingParams, GuidedState, RegexDFA, TokenFSM, TokenVocabulary,
                                            json_schema_to_regex)


@pytest.mark.parametrize("pattern", [r"(yes|no|maybe( so)?)", r"[a-c]{2,3}\d+x?", r"\w+@\w+\.(com|org)",
                                     r"-?(0|[1-9][0-9]*)(\.[0-9]{1,3})?", r"[^,;]*,[ ]?(ab)*", r"a{3}b{2,}c?"])
def test_regex_compiler_agrees_with_re(pattern):
    dfa = RegexDFA(pattern)
    rng = np.random.default_rng(0)
    alphabet = "abcxyz019 .,;-@_omrg"
    samples = ["yes", "no", "maybe so", "abc12x", "ab1", "me@site.com", "a@b.org", "-12.345", "0.5", "007", "q, abab",
               "aaabb", "aaabbbbc", "aabb", ""]
    samples += ["".join(rng.choice(list(alphabet), size=rng.integers(1, 9))) for _ in range(400)]
    for s in samples:
        assert dfa.fullmatch(s) == bool(re.fullmatch(pattern, s)), (pattern, s)


def _toy_vocab():
    pieces = ["<eos>", "y", "e", "s", "n", "o", "yes", "no", "ma", "ybe", " so", "maybe", "{", "}", '"', ":", ",", " ",
              "name", "age", "0", "1", "2", "7", "42", "bob", "al", "ice", "true", "false", '"name"', '":', "[", "]", "-",
              "x", "zz", '{"', '",', "ag", 'e"', "be", "k", "l"]
    return pieces, TokenVocabulary(pieces, eos_token_id=0)


def test_token_fsm_allows_exactly_the_tokens_that_extend_a_match():
    pieces, vocab = _toy_vocab()
    fsm = TokenFSM(RegexDFA(r"(yes|no|maybe( so)?)"), vocab)
    start = {pieces[t] for t in fsm.transitions(0)}
    assert start == {"y", "yes", "n", "no", "ma", "maybe"}
    st = GuidedState(fsm)
    st.sync([pieces.index("ma")])
    assert {pieces[t] for t in fsm.transitions(st.state)} == {"ybe", "y"}
    st.sync([pieces.index("ma"), pieces.index("ybe")])
    m = st.mask(len(pieces), "cpu")
    assert {pieces[i] for i in m.nonzero().flatten().tolist()} == {"<eos>", " so", " "}      # accepting: may stop or go on
    st.sync([pieces.index("ma"), pieces.index("ybe"), pieces.index(" so")])
    assert st.mask(len(pieces), "cpu").nonzero().flatten().tolist() == [0]              # only stopping remains


def test_engine_output_stays_in_the_language():
    from vllm_ascend_b200 import LLM, SamplingParams
    pieces, _ = _toy_vocab()
    llm = LLM("tiny-qwen", device="cpu", seed=0, block_size=16, max_model_len=128, max_num_seqs=8)
    V = llm.cfg.model.vocab_size
    llm.set_guided_vocabulary(pieces + [None] * (V - len(pieces)), eos_token_id=0)
    text = lambda ids: "".join(pieces[t] for t in ids if t != 0)              # noqa: E731
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, 500, size=n).tolist() for n in (9, 14, 5)]
    schema = {"type": "object", "properties": {"name": {"enum": ["bob", "alice"]}, "age": {"type": "integer"},
                                               "ok": {"type": "boolean"}}}
    with pytest.raises(ValueError):
        SamplingParams(guided_decoding={"regex": "a", "choice": ["b"]}).guided_decoding.pattern()
    cases = [GuidedDecodingParams(choice=["yes", "no", "maybe so"]),
             GuidedDecodingParams(regex=r"(no|yes){2,3}"),
             GuidedDecodingParams(json=schema)]
    for temp in (0.0, 1.0):
        sps = [SamplingParams(temperature=temp, max_tokens=40, seed=3, guided_decoding=g) for g in cases]
        outs = llm.generate(prompts, sps)
        got = [text(o.outputs[0].token_ids) for o in outs]
        assert got[0] in ("yes", "no", "maybe so")
        assert re.fullmatch(r"(no|yes){2,3}", got[1])
        doc = json.loads(got[2])
        assert set(doc) == {"name", "age", "ok"} and doc["name"] in ("bob", "alice") and isinstance(doc["age"], int)
        assert all(o.outputs[0].finish_reason == "stop" for o in outs)
    # unguided requests in the same batch are untouched
    plain = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    mixed = llm.generate(prompts[:2], [plain, SamplingParams(temperature=0.0, max_tokens=8, guided_decoding=cases[0])])
    assert mixed[0].outputs[0].token_ids == llm.generate(prompts[:1], plain)[0].outputs[0].token_ids
    assert text(mixed[1].outputs[0].token_ids) in ("yes", "no", "maybe so")


def test_json_schema_regex_matches_documents():
    schema = {"type": "object", "properties": {
        "id": {"type": "integer"}, "score": {"type": "number"}, "tags": {"type": "array", "items": {"type": "string"}},
        "kind": {"enum": ["a", "b"]}, "note": {"type": ["string", "null"]}}}
    pat = json_schema_to_regex(schema)
    dfa = RegexDFA(pat)
    good = {"id": 3, "score": -1.5e3, "tags": ["x", "y z"], "kind": "b", "note": None}
    assert dfa.fullmatch(json.dumps(good, separators=(",", ":")))
    assert dfa.fullmatch(json.dumps(good, separators=(", ", ": ")))
    assert dfa.fullmatch(json.dumps({**good, "tags": []}, separators=(",", ":")))
    assert not dfa.fullmatch(json.dumps({**good, "kind": "c"}, separators=(",", ":")))
    assert not dfa.fullmatch(json.dumps({**good, "id": 1.5}, separators=(",", ":")))
