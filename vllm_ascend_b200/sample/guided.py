"""Guided (structured) decoding: the next token is restricted to those that keep the generated text
inside a regular language given as a regex, a list of choices or a JSON schema.

The pattern is compiled to a DFA over characters (Thompson construction + subset construction on
demand); the DFA is lifted to tokens by walking a trie of the vocabulary from every reached DFA
state, which yields the allowed token set of the state and the state each token leads to.  Per
step the sampler receives a boolean vocabulary mask per request (the role of the grammar bitmask
the reference applies to the logits before sampling, worker/model_runner_v1.py apply_grammar_bitmask
path of upstream structured output).  The end-of-sequence token is allowed exactly in accepting
states.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

# ---------------------------------------------------------------- regex -> NFA
_DIGIT = set("0123456789")
_WORD = set("abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789_")
_SPACE = set(" \t\n\r\f\v")


class _CharSet:
    """A set of characters, possibly negated (then: every character not listed)."""
    __slots__ = ("chars", "negated")

    def __init__(self, chars, negated: bool = False):
        self.chars, self.negated = frozenset(chars), negated

    def __contains__(self, c: str) -> bool:
        return (c in self.chars) != self.negated


class _NFA:
    def __init__(self):
        self.eps: list[list[int]] = []
        self.edges: list[list[tuple[_CharSet, int]]] = []

    def state(self) -> int:
        self.eps.append([])
        self.edges.append([])
        return len(self.eps) - 1


class _Parser:
    """Recursive-descent parser of the supported regex subset: literals and escapes
    (\\d \\w \\s \\D \\W \\S and escaped metacharacters), ``.``, classes ``[...]`` with ranges and
    negation, groups ``( )`` / ``(?: )``, alternation ``|``, quantifiers ``* + ? {m} {m,} {m,n}``."""

    def __init__(self, pattern: str):
        self.p, self.i, self.nfa = pattern, 0, _NFA()

    def parse(self):
        s, e = self._alt()
        if self.i != len(self.p):
            raise ValueError(f"unexpected {self.p[self.i]!r} at {self.i} in regex")
        return self.nfa, s, e

    def _peek(self) -> Optional[str]:
        return self.p[self.i] if self.i < len(self.p) else None

    def _alt(self):
        branches = [self._concat()]
        while self._peek() == "|":
            self.i += 1
            branches.append(self._concat())
        if len(branches) == 1:
            return branches[0]
        s, e = self.nfa.state(), self.nfa.state()
        for bs, be in branches:
            self.nfa.eps[s].append(bs)
            self.nfa.eps[be].append(e)
        return s, e

    def _concat(self):
        s = e = self.nfa.state()
        while self._peek() is not None and self._peek() not in "|)":
            a, b = self._repeat()
            self.nfa.eps[e].append(a)
            e = b
        return s, e

    def _repeat(self):
        start = self.i
        frag = self._atom()
        while self._peek() in ("*", "+", "?", "{"):
            c = self._peek()
            if c == "{":
                j = self.p.find("}", self.i)
                body = self.p[self.i + 1:j] if j > 0 else ""
                parts = body.split(",")
                if j < 0 or not parts[0].strip().isdigit():
                    break                              # a literal brace
                lo = int(parts[0])
                hi = lo if len(parts) == 1 else (int(parts[1]) if parts[1].strip() else None)
                self.i = j + 1
            else:
                self.i += 1
                lo, hi = {"*": (0, None), "+": (1, None), "?": (0, 1)}[c]
            atom_src = self.p[start:self._atom_end]
            frag = self._times(atom_src, lo, hi)
        return frag

    def _times(self, src: str, lo: int, hi: Optional[int]):
        """``src{lo,hi}`` by re-parsing the atom for every copy (fresh NFA states each time)."""
        def copy():
            sub = _Parser(src)
            sub.nfa = self.nfa
            frag = sub._atom()
            return frag
        s = e = self.nfa.state()
        for _ in range(lo):
            a, b = copy()
            self.nfa.eps[e].append(a)
            e = b
        if hi is None:
            a, b = copy()
            self.nfa.eps[e].append(a)
            self.nfa.eps[b].append(e)
        else:
            end = self.nfa.state()
            for _ in range(hi - lo):
                a, b = copy()
                self.nfa.eps[e].append(a)
                self.nfa.eps[e].append(end)
                e = b
            self.nfa.eps[e].append(end)
            e = end
        return s, e

    def _atom(self):
        c = self._peek()
        if c is None:
            raise ValueError("regex ends where an atom is expected")
        if c == "(":
            self.i += 1
            if self.p.startswith("?:", self.i):
                self.i += 2
            frag = self._alt()
            if self._peek() != ")":
                raise ValueError("unbalanced parenthesis in regex")
            self.i += 1
            self._atom_end = self.i
            return frag
        if c == "[":
            cs = self._cls()
        elif c == ".":
            self.i += 1
            cs = _CharSet("\n", negated=True)
        elif c == "\\":
            cs = self._escape()
        elif c in "*+?":
            raise ValueError(f"nothing to repeat at {self.i} in regex")
        else:
            self.i += 1
            cs = _CharSet(c)
        self._atom_end = self.i
        s, e = self.nfa.state(), self.nfa.state()
        self.nfa.edges[s].append((cs, e))
        return s, e

    def _escape(self) -> _CharSet:
        c = self.p[self.i + 1] if self.i + 1 < len(self.p) else ""
        self.i += 2
        table = {"d": (_DIGIT, False), "D": (_DIGIT, True), "w": (_WORD, False), "W": (_WORD, True),
                 "s": (_SPACE, False), "S": (_SPACE, True)}
        if c in table:
            return _CharSet(*table[c])
        return _CharSet({"n": "\n", "t": "\t", "r": "\r", "f": "\f", "v": "\v"}.get(c, c))

    def _cls(self) -> _CharSet:
        self.i += 1
        neg = self._peek() == "^"
        if neg:
            self.i += 1
        chars: set = set()
        first = True
        while True:
            c = self._peek()
            if c is None:
                raise ValueError("unterminated character class in regex")
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            if c == "\\":
                sub = self._escape()
                if sub.negated:
                    raise ValueError("negated escapes inside a class are not supported")
                chars |= sub.chars
                continue
            self.i += 1
            if self._peek() == "-" and self.i + 1 < len(self.p) and self.p[self.i + 1] != "]":
                hi = self.p[self.i + 1]
                self.i += 2
                chars |= {chr(x) for x in range(ord(c), ord(hi) + 1)}
            else:
                chars.add(c)
        return _CharSet(chars, neg)


# ---------------------------------------------------------------- NFA -> DFA (lazy)
class RegexDFA:
    """Deterministic automaton over characters, built state by state as text walks through it.
    State 0 is the start; ``step`` returns -1 when the character leaves the language's prefixes."""

    def __init__(self, pattern: str):
        self.pattern = pattern
        self.nfa, start, self.accept_nfa = _Parser(pattern).parse()
        self._sets: list[frozenset] = []
        self._index: dict[frozenset, int] = {}
        self._trans: list[dict[str, int]] = []
        self._add(self._closure({start}))

    def _closure(self, states) -> frozenset:
        stack, seen = list(states), set(states)
        while stack:
            s = stack.pop()
            for t in self.nfa.eps[s]:
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)

    def _add(self, fs: frozenset) -> int:
        i = self._index.get(fs)
        if i is None:
            i = len(self._sets)
            self._index[fs] = i
            self._sets.append(fs)
            self._trans.append({})
        return i

    def step(self, state: int, c: str) -> int:
        t = self._trans[state].get(c)
        if t is None:
            nxt = {e for s in self._sets[state] for cs, e in self.nfa.edges[s] if c in cs}
            t = self._add(self._closure(nxt)) if nxt else -1
            self._trans[state][c] = t
        return t

    def accepting(self, state: int) -> bool:
        return self.accept_nfa in self._sets[state]

    def walk(self, state: int, text: str) -> int:
        for c in text:
            state = self.step(state, c)
            if state < 0:
                return -1
        return state

    def fullmatch(self, text: str) -> bool:
        s = self.walk(0, text)
        return s >= 0 and self.accepting(s)


# ---------------------------------------------------------------- DFA -> tokens
class _Trie:
    __slots__ = ("children", "tokens")

    def __init__(self):
        self.children: dict[str, "_Trie"] = {}
        self.tokens: list[int] = []


class TokenVocabulary:
    """Token strings of a model (index = token id) as a character trie; shared by all requests."""

    def __init__(self, tokens: Sequence[Optional[str]], eos_token_id: Optional[int] = None):
        self.size = len(tokens)
        self.eos_token_id = eos_token_id
        self.root = _Trie()
        for tid, text in enumerate(tokens):
            if not text or tid == eos_token_id:
                continue                               # special / empty tokens never match text
            node = self.root
            for c in text:
                node = node.children.setdefault(c, _Trie())
            node.tokens.append(tid)

    @classmethod
    def from_tokenizer(cls, tokenizer, vocab_size: Optional[int] = None) -> "TokenVocabulary":
        """Every id decoded on its own (special tokens become empty strings)."""
        n = vocab_size or len(tokenizer)
        special = set(getattr(tokenizer, "all_special_ids", []) or [])
        toks = [None if i in special else tokenizer.decode([i]) for i in range(n)]
        return cls(toks, getattr(tokenizer, "eos_token_id", None))


class TokenFSM:
    """The DFA lifted to the vocabulary: per DFA state the tokens that stay inside the language and
    where each leads (computed on first visit by a joint walk of the trie and the DFA)."""

    def __init__(self, dfa: RegexDFA, vocab: TokenVocabulary):
        self.dfa, self.vocab = dfa, vocab
        self._next: dict[int, dict[int, int]] = {}
        self._mask: dict[tuple, torch.Tensor] = {}

    def transitions(self, state: int) -> dict[int, int]:
        tr = self._next.get(state)
        if tr is None:
            tr = {}
            stack = [(self.vocab.root, state)]
            while stack:
                node, s = stack.pop()
                for tid in node.tokens:
                    tr[tid] = s
                for c, child in node.children.items():
                    t = self.dfa.step(s, c)
                    if t >= 0:
                        stack.append((child, t))
            self._next[state] = tr
        return tr

    def allowed_mask(self, state: int, vocab_size: int, device) -> torch.Tensor:
        key = (state, vocab_size, str(device))
        m = self._mask.get(key)
        if m is None:
            m = torch.zeros(vocab_size, dtype=torch.bool)
            ids = [t for t in self.transitions(state) if t < vocab_size]
            if ids:
                m[torch.tensor(ids, dtype=torch.long)] = True
            eos = self.vocab.eos_token_id
            if eos is not None and eos < vocab_size and (self.dfa.accepting(state) or not ids):
                m[eos] = True                          # finished (or dead end): only stopping remains
            m = m.to(device)
            self._mask[key] = m
        return m


class GuidedState:
    """Per-request cursor: the DFA state after the tokens generated so far."""

    def __init__(self, fsm: TokenFSM):
        self.fsm, self.state, self.consumed = fsm, 0, 0

    def sync(self, output_token_ids) -> None:
        out = output_token_ids or []
        for tok in out[self.consumed:]:
            if self.state >= 0:
                self.state = self.fsm.transitions(self.state).get(int(tok), -1 if int(tok) != self.fsm.vocab.eos_token_id
                                                                  else self.state)
        self.consumed = len(out)

    def mask(self, vocab_size: int, device) -> torch.Tensor:
        if self.state < 0:                             # left the language (forced token, preemption replay)
            m = torch.zeros(vocab_size, dtype=torch.bool, device=device)
            eos = self.fsm.vocab.eos_token_id
            if eos is not None and eos < vocab_size:
                m[eos] = True
            else:
                m[:] = True
            return m
        return self.fsm.allowed_mask(self.state, vocab_size, device)


# ---------------------------------------------------------------- request-level description
_RE_META = set("\\.[]{}()*+?|^$-")


def regex_escape(text: str) -> str:
    return "".join("\\" + c if c in _RE_META else c for c in text)


_JSON_STRING = r'"([^"\\]|\\["\\/bfnrt])*"'
_JSON_INT = r"(-)?(0|[1-9][0-9]*)"
_JSON_NUMBER = _JSON_INT + r"(\.[0-9]+)?([eE][+-]?[0-9]+)?"
_WS = r"[ ]?"


def json_schema_to_regex(schema) -> str:
    """Regex of the JSON documents of a schema: objects (listed properties in order, all emitted),
    arrays, strings, integers, numbers, booleans, null, enum / const, anyOf."""
    if isinstance(schema, str):
        schema = json.loads(schema)
    if "enum" in schema:
        return "(" + "|".join(regex_escape(json.dumps(v)) for v in schema["enum"]) + ")"
    if "const" in schema:
        return regex_escape(json.dumps(schema["const"]))
    if "anyOf" in schema or "oneOf" in schema:
        return "(" + "|".join(json_schema_to_regex(s) for s in schema.get("anyOf") or schema["oneOf"]) + ")"
    t = schema.get("type")
    if isinstance(t, list):
        return "(" + "|".join(json_schema_to_regex({**schema, "type": x}) for x in t) + ")"
    if t == "string":
        if "pattern" in schema:
            return '"' + schema["pattern"].lstrip("^").rstrip("$") + '"'
        if "maxLength" in schema or "minLength" in schema:
            lo, hi = int(schema.get("minLength", 0)), schema.get("maxLength")
            return r'"([^"\\]|\\["\\/bfnrt]){' + str(lo) + "," + ("" if hi is None else str(int(hi))) + '}"'
        return _JSON_STRING
    if t == "integer":
        return _JSON_INT
    if t == "number":
        return _JSON_NUMBER
    if t == "boolean":
        return "(true|false)"
    if t == "null":
        return "null"
    if t == "array":
        item = json_schema_to_regex(schema.get("items") or {"type": "string"})
        lo = int(schema.get("minItems", 0))
        hi = schema.get("maxItems")
        rest = "(," + _WS + item + ")" + ("{" + str(max(lo - 1, 0)) + "," + ("" if hi is None else str(int(hi) - 1)) + "}")
        body = item + rest
        return r"\[" + _WS + (body if lo > 0 else "(" + body + ")?") + _WS + r"\]"
    if t == "object" or "properties" in schema:
        props = schema.get("properties") or {}
        parts = [regex_escape(json.dumps(k)) + ":" + _WS + json_schema_to_regex(v) for k, v in props.items()]
        return r"\{" + _WS + ("," + _WS).join(parts) + _WS + r"\}"
    raise ValueError(f"unsupported JSON schema fragment: {schema}")


@dataclass
class GuidedDecodingParams:
    """Exactly one of: ``regex``; ``choice`` (list of strings); ``json`` (schema as dict or str)."""
    regex: Optional[str] = None
    choice: Optional[list] = None
    json: Optional[object] = None

    def pattern(self) -> str:
        given = [x is not None for x in (self.regex, self.choice, self.json)]
        if sum(given) != 1:
            raise ValueError("guided decoding takes exactly one of regex / choice / json")
        if self.regex is not None:
            return self.regex
        if self.choice is not None:
            return "(" + "|".join(regex_escape(str(c)) for c in self.choice) + ")"
        return json_schema_to_regex(self.json)


class GuidedDecodingManager:
    """Engine-side cache: one token FSM per distinct pattern over the engine's vocabulary."""

    def __init__(self, vocab: TokenVocabulary):
        self.vocab = vocab
        self._fsm: dict[str, TokenFSM] = {}

    def new_state(self, params: GuidedDecodingParams) -> GuidedState:
        pat = params.pattern()
        fsm = self._fsm.get(pat)
        if fsm is None:
            fsm = self._fsm[pat] = TokenFSM(RegexDFA(pat), self.vocab)
        return GuidedState(fsm)
