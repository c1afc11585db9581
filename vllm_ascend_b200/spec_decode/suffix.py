"""Suffix-matching proposer with a cache shared across requests.

Like prompt lookup, but the candidate continuations come from every sequence seen recently
(prompts and generations), indexed by their last tokens; the continuation with the most
occurrences wins.  Serves workloads with repeated structure across requests (role of the
reference's "suffix" method, spec_decode/__init__.py:33-58).
"""
from __future__ import annotations

from collections import Counter, OrderedDict, defaultdict

import numpy as np


class SuffixProposer:
    name = "suffix"
    needs_hidden_states = False

    def __init__(self, num_speculative_tokens: int, max_depth: int = 24, max_model_len: int = 1 << 30,
                 key_len: int = 3, max_entries: int = 1 << 16):
        self.k, self.depth, self.max_model_len = num_speculative_tokens, max_depth, max_model_len
        self.key_len, self.max_entries = key_len, max_entries
        self.table: "OrderedDict[tuple, Counter]" = OrderedDict()
        self._indexed: dict[int, int] = defaultdict(int)       # row -> tokens already indexed

    def _index(self, row: int, toks: np.ndarray) -> None:
        start = max(self._indexed[row], self.key_len)
        if start > len(toks) - 1:
            return
        for i in range(start, len(toks)):
            key = tuple(int(t) for t in toks[i - self.key_len:i])
            cont = tuple(int(t) for t in toks[i:i + self.k])
            c = self.table.get(key)
            if c is None:
                c = self.table[key] = Counter()
                if len(self.table) > self.max_entries:
                    self.table.popitem(last=False)
            else:
                self.table.move_to_end(key)
            c[cont] += 1
        self._indexed[row] = len(toks)

    def forget(self, row: int) -> None:
        self._indexed.pop(row, None)

    def propose(self, token_rows: np.ndarray, lengths: np.ndarray, rows: np.ndarray) -> list[np.ndarray]:
        out = []
        for row, n in zip(rows, lengths):
            n = int(n)
            toks = token_rows[row, :n]
            if self._indexed.get(int(row), 0) > n:          # the row was reused by a new request
                self._indexed[int(row)] = 0
            self._index(int(row), toks[:n - 1] if n > 1 else toks)
            k = min(self.k, self.max_model_len - n - 1)
            best = None
            if n >= self.key_len and k > 0:
                c = self.table.get(tuple(int(t) for t in toks[n - self.key_len:n]))
                if c:
                    best = max(c.items(), key=lambda kv: (kv[1], len(kv[0])))[0]
            out.append(np.asarray(best[:k], dtype=np.int32) if best else np.zeros(0, dtype=np.int32))
        return out
