"""Prompt-lookup (n-gram) proposer.

For each request the longest suffix of its tokens (between ``min_n`` and ``max_n`` long)
that occurred earlier in the same sequence is located and the tokens that followed that
occurrence are proposed.  Runs on the host over the runner's token table
(vllm_ascend/spec_decode/__init__.py:33-58 selects it for method "ngram"; the reference's
CPU implementation is numba-compiled, this one is vectorised numpy).
"""
from __future__ import annotations

import numpy as np


def find_ngram_continuation(tokens: np.ndarray, min_n: int, max_n: int, k: int) -> np.ndarray:
    n_tok = tokens.shape[0]
    for n in range(min(max_n, n_tok - 1), min_n - 1, -1):
        suffix = tokens[n_tok - n:]
        # windows of length n that end before the suffix starts being itself
        limit = n_tok - n
        if limit <= 0:
            continue
        win = np.lib.stride_tricks.sliding_window_view(tokens[:n_tok - 1], n)[:limit]
        hits = np.nonzero((win == suffix).all(axis=1))[0]
        if hits.size:
            start = int(hits[-1]) + n            # most recent earlier occurrence
            out = tokens[start:start + k]
            if out.size:
                return out.astype(np.int32)
    return np.zeros(0, dtype=np.int32)


class NgramProposer:
    name = "ngram"
    needs_hidden_states = False

    def __init__(self, num_speculative_tokens: int, prompt_lookup_min: int = 2, prompt_lookup_max: int = 5,
                 max_model_len: int = 1 << 30):
        self.k, self.min_n, self.max_n = num_speculative_tokens, prompt_lookup_min, prompt_lookup_max
        self.max_model_len = max_model_len

    def propose(self, token_rows: np.ndarray, lengths: np.ndarray, rows: np.ndarray) -> list[np.ndarray]:
        """token_rows: the runner's [max_seqs, max_model_len] table; rows/lengths per request."""
        out = []
        for row, n in zip(rows, lengths):
            k = min(self.k, self.max_model_len - int(n) - 1)
            out.append(find_ngram_continuation(token_rows[row, :n], self.min_n, self.max_n, k) if k > 0
                       else np.zeros(0, dtype=np.int32))
        return out
