"""Paged KV block pool with reference counting and hash-chained prefix caching.

Block 0 is reserved as a null block: padded batch rows and out-of-range table
entries point at it, so kernels always read mapped memory.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from typing import Optional

import numpy as np


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = False):
        assert num_blocks >= 2
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.enable_prefix_caching = enable_prefix_caching
        self.ref = np.zeros(num_blocks, dtype=np.int32)
        self.ref[0] = 1                                   # null block, never freed
        # free blocks in LRU order (oldest first); value unused
        self._free: OrderedDict[int, None] = OrderedDict((i, None) for i in range(1, num_blocks))
        self._hash_to_block: dict[bytes, int] = {}
        self._block_hash: dict[int, bytes] = {}
        self.hits = 0
        self.queries = 0

    # ------------------------------------------------------------------
    @property
    def num_free_blocks(self) -> int:
        return len(self._free)

    @property
    def usage(self) -> float:
        return 1.0 - len(self._free) / max(1, self.num_blocks - 1)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self, n: int) -> list[int]:
        if n > len(self._free):
            raise RuntimeError(f"out of KV blocks: want {n}, free {len(self._free)}")
        out = []
        for _ in range(n):
            b, _ = self._free.popitem(last=False)
            h = self._block_hash.pop(b, None)            # evict a cached block
            if h is not None and self._hash_to_block.get(h) == b:
                del self._hash_to_block[h]
            self.ref[b] = 1
            out.append(b)
        return out

    def free(self, blocks: list[int]) -> None:
        # free in reverse so the tail of a sequence is evicted before its prefix
        for b in reversed(blocks):
            if b == 0:
                continue
            self.ref[b] -= 1
            assert self.ref[b] >= 0, f"double free of block {b}"
            if self.ref[b] == 0:
                self._free[b] = None

    def touch(self, blocks: list[int]) -> None:
        for b in blocks:
            if self.ref[b] == 0:
                self._free.pop(b, None)
            self.ref[b] += 1

    # ------------------------------------------------------------------ prefix cache
    @staticmethod
    def request_key_extra(req, store_fingerprint: bytes = b"") -> Optional[bytes]:
        """Everything besides the token ids that decides what a request's KV blocks hold: the
        adapter, the content hash of every multimodal item (equal placeholder ids, other pixels or
        audio) and, for stores shared between engines, a fingerprint of the model and the cache
        layout.  One helper for the scheduler's prefix cache and every connector, so that they can
        never disagree.  ``None``: the request's blocks must not be shared at all (caller-supplied
        embeddings have placeholder ids and no content hash)."""
        extra = store_fingerprint
        if req.lora_request is not None:
            extra += f"lora{req.lora_request.lora_int_id}".encode()
        for it in getattr(req, "mm_inputs", None) or ():
            if getattr(it, "modality", "") == "embeds" or not getattr(it, "hash", None) \
                    or str(it.hash).startswith("embeds-"):
                return None
            extra += b"mm" + str(it.hash).encode()
        return extra

    @staticmethod
    def store_fingerprint(engine_cfg, tensors) -> bytes:
        """Identity of what a KV block of this engine means: architecture and shape of the model, its
        weights' origin, and the cache tensors' dtype / per-block shape (which carry the TP sharding)."""
        m = engine_cfg.model
        desc = [m.architecture, m.name, str(m.model_path), m.num_hidden_layers, m.hidden_size,
                m.num_attention_heads, m.num_key_value_heads, m.head_dim, m.vocab_size, m.seed,
                str(m.quantization), engine_cfg.cache.block_size]
        for t in tensors:
            desc.append((str(t.dtype), tuple(t.shape[1:])))
        return hashlib.blake2b(repr(desc).encode(), digest_size=8).digest()

    @staticmethod
    def hash_block(parent: Optional[bytes], tokens: np.ndarray, extra: bytes = b"") -> bytes:
        h = hashlib.blake2b(digest_size=16)
        if parent:
            h.update(parent)
        h.update(np.ascontiguousarray(tokens, dtype=np.int32).tobytes())
        h.update(extra)
        return h.digest()

    def block_hashes(self, token_ids: np.ndarray, extra: bytes = b"") -> list[bytes]:
        out, parent = [], None
        bs = self.block_size
        for i in range(len(token_ids) // bs):
            parent = self.hash_block(parent, token_ids[i * bs:(i + 1) * bs], extra)
            out.append(parent)
        return out

    def find_cached_prefix(self, hashes: list[bytes]) -> list[int]:
        """Longest run of cached blocks matching the hash chain (not yet referenced)."""
        if not self.enable_prefix_caching:
            return []
        out = []
        for h in hashes:
            b = self._hash_to_block.get(h)
            if b is None:
                break
            out.append(b)
        self.queries += len(hashes)
        self.hits += len(out)
        return out

    def cache_full_blocks(self, blocks: list[int], hashes: list[bytes], num_full: int) -> None:
        if not self.enable_prefix_caching:
            return
        for i in range(min(num_full, len(hashes), len(blocks))):
            b, h = blocks[i], hashes[i]
            if b in self._block_hash:
                continue
            if h not in self._hash_to_block:
                self._hash_to_block[h] = b
                self._block_hash[b] = h

    def reset_prefix_cache(self) -> bool:
        self._hash_to_block.clear()
        self._block_hash.clear()
        return True
