"""``torch.ops.b200.*``: the kernels as dispatcher ops with schemas and meta (shape) functions.

The kernels are exported with a C ABI and called through ctypes; that is the cheapest call path for
this package's own runner.  Code that addresses ops by schema (a host engine's graph capture or
tracing machinery, ``torch.compile`` users, ``FakeTensorMode`` shape propagation) needs dispatcher
ops instead: this module defines them in the ``b200`` namespace, implements each for CUDA and CPU by
calling the functions of ``vllm_ascend_b200.ops`` (the CPU key runs the PyTorch definitions), and
registers a meta function that allocates outputs of the right shape and dtype without touching data.

The reference registers its kernels the same way in C++ (csrc/torch_binding.cpp:1898-2569, namespace
``_C_ascend``) with the meta functions in csrc/torch_binding_meta.cpp:1480-1578 and
vllm_ascend/meta_registration.py.

``register()`` is idempotent and is called when the package is imported as a plugin.
"""
from __future__ import annotations

from typing import Optional

import torch

_LIB: Optional[torch.library.Library] = None
NAMESPACE = "b200"

# name -> schema.  Ops that write in place name the mutated argument with (a!).
SCHEMAS = {
    "rms_norm": "(Tensor x, Tensor weight, float eps) -> Tensor",
    "add_rms_norm": "(Tensor x, Tensor residual, Tensor weight, float eps) -> (Tensor, Tensor)",
    "layer_norm": "(Tensor x, Tensor weight, Tensor? bias, float eps) -> Tensor",
    "rms_norm_gated": "(Tensor x, Tensor z, Tensor weight, float eps, int group, bool norm_before_gate) -> Tensor",
    "silu_and_mul": "(Tensor x, float limit) -> Tensor",
    "linear": "(Tensor x, Tensor weight, Tensor? bias, Tensor? residual) -> Tensor",
    "linear_swiglu": "(Tensor x, Tensor weight) -> Tensor",
    "embedding": "(Tensor ids, Tensor weight, int vocab_start, int vocab_end) -> Tensor",
    "quant_fp8_group128": "(Tensor x, bool pow2_scale) -> (Tensor, Tensor)",
    "quant_fp8_per_token": "(Tensor x) -> (Tensor, Tensor)",
    "argmax": "(Tensor logits) -> Tensor",
    "paged_attention": "(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_table, Tensor seq_lens, "
                       "Tensor query_start_loc, int max_query_len, int max_seq_len, float scale, bool causal, "
                       "int window) -> Tensor",
    "qknorm_rope_kvwrite_": "(Tensor(a!) qkv, Tensor positions, Tensor cos_sin, Tensor? q_weight, Tensor? k_weight, "
                            "float eps, Tensor(b!) k_cache, Tensor(c!) v_cache, Tensor slot_mapping, int num_heads, "
                            "int num_kv_heads, int head_dim) -> ()",
    "slot_mapping": "(Tensor block_table, Tensor req_idx, Tensor positions, int block_size, int num_blocks) -> Tensor",
    "expand_block_table": "(Tensor block_table, int ratio) -> Tensor",
    "bincount": "(Tensor ids, Tensor? rows, int num_rows, int vocab) -> Tensor",
    "scatter_nd_update_": "(Tensor(a!) var, Tensor indices, Tensor updates) -> ()",
    "sign_bits_pack": "(Tensor x) -> Tensor",
    "sign_bits_unpack": "(Tensor packed, int n, float scale, ScalarType dtype) -> Tensor",
    "swap_blocks_": "(Tensor src, Tensor(a!) dst, Tensor src_to_dst) -> ()",
}


# ---------------------------------------------------------------------------- implementations
def _impls():
    from .. import ops
    from . import bookkeeping as bk

    def rms_norm(x, weight, eps):
        return ops.rms_norm(x, weight, eps)[0]

    def add_rms_norm(x, residual, weight, eps):
        y, r = ops.rms_norm(x, weight, eps, residual=residual)
        return y, r

    def layer_norm(x, weight, bias, eps):
        return ops.layer_norm(x, weight, bias, eps)

    def rms_norm_gated(x, z, weight, eps, group, norm_before_gate):
        return ops.rms_norm_gated(x, z, weight, eps, group, norm_before_gate)

    def silu_and_mul(x, limit):
        return ops.silu_and_mul(x, limit)

    def linear(x, weight, bias, residual):
        return ops.linear(x, weight, bias, residual)

    def linear_swiglu(x, weight):
        return ops.linear_swiglu(x, weight)

    def embedding(ids, weight, vocab_start, vocab_end):
        return ops.embedding(ids, weight, vocab_start, vocab_end)

    def quant_fp8_group128(x, pow2_scale):
        q, s = ops.quant_fp8_group128(x, pow2_scale)
        return q, s

    def quant_fp8_per_token(x):
        q, s = ops.quant_fp8_per_token(x)
        return q, s

    def argmax(logits):
        return ops.argmax(logits).to(torch.int64)

    def paged_attention(q, k_cache, v_cache, block_table, seq_lens, query_start_loc, max_query_len, max_seq_len,
                        scale, causal, window):
        from .. import envs
        from ..attention.metadata import metadata_from_tensors
        meta = metadata_from_tensors(query_start_loc, seq_lens, block_table, max_query_len, max_seq_len, q.shape[1],
                                     k_cache.shape[2], q.shape[2],
                                     decode_kernel=envs.VLLM_B200_DECODE_ATTN == "native")
        return ops.paged_attention(q, k_cache, v_cache, meta, scale, None, causal, window)

    def qknorm_rope_kvwrite_(qkv, positions, cos_sin, q_weight, k_weight, eps, k_cache, v_cache, slot_mapping,
                             num_heads, num_kv_heads, head_dim):
        ops.qknorm_rope_kvwrite(qkv, positions, cos_sin, cos_sin.shape[-1], q_weight, k_weight, eps, k_cache, v_cache,
                                slot_mapping, num_heads, num_kv_heads, head_dim)

    def slot_mapping(block_table, req_idx, positions, block_size, num_blocks):
        return bk.slot_mapping(block_table, req_idx, positions, block_size, num_blocks)

    def expand_block_table(block_table, ratio):
        return bk.expand_block_table(block_table, ratio)

    def bincount(ids, rows, num_rows, vocab):
        return bk.bincount(ids, rows, num_rows, vocab)

    def scatter_nd_update_(var, indices, updates):
        bk.scatter_nd_update(var, indices, updates)

    def sign_bits_pack(x):
        return bk.sign_bits_pack(x)

    def sign_bits_unpack(packed, n, scale, dtype):
        return bk.sign_bits_unpack(packed, n, scale, dtype)

    def swap_blocks_(src, dst, src_to_dst):
        from ..attention.backend import B200AttentionBackend
        B200AttentionBackend.swap_blocks(src, dst, src_to_dst)

    return {k: v for k, v in locals().items() if k in SCHEMAS}


# ---------------------------------------------------------------------------- meta functions
def _metas():
    def like(x, shape=None, dtype=None):
        return x.new_empty(tuple(x.shape) if shape is None else tuple(shape), dtype=dtype or x.dtype)

    def rms_norm(x, weight, eps):
        return like(x)

    def add_rms_norm(x, residual, weight, eps):
        return like(x), like(x)

    def layer_norm(x, weight, bias, eps):
        return like(x)

    def rms_norm_gated(x, z, weight, eps, group, norm_before_gate):
        return like(x)

    def silu_and_mul(x, limit):
        return like(x, (*x.shape[:-1], x.shape[-1] // 2))

    def linear(x, weight, bias, residual):
        return like(x, (*x.shape[:-1], weight.shape[0]))

    def linear_swiglu(x, weight):
        return like(x, (*x.shape[:-1], weight.shape[0] // 2))

    def embedding(ids, weight, vocab_start, vocab_end):
        return like(weight, (*ids.shape, weight.shape[1]))

    def quant_fp8_group128(x, pow2_scale):
        return like(x, dtype=torch.float8_e4m3fn), like(x, (*x.shape[:-1], (x.shape[-1] + 127) // 128), torch.float32)

    def quant_fp8_per_token(x):
        return like(x, dtype=torch.float8_e4m3fn), like(x, x.shape[:-1], torch.float32)

    def argmax(logits):
        return like(logits, logits.shape[:-1], torch.int64)

    def paged_attention(q, k_cache, v_cache, block_table, seq_lens, query_start_loc, max_query_len, max_seq_len,
                        scale, causal, window):
        return like(q, (q.shape[0], q.shape[1], v_cache.shape[-1]))

    def qknorm_rope_kvwrite_(*a):
        return None

    def slot_mapping(block_table, req_idx, positions, block_size, num_blocks):
        return like(req_idx, dtype=torch.int64)

    def expand_block_table(block_table, ratio):
        return like(block_table, (block_table.shape[0], block_table.shape[1] * ratio))

    def bincount(ids, rows, num_rows, vocab):
        return like(ids, (num_rows, vocab), torch.int32)

    def scatter_nd_update_(var, indices, updates):
        return None

    def sign_bits_pack(x):
        return like(x, ((x.numel() + 7) // 8,), torch.uint8)

    def sign_bits_unpack(packed, n, scale, dtype):
        return like(packed, (n,), dtype)

    def swap_blocks_(src, dst, src_to_dst):
        return None

    return {k: v for k, v in locals().items() if k in SCHEMAS}


def register() -> list[str]:
    """Define the ops (once per process); returns their qualified names."""
    global _LIB
    names = [f"{NAMESPACE}::{n}" for n in SCHEMAS]
    if _LIB is not None:
        return names
    lib = torch.library.Library(NAMESPACE, "DEF")
    impls, metas = _impls(), _metas()
    for name, schema in SCHEMAS.items():
        lib.define(name + schema)
        lib.impl(name, impls[name], "CUDA")
        lib.impl(name, impls[name], "CPU")
        lib.impl(name, metas[name], "Meta")
    _LIB = lib
    return names
