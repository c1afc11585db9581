"""The allocation-free decode entry point must agree with the regular one.

Some callers of the native library cannot allocate device memory when they call it
(they run inside a fixed memory pool, or in a host process that owns the allocator),
so ``b200_paged_decode_noalloc`` keeps the split-KV partials in an array that is part
of the library.  The test calls it through its exported C symbol, twice in a row with
different inputs (the array keeps the first call's contents), and compares each
result with ``b200_paged_decode`` working on a caller-provided scratch buffer.
"""
import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

from vllm_ascend_b200 import _native
from gpu_utils import make_paged_case

pytestmark = pytest.mark.gpu
TOO_LARGE = 9200


def _lib():
    lib = _native.lib()
    fn = lib.b200_paged_decode_noalloc
    fn.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                   c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_long, c_long, c_void_p,
                   c_void_p]
    fn.restype = c_int
    lib.b200_paged_decode_noalloc_bytes.argtypes = [c_int, c_int, c_int, c_int]
    lib.b200_paged_decode_noalloc_bytes.restype = c_long
    return lib


def _both(lib, ctx, Hq, Hkv, D, bs, splits, seed):
    q, kc, vc, meta = make_paged_case([1] * len(ctx), ctx, Hq, Hkv, D, bs, seed=seed, layout="NHD")
    B = len(ctx)
    scale = D ** -0.5
    NB = kc.shape[0]
    status = _native.status_word(q.device)
    stream = _native.stream_ptr()
    ref = torch.full_like(q, float("nan"))
    scratch = torch.empty(max(1, B * Hq * splits * (D + 1) * 4), dtype=torch.uint8, device=q.device)
    rc = lib.b200_paged_decode(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                               meta.block_table.data_ptr(), meta.block_table.stride(0),
                               meta.seq_lens.data_ptr(), B, Hq, Hkv, D, bs, scale, 0, splits,
                               ref.data_ptr(), ref.stride(0), scratch.data_ptr(), NB,
                               status.data_ptr(), stream)
    assert rc == 0
    out = torch.full_like(q, float("nan"))
    rc = lib.b200_paged_decode_noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                       meta.block_table.data_ptr(), meta.block_table.stride(0),
                                       meta.seq_lens.data_ptr(), B, Hq, Hkv, D, bs, scale, 0,
                                       splits, out.data_ptr(), out.stride(0), NB,
                                       status.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    _native.check_status(q.device)
    # plain fp32 attention over the same pages, independent of both entry points
    kf, vf = kc.float(), vc.float()
    want = torch.zeros_like(q, dtype=torch.float32)
    for b in range(B):
        n = int(meta.seq_lens[b])
        blocks = meta.block_table[b, :(n + bs - 1) // bs].long()
        k = kf[blocks].reshape(-1, Hkv, D)[:n]
        v = vf[blocks].reshape(-1, Hkv, D)[:n]
        G = Hq // Hkv
        for h in range(Hq):
            s = (k[:, h // G] @ q[b, h].float()) * scale
            want[b, h] = torch.softmax(s, dim=0) @ v[:, h // G]
    return out.float(), ref.float(), want


def test_no_alloc_decode_matches_regular_entry_point_on_two_calls_in_a_row():
    lib = _lib()
    # first call fills the built-in array; the second, with other shapes and data, must not
    # be disturbed by what the first one left there
    out1, ref1, want1 = _both(lib, [700, 33, 1500, 128, 2047], 32, 8, 128, 128, splits=4, seed=21)
    out2, ref2, want2 = _both(lib, [90, 3000, 5], 8, 2, 64, 16, splits=3, seed=22)
    # same kernel, same split count, only the home of the partials differs: bit-identical
    assert torch.equal(out1, ref1)
    assert torch.equal(out2, ref2)
    # and both are right: within bf16 output rounding of fp32 attention
    assert (out1 - want1).abs().max().item() < 2e-2
    assert (out2 - want2).abs().max().item() < 2e-2
    assert torch.isfinite(out1).all() and torch.isfinite(out2).all()


def test_no_alloc_decode_rejects_sizes_beyond_the_builtin_scratch():
    lib = _lib()
    q, kc, vc, meta = make_paged_case([1] * 4, [10] * 4, 32, 8, 128, 128, seed=1, layout="NHD")
    assert lib.b200_paged_decode_noalloc_bytes(4096, 32, 128, 16) > (8 << 20)
    out = torch.empty_like(q)
    rc = lib.b200_paged_decode_noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                       meta.block_table.data_ptr(), meta.block_table.stride(0),
                                       meta.seq_lens.data_ptr(), 4096, 32, 8, 128, 128, 0.1, 0, 16,
                                       out.data_ptr(), out.stride(0), kc.shape[0], None,
                                       _native.stream_ptr())
    assert rc == TOO_LARGE
