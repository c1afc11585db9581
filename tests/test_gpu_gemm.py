"""tcgen05 bf16 GEMM vs fp32 matmul."""
import pytest
import torch

from vllm_ascend_b200 import _native, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check(M, N, K, bn=0, bias=False, residual=False, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.5).bfloat16().to(DEV)
    b = torch.randn(N, generator=g).bfloat16().to(DEV) if bias else None
    r = torch.randn(M, N, generator=g).bfloat16().to(DEV) if residual else None
    out = ops.linear(a, w, b, r, bn=bn)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    exp = a.float() @ w.float().t()
    if bias:
        exp += b.float()
    if residual:
        exp += r.float()
    err = (out.float() - exp).abs().max().item()
    tol = 0.02 * (K ** 0.5) * 0.25 + 0.05
    assert err < tol, f"M={M} N={N} K={K} bn={bn}: max abs err {err} (tol {tol})"


@pytest.mark.parametrize("bn", [128, 256, 512])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (256, 512, 4096),
                                   (1, 256, 128), (77, 1024, 1024), (1000, 768, 2048),
                                   (4096, 6144, 4096), (300, 768, 288), (64, 256, 3424)])
def test_gemm_shapes(M, N, K, bn):
    _check(M, N, K, bn)


def test_gemm_ragged_n_and_k_tail():
    _check(130, 136, 72)         # N % 128 != 0, K % 64 != 0
    _check(64, 151936 // 8 * 8 // 64 * 8, 256)
    _check(33, 8, 8)


def test_gemm_epilogue_bias_residual():
    _check(300, 512, 1024, bias=True)
    _check(300, 512, 1024, residual=True)
    _check(300, 512, 1024, bias=True, residual=True)


def test_gemm_auto_tile_many_waves():
    _check(8192, 4096, 4096)
    _check(1024, 12288, 4096)


def test_gemm_strided_input():
    a_full = (torch.randn(256, 2048) * 0.5).bfloat16().to(DEV)
    a = a_full[:, 512:1536]
    w = (torch.randn(384, 1024) * 0.5).bfloat16().to(DEV)
    out = ops.linear(a, w)
    exp = a.float() @ w.float().t()
    assert (out.float() - exp).abs().max().item() < 0.5


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 768, 2048), (1024, 12288, 4096), (5, 256, 512)])
def test_gemm_swiglu_epilogue(M, I, K):
    g = torch.Generator(device="cpu").manual_seed(3)
    a = (torch.randn(M, K, generator=g) * 0.3).bfloat16().to(DEV)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).bfloat16().to(DEV)
    out = ops.linear_swiglu(a, w)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    h = a.float() @ w.float().t()
    exp = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
    assert (out.float() - exp).abs().max().item() < 0.02 * exp.abs().max().item() + 0.02


@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_gemm(swiglu):
    torch.manual_seed(4)
    E, K, N = 8, 512, 256
    counts = [0, 5, 128, 300, 1, 0, 77, 129]
    offs = torch.tensor([0] + list(__import__("itertools").accumulate(counts)), dtype=torch.int32, device=DEV)
    total = int(offs[-1])
    a = (torch.randn(total, K, device=DEV) * 0.3).bfloat16()
    wrows = 2 * N if swiglu else N
    w = (torch.randn(E, wrows, K, device=DEV) * 0.1).bfloat16()
    out = torch.full((total, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    rc = _native.lib().b200_grouped_gemm_bf16(a.data_ptr(), w.data_ptr(), out.data_ptr(), offs.data_ptr(),
                                              E, total, N, K, K, K, N, int(swiglu),
                                              _native.status_word(torch.device(DEV)).data_ptr(),
                                              _native.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    for e in range(E):
        lo, hi = int(offs[e]), int(offs[e + 1])
        if hi == lo:
            continue
        h = a[lo:hi].float() @ w[e].float().t()
        exp = torch.nn.functional.silu(h[:, :N]) * h[:, N:] if swiglu else h
        assert (out[lo:hi].float() - exp).abs().max().item() < 0.05, e


def test_gemm_2cta_ragged_and_epilogues():
    _check(130, 136, 72, bn=512)
    _check(300, 512, 1024, bn=512, bias=True, residual=True)
    _check(8192, 4096, 4096, bn=512)
    _check(1000, 12288, 512, bn=512)


@pytest.mark.parametrize("M,I,K", [(256, 128, 64), (300, 768, 2048), (1024, 12288, 4096), (5, 256, 512)])
def test_gemm_2cta_swiglu(M, I, K):
    g = torch.Generator(device="cpu").manual_seed(5)
    a = (torch.randn(M, K, generator=g) * 0.3).bfloat16().to(DEV)
    w = (torch.randn(2 * I, K, generator=g) * 0.1).bfloat16().to(DEV)
    out = ops.linear_swiglu(a, w, two_cta=True)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    h = a.float() @ w.float().t()
    exp = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
    assert (out.float() - exp).abs().max().item() < 0.02 * exp.abs().max().item() + 0.02


@pytest.mark.parametrize("width", [128, 144, 160, 176, 192, 208, 224, 240, 256])
def test_gemm_2cta_every_tile_width(width):
    """The paired-CTA kernel picks its tile width (128..256 columns) per problem so that the tiles fill
    whole waves of CTA pairs; every width is forced here on shapes with ragged last tiles in M and N,
    with bias and residual, and on the decode shape that motivated it (768 x 4096)."""
    import ctypes
    lib = _native.lib()
    _native.register_signature("b200_gemm_2cta_set_bn", [ctypes.c_int])
    assert lib.b200_gemm_2cta_set_bn(width) == 0
    try:
        _check(768, 4096, 4096, bn=512)
        _check(300, 520, 1024, bn=512, bias=True, residual=True, seed=3)
        _check(1000, 776, 512, bn=512, seed=4)
        _check(130, 136, 72, bn=512, seed=5)
    finally:
        lib.b200_gemm_2cta_set_bn(0)


def test_gemm_2cta_chooses_narrow_tiles_for_few_tiles():
    # automatic choice: same answers as the fixed widths on the shapes where it departs from 256
    for M, N, K in ((768, 4096, 4096), (1024, 3072, 4096), (512, 6144, 4096), (8192, 768, 4096)):
        _check(M, N, K, bn=512, seed=M)
