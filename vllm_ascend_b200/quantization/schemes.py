"""Quantization schemes.

FP8_BLOCK      128x128 block-scaled e4m3 weights x 1x128 per-token-group e4m3 activations
               (DeepSeek-V3 / ``quant_method: fp8`` checkpoints load as they are;
               vllm_ascend/quantization/methods/fp8.py:32-92).  GPU: tcgen05 f8f6f4 kernel
               with two-level accumulation (csrc/gemm_fp8_block.cu).
W8A8_DYNAMIC   per-output-channel weight scale x per-token dynamic activation scale, int8
               (vllm_ascend/quantization/methods/w8a8_dynamic.py:51-399)
W8A8FP8_DYNAMIC same with e4m3 (methods/w8a8fp8_dynamic.py:27-103)
W8A8           static per-tensor activation scale (methods/w8a8_static.py:32-141)
W4A16 / W8A16  weight-only, group-wise scales
FLOAT          unquantized pass-through (a layer the description lists as "FLOAT")
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native, ops
from ..ops import reference as ref
from .registry import register_scheme

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def quantize_weight_block_fp8(w: torch.Tensor, block=(128, 128)):
    """bf16/fp32 [N, K] -> (e4m3 [N, K], scale_inv fp32 [ceil(N/bn), ceil(K/bk)])."""
    N, K = w.shape
    bn, bk = block
    nb, kb = (N + bn - 1) // bn, (K + bk - 1) // bk
    wp = torch.zeros(nb * bn, kb * bk, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, bn, kb, bk)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.view(nb * bn, kb * bk)[:N, :K].contiguous(), scale.contiguous()


class LinearScheme:
    """Interface of a linear-layer scheme."""
    def convert(self, layer) -> None:            # build quantized tensors from layer.weight
        raise NotImplementedError

    def apply(self, layer, x, residual=None, skip_bias=False):
        raise NotImplementedError

    def named_tensors(self, layer):
        return iter(())


@register_scheme("FLOAT", "linear")
class FloatLinear(LinearScheme):
    def convert(self, layer) -> None:
        pass

    def apply(self, layer, x, residual=None, skip_bias=False):
        return ops.linear(x, layer.weight, None if skip_bias else layer.bias, residual)


@register_scheme("FP8_BLOCK", "linear")
class Fp8BlockLinear(LinearScheme):
    block = (128, 128)

    def convert(self, layer) -> None:
        if layer.weight.dtype != FP8:
            q, s = quantize_weight_block_fp8(layer.weight, self.block)
            layer.weight = q
            layer.weight_scale_inv = s
        elif not hasattr(layer, "weight_scale_inv"):
            N, K = layer.weight.shape
            layer.weight_scale_inv = torch.ones((N + 127) // 128, (K + 127) // 128,
                                                dtype=torch.float32, device=layer.weight.device)

    def named_tensors(self, layer):
        yield "weight_scale_inv", layer.weight_scale_inv

    accepts_quant_act = True       # a fused norm / activation kernel may hand over fp8 directly

    def apply(self, layer, x, residual=None, skip_bias=False):
        bias = None if skip_bias else layer.bias
        if isinstance(x, ops.QuantAct):
            N = layer.weight.shape[0]
            if x.q.is_cuda and N % 8 == 0:
                y = fp8_block_linear(None, layer.weight, layer.weight_scale_inv, bias, quant=(x.q, x.scales))
            else:
                y = ref.block_fp8_linear(x.dequant(), layer.weight, layer.weight_scale_inv, self.block, x.dtype)
                if bias is not None:
                    y = y + bias
            return y + residual if residual is not None else y
        K = x.shape[-1]
        N = layer.weight.shape[0]
        x2 = x.reshape(-1, K)
        if x2.is_cuda and x2.dtype == torch.bfloat16 and K % 128 == 0 and N % 8 == 0:
            y = fp8_block_linear(x2, layer.weight, layer.weight_scale_inv, bias)
        else:
            y = ref.block_fp8_linear(x2, layer.weight, layer.weight_scale_inv, self.block, x.dtype)
            if bias is not None:
                y = y + bias
        y = y.view(*x.shape[:-1], N)
        if residual is not None:
            y = y + residual
        return y




def _declare_native():
    from ctypes import c_int, c_long, c_void_p
    P, I, L = c_void_p, c_int, c_long
    _native.register_signature("b200_gemm_fp8_block", [P, P, P, P, P, P, I, I, I, I, I, I, P, P])
    _native.register_signature("b200_grouped_gemm_fp8_block",
                               [P, P, P, P, P, P, I, L, I, I, I, I, I, P, P])
    _native.register_signature("b200_gemm_fp8_channel", [P, P, P, P, P, P, I, I, I, I, I, I, P, P])
    _native.register_signature("b200_grouped_gemm_fp8_channel",
                               [P, P, P, P, P, P, I, L, I, I, I, I, I, P, P])


_declare_native()


def fp8_block_linear(x: Optional[torch.Tensor], w8: torch.Tensor, w_scale: torch.Tensor,
                     bias: Optional[torch.Tensor] = None, quant: Optional[tuple] = None) -> torch.Tensor:
    """bf16 activations [M,K] -> dynamic 1x128 e4m3 quantisation -> block-scaled GEMM."""
    if quant is not None:
        xq, xs = quant
    else:
        xq, xs = ops.quant_fp8_group128(x if x.is_contiguous() else x.contiguous())
    M, K = xq.shape
    N = w8.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    if M == 0:
        return out
    rc = _native.lib().b200_gemm_fp8_block(
        xq.data_ptr(), xs.data_ptr(), w8.data_ptr(), w_scale.data_ptr(), out.data_ptr(),
        _native.ptr(bias), M, N, K, xq.stride(0), w8.stride(0), out.stride(0),
        _native.status_word(xq.device).data_ptr(), _native.stream_ptr())
    _native.check(rc, "gemm_fp8_block")
    ops.launch_counter[0] += 1
    return out


def fp8_channel_linear(x: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                       bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 activations [M, K] -> dynamic per-token e4m3 quantisation -> tcgen05 GEMM whose epilogue
    applies row scale x column scale.  w8 [N, K] e4m3, w_scale [N] fp32."""
    xq, xs = ops.quant_fp8_per_token(x)
    M, K = xq.shape
    N = w8.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    if M == 0:
        return out
    rc = _native.lib().b200_gemm_fp8_channel(
        xq.data_ptr(), xs.data_ptr(), w8.data_ptr(), w_scale.data_ptr(), out.data_ptr(), _native.ptr(bias),
        M, N, K, xq.stride(0), w8.stride(0), out.stride(0), _native.status_word(xq.device).data_ptr(),
        _native.stream_ptr())
    _native.check(rc, "gemm_fp8_channel")
    ops.launch_counter[0] += 1
    return out


def grouped_fp8_channel(a8: torch.Tensor, a_scale: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                        offsets: torch.Tensor) -> torch.Tensor:
    """Rows of a8 grouped by expert (offsets [E + 1] int32); w8 [E, N, K] e4m3, w_scale [E, N] fp32."""
    rows, K = a8.shape
    E, N = w8.shape[0], w8.shape[1]
    out = torch.empty((rows, N), dtype=torch.bfloat16, device=a8.device)
    rc = _native.lib().b200_grouped_gemm_fp8_channel(
        a8.data_ptr(), a_scale.data_ptr(), w8.data_ptr(), w_scale.data_ptr(), out.data_ptr(), offsets.data_ptr(),
        E, rows, N, K, a8.stride(0), w8.stride(1), out.stride(0), _native.status_word(a8.device).data_ptr(),
        _native.stream_ptr())
    _native.check(rc, "grouped_gemm_fp8_channel")
    ops.launch_counter[0] += 1
    return out


class _PerChannelDynamic(LinearScheme):
    """Per-token dynamic activations x per-output-channel weights."""
    qdtype = torch.int8
    qmax = 127.0

    def _q(self, t: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        v = t.float() / scale
        if self.qdtype == torch.int8:
            return v.round().clamp(-self.qmax, self.qmax).to(torch.int8)
        return v.clamp(-self.qmax, self.qmax).to(self.qdtype)

    def convert(self, layer) -> None:
        if layer.weight.dtype in (torch.int8, FP8):
            if not hasattr(layer, "weight_scale"):
                layer.weight_scale = torch.ones(layer.weight.shape[0], 1, dtype=torch.float32,
                                                device=layer.weight.device)
            return
        w = layer.weight.float()
        scale = (w.abs().amax(dim=1, keepdim=True) / self.qmax).clamp_min(1e-10)
        layer.weight = self._q(w, scale)
        layer.weight_scale = scale

    def named_tensors(self, layer):
        yield "weight_scale", layer.weight_scale

    def apply(self, layer, x, residual=None, skip_bias=False):
        K = x.shape[-1]
        x2 = x.reshape(-1, K).float()
        a_scale = (x2.abs().amax(dim=1, keepdim=True) / self.qmax).clamp_min(1e-10)
        xq = self._q(x2, a_scale).float()
        y = (xq @ layer.weight.float().t()) * a_scale * layer.weight_scale.view(1, -1)
        if layer.bias is not None and not skip_bias:
            y = y + layer.bias.float()
        y = y.to(x.dtype).view(*x.shape[:-1], layer.weight.shape[0])
        return y + residual if residual is not None else y


@register_scheme("W8A8_DYNAMIC", "linear")
class W8A8DynamicLinear(_PerChannelDynamic):
    pass


@register_scheme("W8A8FP8_DYNAMIC", "linear")
class W8A8Fp8DynamicLinear(_PerChannelDynamic):
    """e4m3 weights with one scale per output channel, activations quantised per token at run
    time; on the GPU both steps are native (per-token quant kernel, tcgen05 GEMM with the scale
    product in its epilogue)."""
    qdtype = FP8
    qmax = FP8_MAX

    def apply(self, layer, x, residual=None, skip_bias=False):
        K, N = x.shape[-1], layer.weight.shape[0]
        if not (x.is_cuda and x.dtype == torch.bfloat16 and layer.weight.dtype == FP8 and K % 128 == 0
                and N % 8 == 0):
            return super().apply(layer, x, residual, skip_bias)
        ws = getattr(layer, "_ws_flat", None)
        if ws is None or ws.data_ptr() != layer.weight_scale.data_ptr():
            ws = layer._ws_flat = layer.weight_scale.view(-1)
            if not ws.is_contiguous() or ws.dtype != torch.float32:
                ws = layer._ws_flat = ws.float().contiguous()
        y = fp8_channel_linear(x.reshape(-1, K), layer.weight, ws, None if skip_bias else layer.bias)
        y = y.view(*x.shape[:-1], N)
        return y + residual if residual is not None else y


@register_scheme("W8A8", "linear")
class W8A8StaticLinear(_PerChannelDynamic):
    """Static per-tensor activation scale (``input_scale``) instead of per-token."""

    def convert(self, layer) -> None:
        super().convert(layer)
        if not hasattr(layer, "input_scale"):
            layer.input_scale = torch.tensor(1.0 / 16, dtype=torch.float32, device=layer.weight.device)

    def named_tensors(self, layer):
        yield "weight_scale", layer.weight_scale
        yield "input_scale", layer.input_scale

    def apply(self, layer, x, residual=None, skip_bias=False):
        K = x.shape[-1]
        x2 = x.reshape(-1, K).float()
        xq = self._q(x2, layer.input_scale).float()
        y = (xq @ layer.weight.float().t()) * layer.input_scale * layer.weight_scale.view(1, -1)
        if layer.bias is not None and not skip_bias:
            y = y + layer.bias.float()
        y = y.to(x.dtype).view(*x.shape[:-1], layer.weight.shape[0])
        return y + residual if residual is not None else y


class _WeightOnly(LinearScheme):
    bits = 8
    group = 128

    def convert(self, layer) -> None:
        if hasattr(layer, "weight_scale"):
            return
        w = layer.weight.float()
        N, K = w.shape
        g = self.group if K % self.group == 0 else K
        qmax = float(2 ** (self.bits - 1) - 1)
        wg = w.view(N, K // g, g)
        scale = (wg.abs().amax(dim=-1, keepdim=True) / qmax).clamp_min(1e-10)
        layer.weight = (wg / scale).round().clamp(-qmax, qmax).to(torch.int8).view(N, K)
        layer.weight_scale = scale.squeeze(-1)
        layer.group_size = g

    def named_tensors(self, layer):
        yield "weight_scale", layer.weight_scale

    def apply(self, layer, x, residual=None, skip_bias=False):
        N, K = layer.weight.shape
        g = layer.group_size
        w = (layer.weight.float().view(N, K // g, g) * layer.weight_scale.unsqueeze(-1)).view(N, K)
        return ops.linear(x, w.to(x.dtype), None if skip_bias else layer.bias, residual)


@register_scheme("W8A16", "linear")
class W8A16Linear(_WeightOnly):
    bits = 8


@register_scheme("W4A16", "linear")
class W4A16Linear(_WeightOnly):
    bits = 4


# ---------------------------------------------------------------- MoE schemes
class MoEScheme:
    def convert(self, block) -> None:
        raise NotImplementedError

    def apply_experts(self, x, w13, w2, topk_w, topk_ids, expert_map):
        raise NotImplementedError


@register_scheme("FP8_BLOCK", "moe")
class Fp8BlockMoE(MoEScheme):
    """Expert weights as block-scaled e4m3; grouped GEMM1 -> SwiGLU -> 1x128 requant -> GEMM2."""

    def convert(self, block) -> None:
        if block.w13.dtype == FP8:
            return
        q13, s13, q2, s2 = [], [], [], []
        for e in range(block.w13.shape[0]):
            q, s = quantize_weight_block_fp8(block.w13[e])
            q13.append(q); s13.append(s)
            q, s = quantize_weight_block_fp8(block.w2[e])
            q2.append(q); s2.append(s)
        block.w13, block.w13_scale = torch.stack(q13), torch.stack(s13)
        block.w2, block.w2_scale = torch.stack(q2), torch.stack(s2)
        self.block_ref = block

    def apply_experts(self, x, w13, w2, topk_w, topk_ids, expert_map):
        from ..ops import moe_native
        blk = self.block_ref
        if x.is_cuda and x.dtype == torch.bfloat16 and moe_native.available():
            return moe_native.fused_experts_fp8(x, w13, blk.w13_scale, w2, blk.w2_scale, topk_w,
                                                topk_ids, expert_map)
        # reference: dequantise per expert
        T, H = x.shape
        out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        ids = topk_ids.long()
        if expert_map is not None:
            ids = expert_map.long()[ids]
        for e in range(w13.shape[0]):
            tok, slot = (ids == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            h = ref.block_fp8_linear(x[tok], w13[e], blk.w13_scale[e], out_dtype=torch.float32)
            a = ref.silu_and_mul(h).to(x.dtype)
            y = ref.block_fp8_linear(a, w2[e], blk.w2_scale[e], out_dtype=torch.float32)
            out.index_add_(0, tok, y * topk_w[tok, slot].unsqueeze(-1).float())
        return out.to(x.dtype)


@register_scheme("W8A8_DYNAMIC", "moe")
class W8A8DynamicMoE(MoEScheme):
    def convert(self, block) -> None:
        def q(w):
            scale = (w.float().abs().amax(dim=-1, keepdim=True) / 127.0).clamp_min(1e-10)
            return (w.float() / scale).round().clamp(-127, 127).to(torch.int8), scale
        block.w13, block.w13_scale = q(block.w13)
        block.w2, block.w2_scale = q(block.w2)
        self.block_ref = block

    def apply_experts(self, x, w13, w2, topk_w, topk_ids, expert_map):
        from ..ops.fused_moe import fused_experts_ref
        blk = self.block_ref
        w13f = (w13.float() * blk.w13_scale).to(x.dtype)
        w2f = (w2.float() * blk.w2_scale).to(x.dtype)
        return fused_experts_ref(x, w13f, w2f, topk_w, topk_ids, expert_map)


@register_scheme("W8A8FP8_DYNAMIC", "moe")
class W8A8Fp8DynamicMoE(MoEScheme):
    """Experts in e4m3 with per-channel scales: permute -> per-token quant -> grouped GEMM1 ->
    SiLU-mul -> per-token quant -> grouped GEMM2 -> weighted combine."""

    def convert(self, block) -> None:
        def q(w):
            if w.dtype == FP8:
                return w, None
            scale = (w.float().abs().amax(dim=-1, keepdim=True) / FP8_MAX).clamp_min(1e-10)
            return (w.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8), scale.squeeze(-1).contiguous()
        w13, s13 = q(block.w13)
        w2, s2 = q(block.w2)
        block.w13, block.w2 = w13, w2
        if s13 is not None:
            block.w13_scale = s13                    # [E, 2I]
        if s2 is not None:
            block.w2_scale = s2                      # [E, H]
        self.block_ref = block

    def apply_experts(self, x, w13, w2, topk_w, topk_ids, expert_map):
        blk = self.block_ref
        E, two_i, H = w13.shape
        if x.is_cuda and x.dtype == torch.bfloat16 and H % 128 == 0 and (two_i // 2) % 128 == 0 and E <= 512 \
                and x.shape[0] > 0:
            from ..ops import moe_native
            perm = moe_native.Permutation(topk_ids, expert_map, E)
            xs = perm.gather(x)
            a8, a_s = ops.quant_fp8_per_token(xs)
            h = grouped_fp8_channel(a8, a_s, w13, blk.w13_scale, perm.offsets)
            a = ops.silu_and_mul(h)
            b8, b_s = ops.quant_fp8_per_token(a)
            y = grouped_fp8_channel(b8, b_s, w2, blk.w2_scale, perm.offsets)
            return perm.combine(y, topk_w)
        T = x.shape[0]
        out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        ids = topk_ids.long()
        if expert_map is not None:
            ids = expert_map.long()[ids]

        def lin(a, w, ws):
            q, s = ref.quant_fp8_per_token(a)
            return (q.float() @ w.float().t()) * s.unsqueeze(-1) * ws.view(1, -1)
        for e in range(E):
            tok, slot = (ids == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            h = lin(x[tok], w13[e], blk.w13_scale[e])
            a = ref.silu_and_mul(h).to(x.dtype)
            y = lin(a, w2[e], blk.w2_scale[e])
            out.index_add_(0, tok, y * topk_w[tok, slot].unsqueeze(-1).float())
        return out.to(x.dtype)


# ---------------------------------------------------------------- microscaling (MX) formats
def _e8m0_scale(amax: torch.Tensor, elem_max_pow2: int) -> torch.Tensor:
    """Power-of-two block scale of the OCP microscaling formats: 2^(floor(log2 amax) - emax_elem)."""
    e = torch.floor(torch.log2(amax.clamp_min(2.0 ** -126))) - elem_max_pow2
    return torch.exp2(e.clamp(-127, 127))


_FP4_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _round_fp4(v: torch.Tensor) -> torch.Tensor:
    """Round to the e2m1 grid (+-{0, .5, 1, 1.5, 2, 3, 4, 6}), saturating."""
    grid = _FP4_GRID.to(v.device)
    mag = v.abs().clamp(max=6.0)
    idx = (mag.unsqueeze(-1) - grid).abs().argmin(dim=-1)
    return grid[idx] * v.sign()


def mx_quantize(t: torch.Tensor, elem: str, block: int = 32):
    """[..., K] -> (values on the element grid as fp32, e8m0 scales [..., K / block]) with one
    power-of-two scale per ``block`` consecutive elements of the last dim."""
    K = t.shape[-1]
    assert K % block == 0, "the last dimension must be a multiple of the MX block"
    g = t.float().reshape(*t.shape[:-1], K // block, block)
    amax = g.abs().amax(dim=-1, keepdim=True)
    if elem == "fp8":
        scale = _e8m0_scale(amax, 8)                       # e4m3: largest power of two is 2^8
        q = (g / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8).float()
    elif elem == "fp4":
        scale = _e8m0_scale(amax, 2)                       # e2m1: largest power of two is 2^2
        q = _round_fp4(g / scale)
    else:
        raise ValueError(elem)
    return q.reshape(t.shape), scale.squeeze(-1)


def mx_dequantize(q: torch.Tensor, scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    K = q.shape[-1]
    return (q.float().reshape(*q.shape[:-1], K // block, block) * scale.unsqueeze(-1)).reshape(q.shape)


class _MXLinear(LinearScheme):
    """Microscaling linear: weights and (dynamically) activations carry one e8m0 scale per 32
    elements along K (vllm_ascend/quantization/methods/w8a8_mxfp8.py, w4a4_mxfp4.py,
    w4a8_mxfp.py).  Checkpoints that ship ``weight`` in the element type with ``weight_scale`` in
    e8m0 load as they are; float weights are converted.  The product is evaluated on the
    dequantised operands, which is exact for these formats (block scales are powers of two)."""
    w_elem = "fp8"
    a_elem = "fp8"

    def convert(self, layer) -> None:
        if hasattr(layer, "weight_scale"):
            return
        q, s = mx_quantize(layer.weight, self.w_elem)
        layer.weight = q.to(FP8) if self.w_elem == "fp8" else q.to(torch.bfloat16)
        layer.weight_scale = s

    def named_tensors(self, layer):
        yield "weight_scale", layer.weight_scale

    def apply(self, layer, x, residual=None, skip_bias=False):
        if isinstance(x, ops.QuantAct):
            x = x.dequant()
        K = x.shape[-1]
        xq, xs = mx_quantize(x.reshape(-1, K), self.a_elem)
        a = mx_dequantize(xq, xs).to(x.dtype)
        w = mx_dequantize(layer.weight, layer.weight_scale).to(x.dtype)
        y = ops.linear(a, w, None if skip_bias else layer.bias)
        y = y.view(*x.shape[:-1], w.shape[0])
        return y + residual if residual is not None else y


@register_scheme("W8A8_MXFP8", "linear")
class MXFP8Linear(_MXLinear):
    pass


@register_scheme("W4A4_MXFP4", "linear")
class MXFP4Linear(_MXLinear):
    w_elem = a_elem = "fp4"


@register_scheme("W4A8_MXFP", "linear")
class W4A8MXLinear(_MXLinear):
    w_elem, a_elem = "fp4", "fp8"


@register_scheme("W4A8_DYNAMIC", "linear")
class W4A8DynamicLinear(_PerChannelDynamic):
    """int4 weights with group-wise scales x per-token dynamic int8 activations
    (vllm_ascend/quantization/methods/w4a8.py)."""
    group = 128

    def convert(self, layer) -> None:
        if hasattr(layer, "weight_scale"):
            return
        w = layer.weight.float()
        N, K = w.shape
        g = self.group if K % self.group == 0 else K
        wg = w.view(N, K // g, g)
        scale = (wg.abs().amax(dim=-1, keepdim=True) / 7.0).clamp_min(1e-10)
        layer.weight = (wg / scale).round().clamp(-8, 7).to(torch.int8).view(N, K)
        layer.weight_scale = scale.squeeze(-1)
        layer.group_size = g

    def apply(self, layer, x, residual=None, skip_bias=False):
        N, K = layer.weight.shape
        g = layer.group_size
        x2 = x.reshape(-1, K).float()
        a_scale = (x2.abs().amax(dim=1, keepdim=True) / 127.0).clamp_min(1e-10)
        xq = (x2 / a_scale).round().clamp(-127, 127)
        # integer partial sums per group, scaled per (row, group) like the int8 x int4 kernels do
        part = torch.einsum("tgk,ngk->tng", xq.view(-1, K // g, g), layer.weight.float().view(N, K // g, g))
        y = (part * layer.weight_scale.unsqueeze(0)).sum(-1) * a_scale
        if layer.bias is not None and not skip_bias:
            y = y + layer.bias.float()
        y = y.to(x.dtype).view(*x.shape[:-1], N)
        return y + residual if residual is not None else y


class _DequantMoE(MoEScheme):
    """Expert weights in a compressed format, evaluated on dequantised weights."""

    def _q(self, w):
        raise NotImplementedError

    def _dq(self, q, s, dtype):
        raise NotImplementedError

    def convert(self, block) -> None:
        block.w13, block.w13_scale = self._q(block.w13)
        block.w2, block.w2_scale = self._q(block.w2)
        self.block_ref = block

    def apply_experts(self, x, w13, w2, topk_w, topk_ids, expert_map):
        from ..ops.fused_moe import fused_experts_ref
        blk = self.block_ref
        return fused_experts_ref(x, self._dq(w13, blk.w13_scale, x.dtype), self._dq(w2, blk.w2_scale, x.dtype),
                                 topk_w, topk_ids, expert_map)


@register_scheme("W8A8_MXFP8", "moe")
class MXFP8MoE(_DequantMoE):
    elem = "fp8"

    def _q(self, w):
        q, s = mx_quantize(w, self.elem)
        return (q.to(FP8) if self.elem == "fp8" else q.to(torch.bfloat16)), s

    def _dq(self, q, s, dtype):
        return mx_dequantize(q, s).to(dtype)


@register_scheme("W4A4_MXFP4", "moe")
class MXFP4MoE(MXFP8MoE):
    elem = "fp4"


@register_scheme("W4A8_MXFP", "moe")
class W4A8MXMoE(MXFP8MoE):
    elem = "fp4"


@register_scheme("W4A16_MXFP4", "moe")
class W4A16MXMoE(MXFP8MoE):
    elem = "fp4"


@register_scheme("W4A8_DYNAMIC", "moe")
@register_scheme("W4A16", "moe")
class W4GroupMoE(_DequantMoE):
    group = 128

    def _q(self, w):
        E, N, K = w.shape
        g = self.group if K % self.group == 0 else K
        wg = w.float().view(E, N, K // g, g)
        scale = (wg.abs().amax(dim=-1, keepdim=True) / 7.0).clamp_min(1e-10)
        return (wg / scale).round().clamp(-8, 7).to(torch.int8).view(E, N, K), scale.squeeze(-1)

    def _dq(self, q, s, dtype):
        E, N, K = q.shape
        g = K // s.shape[-1]
        return (q.float().view(E, N, K // g, g) * s.unsqueeze(-1)).view(E, N, K).to(dtype)


# ---------------------------------------------------------------- KV-cache quantization
def kv_quant_fp8(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Per-head static scale, e4m3 storage (the C8 KV scheme's role,
    vllm_ascend/quantization/methods/kv_c8.py): x [T, H, D], scale [H] -> e4m3 [T, H, D]."""
    return (x.float() / scale.view(1, -1, 1)).clamp(-FP8_MAX, FP8_MAX).to(FP8)


def kv_dequant_fp8(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return (q.float() * scale.view(1, -1, 1)).to(dtype)
