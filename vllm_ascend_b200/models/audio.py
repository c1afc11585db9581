"""Whisper-style audio tower of Qwen2-Audio style models and the audio-language model around it.

Log-mel features [mel bins, frames] go through two 1-D convolutions (kernel 3; the second with
stride 2) written as unfold + GEMM, get the learned position table added, run through pre-LayerNorm
encoder layers (bidirectional attention over the valid frames of each clip, GELU MLP), are average
pooled in pairs, normalised and projected to the language model's width.  The outputs replace the
audio placeholder tokens of the prompt, exactly like image tokens.

The reference serves the family through upstream model code on its attention / linear ops; here
tower and merge are native: attention through ``ops.mm_encoder.encoder_attention`` (tcgen05 prefill
kernel, causal masking off), GEMMs with bias / residual epilogues, LayerNorm and GELU kernels.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Iterable

import numpy as np
import torch

from .. import ops
from ..ops import mm_encoder as enc
from .layers import Linear
from .transformer import CausalLM
from .vision import _LN, _Maker


@dataclass
class AudioConfig:
    num_mel_bins: int = 128
    d_model: int = 1280
    encoder_layers: int = 32
    encoder_attention_heads: int = 20
    encoder_ffn_dim: int = 5120
    max_source_positions: int = 1500
    init_std: float = 0.02
    output_dim: int = 0                 # language-model width (set by the owning model)

    @property
    def head_dim(self) -> int:
        return self.d_model // self.encoder_attention_heads

    @classmethod
    def from_hf(cls, d: dict) -> "AudioConfig":
        names = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in names})


def audio_output_lengths(mel_frames):
    """(frames after the stride-2 convolution, tokens after pair pooling) for clips of the given
    number of valid mel frames."""
    n = np.asarray(mel_frames, dtype=np.int64)
    conv = (n - 1) // 2 + 1
    return conv, (conv - 2) // 2 + 1


def _conv1d_k3(x: torch.Tensor, lin: Linear, stride: int) -> torch.Tensor:
    """x [L, C_in] (time-major) -> [L_out, C_out]: kernel 3, padding 1, as one GEMM over unfolded
    windows; the weight is stored [C_out, 3 * C_in] with the tap index outermost."""
    L, C = x.shape
    xp = torch.zeros((L + 2, C), dtype=x.dtype, device=x.device)
    xp[1:L + 1] = x
    L_out = (L + 2 - 3) // stride + 1
    win = xp.unfold(0, 3, stride)[:L_out]                    # [L_out, C, 3]
    cols = win.permute(0, 2, 1).reshape(L_out, 3 * C).contiguous()
    return lin(cols)


class AudioEncoderLayer:
    def __init__(self, cfg: AudioConfig, mk, idx: int):
        D, F = cfg.d_model, cfg.encoder_ffn_dim
        self.cfg = cfg
        self.ln1, self.ln2 = _LN(mk, D, 1e-5), _LN(mk, D, 1e-5)
        # q | k | v in one GEMM; the key projection has no bias (its rows of the bias stay zero)
        self.qkv = Linear(mk.normal((3 * D, D)), mk.zeros((3 * D,)), f"layers.{idx}.self_attn.qkv")
        self.out_proj = Linear(mk.normal((D, D)), mk.zeros((D,)), f"layers.{idx}.self_attn.out_proj")
        self.fc1 = Linear(mk.normal((F, D)), mk.zeros((F,)), f"layers.{idx}.fc1")
        self.fc2 = Linear(mk.normal((D, F)), mk.zeros((D,)), f"layers.{idx}.fc2")

    def __call__(self, h, plan):
        cfg = self.cfg
        N, nh, Dh = h.shape[0], cfg.encoder_attention_heads, cfg.head_dim
        qkv = self.qkv(self.ln1(h))
        q, k, v = (qkv[:, i * nh * Dh:(i + 1) * nh * Dh].view(N, nh, Dh) for i in range(3))
        o = enc.encoder_attention(q, k, v, plan, Dh ** -0.5)
        h = self.out_proj(o.reshape(N, nh * Dh), residual=h)
        return self.fc2(ops.activation(self.fc1(self.ln2(h)).contiguous(), "gelu"), residual=h)


class AudioEncoder:
    """``forward(features, valid_frames)``: features is a list of [mel bins, frames] tensors (padded
    clips), valid_frames the number of real frames of each; returns [sum tokens, output_dim]."""

    def __init__(self, cfg: AudioConfig, device, dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        mk = _Maker(self.device, dtype, cfg.init_std)
        D, C = cfg.d_model, cfg.num_mel_bins
        self.conv1 = Linear(mk.normal((D, 3 * C)), mk.zeros((D,)), "conv1")
        self.conv2 = Linear(mk.normal((D, 3 * D)), mk.zeros((D,)), "conv2")
        self.embed_positions = mk.normal((cfg.max_source_positions, D))
        self.layers = [AudioEncoderLayer(cfg, mk, i) for i in range(cfg.encoder_layers)]
        self.ln_post = _LN(mk, D, 1e-5)
        self.projector = Linear(mk.normal((cfg.output_dim, D)), mk.zeros((cfg.output_dim,)), "projector")

    def forward(self, features, valid_frames) -> torch.Tensor:
        cfg = self.cfg
        conv_len, out_len = audio_output_lengths(valid_frames)
        hs = []
        for f, n in zip(features, conv_len):
            x = f.to(self.device, self.dtype).t().contiguous()             # [frames, mel]
            x = ops.activation(_conv1d_k3(x, self.conv1, 1), "gelu")
            x = ops.activation(_conv1d_k3(x, self.conv2, 2), "gelu")
            n = int(n)
            if n > cfg.max_source_positions or n > x.shape[0]:
                raise ValueError("audio clip longer than the encoder's position table")
            hs.append(x[:n] + self.embed_positions[:n])
        h = torch.cat(hs)
        cu = np.concatenate([[0], np.cumsum(conv_len)])
        plan = enc.make_plan(cu, self.device)
        for layer in self.layers:
            h = layer(h, plan)
        # average consecutive pairs inside every clip (an odd last frame is dropped)
        pooled = []
        for a, n in zip(cu[:-1], out_len):
            a, n = int(a), int(n)
            pooled.append(h[a:a + 2 * n].view(n, 2, -1).float().mean(1).to(h.dtype))
        return self.projector(self.ln_post(torch.cat(pooled)))

    __call__ = forward

    # -- parameters ----------------------------------------------------------------
    def named_parameters(self):
        yield "conv1.weight", self.conv1.weight
        yield "conv1.bias", self.conv1.bias
        yield "conv2.weight", self.conv2.weight
        yield "conv2.bias", self.conv2.bias
        yield "embed_positions.weight", self.embed_positions
        for i, L in enumerate(self.layers):
            p = f"layers.{i}"
            for nm, ln in (("self_attn_layer_norm", L.ln1), ("final_layer_norm", L.ln2)):
                yield f"{p}.{nm}.weight", ln.weight
                yield f"{p}.{nm}.bias", ln.bias
            for nm, lin in (("self_attn.qkv", L.qkv), ("self_attn.out_proj", L.out_proj), ("fc1", L.fc1), ("fc2", L.fc2)):
                yield f"{p}.{nm}.weight", lin.weight
                yield f"{p}.{nm}.bias", lin.bias
        yield "layer_norm.weight", self.ln_post.weight
        yield "layer_norm.bias", self.ln_post.bias
        yield "projector.weight", self.projector.weight
        yield "projector.bias", self.projector.bias

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """Names as in the transformers checkpoint below ``audio_tower.`` (plus ``projector.*``)."""
        params = dict(self.named_parameters())
        D = self.cfg.d_model
        loaded = set()
        for name, w in weights:
            m = re.match(r"(layers\.\d+\.self_attn)\.([qkv])_proj\.(weight|bias)", name)
            if m:
                i = "qkv".index(m.group(2))
                params[f"{m.group(1)}.qkv.{m.group(3)}"][i * D:(i + 1) * D].copy_(w)
                loaded.add(name)
                continue
            if name in ("conv1.weight", "conv2.weight"):
                w = w.permute(0, 2, 1).reshape(w.shape[0], -1)            # [out, in, tap] -> [out, tap * in]
            if name in params:
                params[name].copy_(w.to(params[name].dtype))
                loaded.add(name)
        return loaded


class AudioLMForConditionalGeneration(CausalLM):
    """Decoder of ``CausalLM`` plus the audio tower; audio placeholder tokens take the tower's
    outputs (Qwen2-Audio checkpoint layout: ``audio_tower.*``, ``multi_modal_projector.linear.*``,
    ``language_model.*``)."""
    is_multimodal = True
    num_deepstack = 0

    def __init__(self, cfg, device, **kw):
        super().__init__(cfg, device, **kw)
        self.audio_cfg = AudioConfig.from_hf(cfg.audio_config or {})
        self.audio_cfg.output_dim = cfg.hidden_size
        self.audio_tower = AudioEncoder(self.audio_cfg, self.device, self.dtype) if self.is_first else None
        self.visual = None

    def embed_audio(self, features, valid_frames) -> torch.Tensor:
        return self.audio_tower(features, valid_frames)

    def named_parameters(self):
        yield from super().named_parameters()
        if self.audio_tower is not None:
            for n, t in self.audio_tower.named_parameters():
                yield f"audio_tower.{n}", t

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, aud, names = [], [], {}
        for name, w in weights:
            m = re.match(r"(?:model\.)?audio_tower\.(.*)", name)
            if m:
                aud.append((m.group(1), w))
                names[m.group(1)] = name
                continue
            m = re.match(r"(?:model\.)?multi_modal_projector\.linear\.(weight|bias)", name)
            if m:
                aud.append((f"projector.{m.group(1)}", w))
                names[f"projector.{m.group(1)}"] = name
                continue
            new = re.sub(r"^(?:model\.)?language_model\.", "", name)
            if not new.startswith(("model.", "lm_head.")):
                new = "model." + new
            names[new] = name
            lm.append((new, w))
        loaded = {names[n] for n in super().load_weights(lm)}
        if self.audio_tower is not None:
            loaded |= {names[n] for n in self.audio_tower.load_weights(aud)}
        return loaded
