"""RopeConfig and RotaryEmbedding with the reference's interface (nsa_ref/module/rope.py:43-134),
without transformers or flash-attn: the llama3 / default inverse frequencies are computed here
and the rotation runs in libfsa_sm100.so.

llama3 rule (the published rule the reference obtains from transformers'
``ROPE_INIT_FUNCTIONS["llama3"]``, call site rope.py:76-78): with ``inv_freq_i = theta^(-2i/d)`` and
``wavelen = 2*pi / inv_freq``: ``wavelen > orig/low_freq_factor`` -> ``inv_freq / factor``;
``wavelen < orig/high_freq_factor`` -> unchanged; otherwise the smooth blend
``(1-s) inv_freq/factor + s inv_freq`` with ``s = (orig/wavelen - low) / (high - low)``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch import nn

from fsa import _lib


@dataclass
class RopeConfig:
    max_position_embeddings: int = 131072
    head_dim: int = 128
    rope_theta: float = 500000
    rope_scaling: dict = field(
        default_factory=lambda: {
            "factor": 8.0,
            "high_freq_factor": 4.0,
            "low_freq_factor": 1.0,
            "original_max_position_embeddings": 8192,
            "rope_type": "llama3",
        }
    )
    # kept for compatibility with the reference dataclass; head_dim is what is used
    hidden_size: int = 4096
    num_attention_heads: int = 32


def compute_inv_freq(config: RopeConfig, device=None) -> torch.Tensor:
    d = config.head_dim
    inv_freq = 1.0 / (config.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).to(device=device, dtype=torch.float) / d))
    scaling = getattr(config, "rope_scaling", None)
    rope_type = "default" if not scaling else scaling.get("rope_type", scaling.get("type", "default"))
    if rope_type == "default":
        return inv_freq
    if rope_type != "llama3":
        raise ValueError(f"rope_type {rope_type!r} is not supported (default, llama3)")
    factor = scaling["factor"]
    low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
    orig = scaling["original_max_position_embeddings"]
    low_wavelen, high_wavelen = orig / low, orig / high
    wavelen = 2 * math.pi / inv_freq
    out = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (orig / wavelen - low) / (high - low)
    blended = (1 - smooth) * out / factor + smooth * out
    medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(medium, blended, out)


class _Rotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, cu_seqlens):
        ctx.save_for_backward(cos, sin, cu_seqlens)
        return _rotate(x, cos, sin, cu_seqlens, 0)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, cu_seqlens = ctx.saved_tensors
        return _rotate(dy, cos, sin, cu_seqlens, 1), None, None, None


def _rotate(x, cos, sin, cu_seqlens, conj):
    assert x.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
    if x.stride(2) != 1 or x.stride(0) % 8 or x.stride(1) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    N, H, D = x.shape
    out = torch.empty((N, H, D), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().fsa_rope(_lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(cu_seqlens),
                                 cu_seqlens.numel() - 1, N, H, D, _lib.DTYPE_CODE[x.dtype], conj, _lib.ptr(out),
                                 _lib.current_stream(x.device))
    _lib.check(rc, "fsa_rope")
    return out


class RotaryEmbedding(nn.Module):
    def __init__(self, config: RopeConfig, device=None):
        super().__init__()
        self.config = config
        self.attention_scaling = 1.0
        # Deliberately NOT a registered buffer: `module.to(torch.bfloat16)` would round a buffer to bf16 and
        # with it every rotation angle (the reference keeps it as a buffer, rope.py:79, and inherits that loss).
        self._inv_freq = compute_inv_freq(config, device)

    @property
    def inv_freq(self) -> torch.Tensor:
        return self._inv_freq

    @torch.no_grad()
    def generate_cos_sin(self, x: torch.Tensor, position_ids: torch.Tensor):
        """cos / sin ``[len, head_dim/2]`` for the given positions, angles in fp32, rounded to x.dtype (rope.py:102-124)."""
        if self._inv_freq.device != position_ids.device:
            self._inv_freq = self._inv_freq.to(position_ids.device)
        freqs = position_ids.float()[:, None] * self._inv_freq[None, :]
        return (freqs.cos() * self.attention_scaling).to(x.dtype), (freqs.sin() * self.attention_scaling).to(x.dtype)

    def forward(self, x: torch.Tensor, cu_seqlens: torch.Tensor, start: int = 0, stride: int = 1, max_seqlen: int | None = None):
        """Rotate ``x [total, heads, head_dim]``; token i of a sequence sits at position ``start + i * stride``.
        ``max_seqlen`` avoids the host sync the reference pays for ``seqlens.max().item()`` (rope.py:128-129)."""
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item()) if cu_seqlens.numel() > 1 else 0
        if x.shape[0] == 0 or max_seqlen == 0:
            return x
        pos = torch.arange(start, max_seqlen * stride + start, stride, device=x.device)[:max_seqlen]
        cos, sin = self.generate_cos_sin(x, pos)
        return _Rotary.apply(x, cos.contiguous(), sin.contiguous(), cu_seqlens.to(torch.int32))
