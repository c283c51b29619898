"""CPU oracle for the two dense NSA branches.  TEST INFRASTRUCTURE ONLY (see sel_attn_oracle.py).

* compressed branch: restates ``forward_kernel`` of nsa_ref/ops/compressed_attention.py:28-156 --
  query ``t`` (position inside its sequence) sees compressed key ``c`` iff
  ``t >= c * kernel_stride + kernel_size - 1`` (:77-80, :118-123); logits ``q.k * scale * log2(e)``;
  ``lse`` in log2 units; rows that see nothing give ``o = 0, lse = -inf`` (:548-553).
* sliding window: restates the semantics of ``flash_attn_varlen_func(causal=True,
  window_size=(W, -1))`` (third-party flash-attn 2.8.3, call site fsa/module/fsa.py:149-159): key ``j``
  visible iff ``t - W <= j <= t`` inside the sequence.

Gradients come from autograd through the fp32 forward.
"""
from __future__ import annotations

import math

import torch

LOG2E = 1.4426950408889634


def masked_attention(q, k, v, mask_fn, cu_q, cu_k, sm_scale=None):
    """fp32 attention with ``mask_fn(t_local [Lq,1], c_local [1,Lk]) -> bool visible``; returns (o, lse_log2)."""
    N, Hq, d = q.shape
    Hk = k.shape[1]
    G = Hq // Hk
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    outs, lses = [], []
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for b in range(len(cq) - 1):
        qs, qe, ks, ke = cq[b], cq[b + 1], ck[b], ck[b + 1]
        Lq, Lk = qe - qs, ke - ks
        if Lq == 0:
            continue
        qf = q[qs:qe].float()
        kf = k[ks:ke].float().repeat_interleave(G, dim=1)
        vf = v[ks:ke].float().repeat_interleave(G, dim=1)
        vis = mask_fn(torch.arange(Lq).view(-1, 1), torch.arange(Lk).view(1, -1)) if Lk > 0 else torch.zeros(Lq, 0, dtype=torch.bool)
        logits = torch.einsum("thd,chd->htc", qf, kf) * (sm_scale * LOG2E)
        logits = logits.masked_fill(~vis.unsqueeze(0), float("-inf"))
        m = logits.max(-1, keepdim=True).values if Lk > 0 else torch.full((Hq, Lq, 1), float("-inf"))
        m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = torch.exp2(logits - m_safe)
        l = p.sum(-1, keepdim=True)
        o = torch.einsum("htc,chd->thd", p / torch.where(l > 0, l, torch.ones_like(l)), vf)
        lse = torch.where(l > 0, m_safe + torch.log2(torch.where(l > 0, l, torch.ones_like(l))), torch.full_like(l, float("-inf")))
        outs.append(o)
        lses.append(lse.squeeze(-1))
    return torch.cat(outs, 0), torch.cat(lses, 1)


def compressed_attention(q, ck, cv, kernel_size, kernel_stride, cu_q, cu_k, sm_scale=None):
    return masked_attention(q, ck, cv, lambda t, c: t >= c * kernel_stride + kernel_size - 1, cu_q, cu_k, sm_scale)


def sliding_window_attention(q, k, v, cu, window, sm_scale=None):
    return masked_attention(q, k, v, lambda t, j: (j <= t) & (j >= t - window), cu, cu, sm_scale)


def with_grads(fn, q, k, v, do, *args):
    qf, kf, vf = (x.detach().float().requires_grad_(True) for x in (q, k, v))
    o, lse = fn(qf, kf, vf, *args)
    dq, dk, dv = torch.autograd.grad(o, (qf, kf, vf), do.float())
    return o.detach(), lse.detach(), dq, dk, dv
