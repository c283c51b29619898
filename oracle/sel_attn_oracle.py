"""CPU oracle for NSA *selected* (top-k block-sparse) attention.  TEST INFRASTRUCTURE ONLY.

This file is a checker: only the test-suite, the smoke test and the CPU-baseline leg of the
benchmark may import it.  No product code path may call into it.

It restates, in fp32 PyTorch on the CPU, the algorithm of the reference's query-outer
kernels:

* forward  -- ``forward_kernel_orig`` (nsa_ref/ops/topk_sparse_attention.py:27-194)
    - slot validity: the number of usable slots of token ``t`` is
      ``#(0 <= idx <= t_local // block_size)`` and the kernel consumes the *first* that many
      entries (:116-119, :154-157), so valid ids must precede the ``-1`` padding;
    - causal rule inside a block: key position ``c + j <= t_local`` (:162);
    - logits are ``q.k * sm_scale * log2(e)`` and probabilities ``exp2`` of them (:73, :164-167);
    - ``lse`` is returned in **log2 units** (:178) with layout ``[num_q_heads, total_len]``;
    - output ``o = softmax(logits) @ v`` over all keys of all selected blocks (:181).
* backward -- ``backward_dkdv`` (:480-644) and ``backward_dq`` (:648-811):
    ``p = exp2(s*log2e*scale - lse)``, ``dp = do.v^T``, ``ds = scale * p * (dp - delta)``,
    ``delta = sum_d o*do`` (``backward_sum_o_do``, :198-230), ``dv = p^T do``, ``dk = ds^T q``,
    ``dq = ds k``.  Here the gradients come from autograd through the fp32 forward, which is
    the same math.

Pinned against the reference itself: ``tests/golden/make_sel_attn_golden.py`` runs the
reference's own ``_topk_sparse_attention_fwd/_bwd`` on the CPU through Triton's interpreter
(fp16 inputs) and stores inputs and outputs; ``tests/test_oracle_sel_attn.py`` checks this
oracle against those stored vectors.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

LOG2E = 1.4426950408889634


def check_topk_idx_wellformed(topk_idx: torch.Tensor, cu_seqlens: torch.Tensor, block_size: int) -> None:
    """Assert the input contract both reference kernels rely on: per (head, token) the usable
    ids (``0 <= id <= t_local // block_size``) come first, everything after is unusable."""
    Hk, N, T = topk_idx.shape
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        if e == s:
            continue
        t_loc = torch.arange(e - s)
        lim = (t_loc // block_size).view(1, -1, 1)
        idx = topk_idx[:, s:e].long()
        valid = (idx >= 0) & (idx <= lim)
        n_valid = valid.sum(-1, keepdim=True)
        first = torch.arange(T).view(1, 1, T) < n_valid
        assert bool((valid == first).all()), "usable block ids must precede padding"


def sel_attn_forward(
    q: torch.Tensor,  # [N, Hq, d]
    k: torch.Tensor,  # [N, Hk, d]
    v: torch.Tensor,  # [N, Hk, d]
    topk_idx: torch.Tensor,  # [Hk, N, T] int32, block ids local to each sequence
    block_size: int,
    cu_seqlens: torch.Tensor,  # [B+1] int32
    sm_scale: Optional[float] = None,
    token_chunk: int = 256,
    p_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 selected attention.  Returns ``(o [N,Hq,d] fp32, lse [Hq,N] fp32 in log2 units)``.

    Differentiable in q, k, v.  ``p_dtype`` optionally rounds the un-normalised
    probabilities before the P.V product the way the reference does (``p.to(v.dtype)``,
    nsa_ref/ops/topk_sparse_attention.py:174); ``None`` keeps everything fp32.
    """
    N, Hq, d = q.shape
    Hk = k.shape[1]
    G = Hq // Hk
    T = topk_idx.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    qf, kf, vf = q.float(), k.float(), v.float()
    o = torch.zeros(N, Hq, d, dtype=torch.float32)
    lse = torch.full((Hq, N), float("-inf"), dtype=torch.float32)
    cu = cu_seqlens.tolist()
    o_chunks = []
    lse_chunks = []
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        L = e - s
        if L == 0:
            continue
        nb = (L + block_size - 1) // block_size
        Lp = nb * block_size
        # zero-pad K/V of this sequence to whole blocks (the kernels zero-fill out-of-range rows)
        kp = torch.zeros(Lp, Hk, d, dtype=torch.float32)
        vp = torch.zeros(Lp, Hk, d, dtype=torch.float32)
        kp = torch.cat([kf[s:e], kp[L:]], 0)
        vp = torch.cat([vf[s:e], vp[L:]], 0)
        kb = kp.view(nb, block_size, Hk, d)
        vb = vp.view(nb, block_size, Hk, d)
        for c0 in range(0, L, token_chunk):
            c1 = min(L, c0 + token_chunk)
            C = c1 - c0
            t_loc = torch.arange(c0, c1)
            idx = topk_idx[:, s + c0 : s + c1].long()  # [Hk, C, T]
            lim = (t_loc // block_size).view(1, C, 1)
            valid = (idx >= 0) & (idx <= lim)
            n_valid = valid.sum(-1, keepdim=True)
            use = torch.arange(T).view(1, 1, T) < n_valid  # first n_valid slots
            blk = idx.clamp(min=0, max=nb - 1)
            o_heads = []
            lse_heads = []
            for h in range(Hk):
                kg = kb[blk[h], :, h]  # [C, T, B, d]
                vg = vb[blk[h], :, h]
                qh = qf[s + c0 : s + c1, h * G : (h + 1) * G]  # [C, G, d]
                logits = torch.einsum("cgd,ctjd->cgtj", qh, kg) * (sm_scale * LOG2E)
                key_pos = blk[h].unsqueeze(-1) * block_size + torch.arange(block_size).view(1, 1, -1)
                ok = use[h].unsqueeze(-1) & (key_pos <= t_loc.view(C, 1, 1))  # [C, T, B]
                logits = logits.masked_fill(~ok.unsqueeze(1), float("-inf"))
                flat = logits.reshape(C, G, T * block_size)
                m = flat.max(-1, keepdim=True).values
                m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
                p = torch.exp2(flat - m_safe)
                l = p.sum(-1, keepdim=True)
                lse_h = (m_safe + torch.log2(l)).squeeze(-1)  # [C, G]; -inf when nothing is attended
                if p_dtype is not None:
                    p = p.to(p_dtype).float()
                oh = torch.einsum("cgx,cxd->cgd", p, vg.reshape(C, T * block_size, d))
                oh = oh / torch.where(l > 0, l, torch.ones_like(l))
                o_heads.append(oh)
                lse_heads.append(lse_h)
            o_chunks.append((s + c0, s + c1, torch.cat(o_heads, 1)))
            lse_chunks.append((s + c0, s + c1, torch.cat(lse_heads, 1)))
    if o_chunks:
        pieces = sorted(o_chunks, key=lambda x: x[0])
        o = _assemble(pieces, N, (Hq, d))
        lse = _assemble(sorted(lse_chunks, key=lambda x: x[0]), N, (Hq,), fill=float("-inf")).transpose(0, 1)
    return o, lse.contiguous()


def _assemble(pieces, N, tail, fill=0.0):
    """Concatenate [start, end, tensor] pieces into an [N, *tail] tensor without in-place
    writes (keeps autograd simple)."""
    out = []
    pos = 0
    for s, e, t in pieces:
        if s > pos:
            out.append(torch.full((s - pos, *tail), fill, dtype=torch.float32))
        out.append(t)
        pos = e
    if pos < N:
        out.append(torch.full((N - pos, *tail), fill, dtype=torch.float32))
    return torch.cat(out, 0)


def sel_attn_forward_backward(q, k, v, do, topk_idx, block_size, cu_seqlens, sm_scale=None):
    """Forward + gradients (fp32, autograd).  Returns ``(o, lse, dq, dk, dv)``."""
    qf = q.detach().float().requires_grad_(True)
    kf = k.detach().float().requires_grad_(True)
    vf = v.detach().float().requires_grad_(True)
    o, lse = sel_attn_forward(qf, kf, vf, topk_idx, block_size, cu_seqlens, sm_scale)
    dq, dk, dv = torch.autograd.grad(o, (qf, kf, vf), do.float())
    return o.detach(), lse.detach(), dq, dk, dv


def sel_attn_forward_backward_chunked(q, k, v, do, topk_idx, block_size, cu_seqlens, sm_scale=None, token_chunk=512):
    """The same forward + gradients for problems whose autograd graph would not fit in memory:
    one graph per chunk of query tokens (rows of the softmax are independent, so dq comes out
    per chunk and dk / dv are sums over chunks).  Single sequence per call keeps it simple:
    ``cu_seqlens`` must be ``[0, N]``.  Returns ``(o, lse, dq, dk, dv)`` in fp32."""
    N, Hq, d = q.shape
    assert cu_seqlens.tolist() == [0, N], "one sequence per call"
    kf = k.detach().float()
    vf = v.detach().float()
    dk = torch.zeros_like(kf)
    dv = torch.zeros_like(vf)
    o_parts, lse_parts, dq_parts = [], [], []
    for c0 in range(0, N, token_chunk):
        c1 = min(N, c0 + token_chunk)
        # keys a chunk can see end at its last token: the prefix [0, c1) is a complete problem for these rows
        qc = q[c0:c1].detach().float().requires_grad_(True)
        kc = kf[:c1].clone().requires_grad_(True)
        vc = vf[:c1].clone().requires_grad_(True)
        o_c, lse_c = sel_attn_forward_rows(qc, kc, vc, topk_idx[:, :c1], block_size, c0, c1, sm_scale)
        gq, gk, gv = torch.autograd.grad(o_c, (qc, kc, vc), do[c0:c1].float())
        o_parts.append(o_c.detach())
        lse_parts.append(lse_c.detach())
        dq_parts.append(gq)
        dk[:c1] += gk
        dv[:c1] += gv
    return torch.cat(o_parts, 0), torch.cat(lse_parts, 1), torch.cat(dq_parts, 0), dk, dv


def sel_attn_forward_rows(q_rows, kf, vf, topk_idx, block_size, c0, c1, sm_scale):
    """Rows [c0, c1) of a single sequence: ``q_rows [c1-c0, Hq, d]`` are those rows' queries, ``kf``/``vf`` the
    sequence's K/V (at least the prefix [0, c1)); same rules as ``sel_attn_forward``.  Returns
    ``(o [C,Hq,d], lse [Hq,C])``."""
    Lk, Hk, d = kf.shape
    Hq = q_rows.shape[1]
    G = Hq // Hk
    T = topk_idx.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    nb = (Lk + block_size - 1) // block_size
    pad = nb * block_size - Lk
    if pad:
        kf = torch.cat([kf, kf.new_zeros(pad, Hk, d)], 0)
        vf = torch.cat([vf, vf.new_zeros(pad, Hk, d)], 0)
    kb = kf.view(nb, block_size, Hk, d)
    vb = vf.view(nb, block_size, Hk, d)
    C = c1 - c0
    t_loc = torch.arange(c0, c1)
    idx = topk_idx[:, c0:c1].long()
    lim = (t_loc // block_size).view(1, C, 1)
    valid = (idx >= 0) & (idx <= lim)
    use = torch.arange(T).view(1, 1, T) < valid.sum(-1, keepdim=True)
    blk = idx.clamp(min=0, max=nb - 1)
    o_heads, lse_heads = [], []
    for h in range(Hk):
        kg = kb[blk[h], :, h]
        vg = vb[blk[h], :, h]
        qh = q_rows[:, h * G : (h + 1) * G]
        logits = torch.einsum("cgd,ctjd->cgtj", qh, kg) * (sm_scale * LOG2E)
        key_pos = blk[h].unsqueeze(-1) * block_size + torch.arange(block_size).view(1, 1, -1)
        ok = use[h].unsqueeze(-1) & (key_pos <= t_loc.view(C, 1, 1))
        logits = logits.masked_fill(~ok.unsqueeze(1), float("-inf"))
        flat = logits.reshape(C, G, T * block_size)
        m = flat.max(-1, keepdim=True).values
        m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = torch.exp2(flat - m_safe)
        l = p.sum(-1, keepdim=True)
        lse_heads.append((m_safe + torch.log2(l)).squeeze(-1))
        oh = torch.einsum("cgx,cxd->cgd", p, vg.reshape(C, T * block_size, d))
        o_heads.append(oh / torch.where(l > 0, l, torch.ones_like(l)))
    return torch.cat(o_heads, 1), torch.cat(lse_heads, 1).transpose(0, 1)


def attended_key_count(topk_idx: torch.Tensor, cu_seqlens: torch.Tensor, block_size: int, group: int) -> int:
    """P = number of (query head, token, key) triples actually attended: the figure the
    effective-FLOP count is built on (forward 4*d*P, backward 10*d*P)."""
    Hk, N, T = topk_idx.shape
    total = 0
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        if e == s:
            continue
        t_loc = torch.arange(e - s)
        lim = (t_loc // block_size).view(1, -1, 1)
        idx = topk_idx[:, s:e].long()
        valid = (idx >= 0) & (idx <= lim)
        own = valid & (idx == lim)
        full = valid & ~own
        total += int(full.sum()) * block_size
        total += int((own.any(-1) * (t_loc % block_size + 1).view(1, -1)).sum())
    return total * group
