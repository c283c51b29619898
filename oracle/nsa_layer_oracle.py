"""CPU oracle for the NSA pieces around selected attention and for the whole layer.
TEST INFRASTRUCTURE ONLY (see sel_attn_oracle.py).

Restates, in fp32 PyTorch:
* ``linear_compress`` (nsa_ref/ops/linear_compress.py:334-346 lengths, :113-131 the product, :495-502 the
  intra-block PE bias);
* the rotary embedding of ``RotaryEmbedding.forward`` (nsa_ref/module/rope.py:102-134): angles in fp32,
  cos/sin rounded to the activation dtype, half-split rotation, positions ``start + i*stride`` per sequence;
* block scores and top-k ids (nsa_ref/ops/compressed_attention.py:866-930 score, :1046-1084 and :1099-1117
  transform, :1307-1313 bf16 cast / topk / sort / mask) with the tie rule "lower block id wins";
* the gate mix and the layer forward (fsa/module/fsa.py:71-173).
"""
from __future__ import annotations

import math

import torch

from oracle.range_attn_oracle import compressed_attention as cmp_attn_ref
from oracle.range_attn_oracle import sliding_window_attention as win_attn_ref
from oracle.sel_attn_oracle import sel_attn_forward

LOG2E = 1.4426950408889634


def linear_compress_ref(x, w, seqlens, kernel_size, kernel_stride, pe=None):
    H, d = x.shape[1], x.shape[2]
    outs, lens, start = [], [], 0
    for L in seqlens:
        n = (L - kernel_size) // kernel_stride + 1 if L >= kernel_size else 0
        lens.append(n)
        for c in range(n):
            win = x[start + c * kernel_stride : start + c * kernel_stride + kernel_size].float()   # [ks, H, d]
            outs.append(torch.einsum("khd,hkde->he", win, w.float().view(H, kernel_size, d, d)))
        start += L
    y = torch.stack(outs, 0) if outs else x.new_zeros((0, H, d), dtype=torch.float32)
    if pe is not None:
        y = y + torch.einsum("hD,hDd->hd", pe.float().reshape(H, -1), w.float()).unsqueeze(0)
    return y, lens


def rope_ref(x, inv_freq, seqlens, start=0, stride=1, table_dtype=torch.bfloat16):
    d = x.shape[-1]
    out = torch.empty_like(x, dtype=torch.float32)
    s = 0
    for L in seqlens:
        pos = torch.arange(start, L * stride + start, stride)[:L].float()
        ang = pos[:, None] * inv_freq.float()[None, :]
        cos = ang.cos().to(table_dtype).float()[:, None, :]
        sin = ang.sin().to(table_dtype).float()[:, None, :]
        x1, x2 = x[s : s + L, :, : d // 2].float(), x[s : s + L, :, d // 2 :].float()
        out[s : s + L, :, : d // 2] = x1 * cos - x2 * sin
        out[s : s + L, :, d // 2 :] = x1 * sin + x2 * cos
        s += L
    return out


def block_scores_ref(p, t, kernel_size, kernel_stride, block_size, init_blocks, local_blocks):
    """bf16-rounded block scores of one token from its probabilities ``p [ncmp]`` (causal blocks only)."""
    a, b = kernel_size // kernel_stride, block_size // kernel_stride
    w = torch.zeros(a + b - 1)
    for i in range(a):
        for j in range(b):
            w[i + j] += 1
    bq = t // block_size
    bs = torch.zeros(bq + 1)
    for blk in range(bq + 1):
        s = torch.zeros((), dtype=torch.float32)
        for o in range(a + b - 1):
            c = blk * b - (a - 1) + o
            if 0 <= c < p.numel():
                s = s + p[c] * w[o]
        if blk < init_blocks or (blk <= bq < blk + local_blocks):
            s = torch.tensor(float("inf"))
        bs[blk] = s
    return bs.to(torch.bfloat16).float()


def topk_from_block_scores(bs, topk_out):
    """Indices of the top ``min(topk_out, len)`` scores, ties to the lower index; ascending; -1 padded."""
    order = sorted(range(bs.numel()), key=lambda i: (-float(bs[i]), i))[: min(topk_out, bs.numel())]
    order = sorted(order)
    return order + [-1] * (topk_out - len(order))


def select_topk_ref(qk, lse0, seqlen, ncmp, sm_scale, kernel_size, kernel_stride, block_size, init_blocks, local_blocks, max_blocks, topk):
    """``qk [L, ncmp]`` raw products of one head, ``lse0 [L]`` (log2).  Returns ``[L, min(topk, max_blocks)]`` ids."""
    t_out = min(topk, max_blocks)
    out = torch.full((seqlen, t_out), -1, dtype=torch.int32)
    for t in range(seqlen):
        nvis = min((t - (kernel_size - 1)) // kernel_stride + 1, ncmp) if t >= kernel_size - 1 else 0
        p = torch.zeros(ncmp)
        if nvis > 0:
            p[:nvis] = torch.exp2(qk[t, :nvis].float() * (sm_scale * LOG2E) - lse0[t])
        bs = block_scores_ref(p, t, kernel_size, kernel_stride, block_size, init_blocks, local_blocks)
        out[t] = torch.tensor(topk_from_block_scores(bs, t_out), dtype=torch.int32)
    return out


def layer_forward_ref(params, x, seqlens, cfg, inv_freq, topk_idx=None, dtype=torch.bfloat16):
    """fp32 layer forward.  ``params``: dict of fp32 tensors with the layer's parameter names; intermediate
    tensors are rounded to ``dtype`` where the layer materialises them in that dtype, so that the same top-k
    ids come out.  Returns (y, topk_idx, branches)."""
    Hq, Hk, d = cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    ks, st, bs_, T = cfg["kernel_size"], cfg["kernel_stride"], cfg["block_size"], cfg["topk"]
    rd = lambda t: t.to(dtype).float()
    cu = torch.zeros(len(seqlens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(seqlens).cumsum(0)
    xf = x.float()
    q = rd(xf @ params["proj_q.weight"].float().t()).view(-1, Hq, d)
    k = rd(xf @ params["proj_k.weight"].float().t()).view(-1, Hk, d)
    v = rd(xf @ params["proj_v.weight"].float().t()).view(-1, Hk, d)
    ck, clens = linear_compress_ref(k, params["compress_key"], seqlens, ks, st, params["intra_block_pe"])
    cv, _ = linear_compress_ref(v, params["compress_value"], seqlens, ks, st, None)
    ck, cv = rd(ck), rd(cv)
    ccu = torch.zeros(len(seqlens) + 1, dtype=torch.int32)
    ccu[1:] = torch.tensor(clens).cumsum(0)
    q = rd(rope_ref(q, inv_freq, seqlens, table_dtype=dtype))
    ck = rd(rope_ref(ck, inv_freq, clens, start=0, stride=st, table_dtype=dtype))
    o_cmp, lse_cmp = cmp_attn_ref(q, ck, cv, ks, st, cu, ccu)
    if topk_idx is None:
        G = Hq // Hk
        max_blocks = math.ceil(max(seqlens) / bs_)
        rows = []
        for h in range(Hk):
            per_seq, qs, cs = [], 0, 0
            for L, n in zip(seqlens, clens):
                qk = q[qs : qs + L, h * G] @ ck[cs : cs + n, h].t() if n > 0 else torch.zeros(L, 0)
                per_seq.append(select_topk_ref(qk, lse_cmp[h * G, qs : qs + L], L, n, d ** -0.5, ks, st, bs_, cfg["init_blocks"],
                                               cfg["local_blocks"], max_blocks, T))
                qs += L
                cs += n
            rows.append(torch.cat(per_seq, 0))
        topk_idx = torch.stack(rows, 0)
    k = rd(rope_ref(k, inv_freq, seqlens, table_dtype=dtype))
    o_sel, _ = sel_attn_forward(q, k, v, topk_idx, bs_, cu)
    o_win, _ = win_attn_ref(q, k, v, cu, cfg["window_size"])
    gate = torch.sigmoid(rd(xf @ params["gate.0.weight"].float().t()))
    gate = rd(gate)
    o = gate[:, 0:1, None] * rd(o_cmp) + gate[:, 1:2, None] * rd(o_sel) + gate[:, 2:3, None] * rd(o_win)
    y = rd(o).reshape(o.shape[0], -1) @ params["proj_o.weight"].float().t()
    return y, topk_idx, (o_cmp, o_sel, o_win)
