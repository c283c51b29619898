"""CPU oracle for the one-step NSA decode.  TEST INFRASTRUCTURE ONLY (see sel_attn_oracle.py): nothing in the
shipped package imports this file.

Decode semantics: the decoded token is the LAST token (position t = L - 1) of its sequence and receives exactly
what the prefill path computes for row t:
* compressed branch: softmax over the compressed tokens c with c*stride + ks - 1 <= t
  (nsa_ref/ops/compressed_attention.py:106-156);
* block scores / top-k ids from the probabilities of the FIRST query head of each GQA group
  (:866-930, :1046-1117, :1307-1313), tie -> lower block id, ascending, -1 padded;
* selected branch: softmax over the keys <= t of the selected blocks (nsa_ref/ops/topk_sparse_attention.py:95-194);
* sliding window: keys in [t - window, t] (flash-attn ``window_size=(window, -1)`` with one query at the end,
  fsa_preview/module/fsa_decode.py:175-185).
The reference's own decode operators are not pinned by any test and differ from its prefill
(fsa_preview/ops/compressed_attention_decode.py:329-355, selected_attention_decode.py:29-40).

Two parts: ``decode_branches_ref`` (direct dense formulas per sequence) and ``OracleDecodeOps`` (the four device
operators of the decode step restated on the CPU with the same signatures, so that the step's sharding protocol
can run on CPU ranks).
"""
from __future__ import annotations

import math

import torch

from oracle.nsa_layer_oracle import block_scores_ref, topk_from_block_scores

LOG2E = 1.4426950408889634


def _softmax_rows(q, k, v, scale):
    """q [G, d], k/v [n, d] fp32 -> (o [G, d], lse log2 [G]); n == 0 gives (0, -inf)."""
    if k.shape[0] == 0:
        return torch.zeros(q.shape[0], v.shape[1]), torch.full((q.shape[0],), float("-inf"))
    s = (q @ k.t()) * (scale * LOG2E)
    m = s.max(dim=1, keepdim=True).values
    p = torch.exp2(s - m)
    l = p.sum(1, keepdim=True)
    return (p @ v) / l, (m + torch.log2(l)).squeeze(1)


def decode_branches_ref(q, k_seqs, v_seqs, ck_seqs, cv_seqs, cfg, sm_scale=None, topk_idx=None):
    """q [B, Hq, d]; *_seqs: per-sequence tensors [L_b, Hk, d] / [C_b, Hk, d] (k and compressed k already rotated,
    the decoded token included as the last row).  ``topk_idx [B, Hk, T]`` overrides the selection for the selected
    branch (the returned ids are always the oracle's own).  Returns o_cmp, o_sel, o_win [B, Hq, d] fp32, lse x3 [B, Hq],
    topk_idx [B, Hk, T]."""
    B, Hq, d = q.shape
    Hk = k_seqs[0].shape[1]
    G = Hq // Hk
    ks, st, BK, T, W = cfg["kernel_size"], cfg["kernel_stride"], cfg["block_size"], cfg["topk"], cfg["window_size"]
    scale = d ** -0.5 if sm_scale is None else sm_scale
    oc, osel, ow = (torch.zeros(B, Hq, d) for _ in range(3))
    lc, ls, lw = (torch.full((B, Hq), float("-inf")) for _ in range(3))
    idx = torch.full((B, Hk, T), -1, dtype=torch.int32)
    for b in range(B):
        k, v, ck, cv = (x.float() for x in (k_seqs[b], v_seqs[b], ck_seqs[b], cv_seqs[b]))
        L = k.shape[0]
        t = L - 1
        nvis = min((t - (ks - 1)) // st + 1, ck.shape[0]) if t >= ks - 1 else 0
        for h in range(Hk):
            qg = q[b, h * G : (h + 1) * G].float()
            o, lse = _softmax_rows(qg, ck[:nvis, h], cv[:nvis, h], scale)
            oc[b, h * G : (h + 1) * G], lc[b, h * G : (h + 1) * G] = o, lse
            p = torch.zeros(max(ck.shape[0], 1))
            if nvis > 0:
                p[:nvis] = torch.exp2((qg[0] @ ck[:nvis, h].t()) * (scale * LOG2E) - lse[0])
            bs = block_scores_ref(p, t, ks, st, BK, cfg["init_blocks"], cfg["local_blocks"])
            ids = topk_from_block_scores(bs, T)
            idx[b, h] = torch.tensor(ids, dtype=torch.int32)
            use = ids if topk_idx is None else [int(i) for i in topk_idx[b, h]]
            rows = [r for i in use if 0 <= i <= t // BK for r in range(i * BK, min(i * BK + BK, L))]
            o, lse = _softmax_rows(qg, k[rows, h], v[rows, h], scale)
            osel[b, h * G : (h + 1) * G], ls[b, h * G : (h + 1) * G] = o, lse
            w0 = max(0, t - W)
            o, lse = _softmax_rows(qg, k[w0:L, h], v[w0:L, h], scale)
            ow[b, h * G : (h + 1) * G], lw[b, h * G : (h + 1) * G] = o, lse
    return oc, osel, ow, lc, ls, lw, idx


class OracleDecodeOps:
    """CPU restatement of the decode step's device operators (same call signatures as the CUDA operator set)."""

    def attn_partial(self, q, k, v, rng_lo, rng_hi, chunk, nchunk, sm_scale, want_scores=False, rpp=1):
        B, Hq, D = q.shape
        Hk = k.shape[1]
        G = Hq // Hk
        R = rng_lo.shape[-1]
        NP = -(-R // rpp)
        assert rpp == 1 or nchunk == 1
        P = NP * nchunk
        o_part = torch.zeros(B, Hq, P, D)
        ml = torch.zeros(B, Hq, P, 2)
        ml[..., 0] = float("-inf")
        scores = torch.zeros(B, Hk, chunk * nchunk) if want_scores else None
        for b in range(B):
            for h in range(Hk):
                qg = q[b, h * G : (h + 1) * G].float()
                for pr in range(NP):
                    for c in range(nchunk):
                        rows = []
                        for r in range(pr * rpp, min(R, pr * rpp + rpp)):
                            lo_r, hi_r = int(rng_lo[b, h, r]), int(rng_hi[b, h, r])
                            if lo_r < 0:
                                continue
                            lo, hi = lo_r + c * chunk, min(hi_r, lo_r + (c + 1) * chunk)
                            rows += list(range(lo, hi))
                            if want_scores and r == 0 and lo < hi:
                                scores[b, h, lo - lo_r : hi - lo_r] = (qg[0] @ k[lo:hi, h].float().t()) * (sm_scale * LOG2E)
                        if not rows:
                            continue
                        s = (qg @ k[rows, h].float().t()) * (sm_scale * LOG2E)
                        m = s.max(1).values
                        p = torch.exp2(s - m[:, None])
                        o_part[b, h * G : (h + 1) * G, pr * nchunk + c] = p @ v[rows, h].float()
                        ml[b, h * G : (h + 1) * G, pr * nchunk + c, 0] = m
                        ml[b, h * G : (h + 1) * G, pr * nchunk + c, 1] = p.sum(1)
        return o_part, ml, scores

    def lse_merge(self, o_part, ml, out_dtype, p0=0, pn=None):
        P = o_part.shape[-2]
        pn = P - p0 if pn is None else pn
        o_part, ml = o_part[..., p0 : p0 + pn, :].float(), ml[..., p0 : p0 + pn, :].float()
        m, l = ml[..., 0], ml[..., 1]
        m = torch.where(l > 0, m, torch.full_like(m, float("-inf")))
        M = m.max(-1, keepdim=True).values
        w = torch.where(l > 0, torch.exp2(m - torch.where(torch.isfinite(M), M, torch.zeros_like(M))), torch.zeros_like(m))
        Lsum = (w * l).sum(-1)
        o = (w[..., None] * o_part).sum(-2) / torch.where(Lsum > 0, Lsum, torch.ones_like(Lsum))[..., None]
        lse = torch.where(Lsum > 0, M.squeeze(-1) + torch.log2(torch.where(Lsum > 0, Lsum, torch.ones_like(Lsum))),
                          torch.full_like(Lsum, float("-inf")))
        return o.to(out_dtype), lse

    def select_topk(self, scores, ld, shard_len, shard_stride, lse, seq_len, num_cmp, num_kv_heads, kernel_size, kernel_stride,
                    block_size, init_blocks, local_blocks, topk, max_blocks):
        B, Hq = lse.shape
        G = Hq // num_kv_heads
        flat = scores.reshape(-1)
        out = torch.full((B, num_kv_heads, topk), -1, dtype=torch.int32)
        for b in range(B):
            t, n = int(seq_len[b]) - 1, int(num_cmp[b])
            for h in range(num_kv_heads):
                p = torch.zeros(max(n, 1))
                for c in range(n):
                    off = (c // shard_len) * shard_stride + (b * num_kv_heads + h) * ld + c % shard_len
                    p[c] = torch.exp2(flat[off] - lse[b, h * G])
                bs = block_scores_ref(p, t, kernel_size, kernel_stride, block_size, init_blocks, local_blocks)
                out[b, h] = torch.tensor(topk_from_block_scores(bs[:max_blocks], topk), dtype=torch.int32)
        return out

    def cmp_ranges(self, seq_len, cmp_row0, num_kv_heads, kernel_size, kernel_stride, cmp_lo, cmp_hi):
        B = seq_len.numel()
        num_cmp = torch.zeros(B, dtype=torch.int32)
        lo = torch.full((B, num_kv_heads, 1), -1, dtype=torch.int32)
        hi = torch.full((B, num_kv_heads, 1), -1, dtype=torch.int32)
        for b in range(B):
            L = int(seq_len[b])
            n = (L - kernel_size) // kernel_stride + 1 if L >= kernel_size else 0
            num_cmp[b] = n
            e = min(n, cmp_hi) - cmp_lo
            if e > 0:
                lo[b], hi[b] = int(cmp_row0[b]), int(cmp_row0[b]) + e
        return num_cmp, lo, hi

    def ranges(self, topk_idx, seq_len, seq_row0, num_kv_heads, topk, block_size, window, piece, num_pieces, shard_lo, shard_hi):
        B = seq_len.numel()
        R = topk + num_pieces
        lo = torch.full((B, num_kv_heads, R), -1, dtype=torch.int32)
        hi = torch.full((B, num_kv_heads, R), -1, dtype=torch.int32)
        for b in range(B):
            L = int(seq_len[b])
            t = L - 1
            for h in range(num_kv_heads):
                for r in range(R):
                    a = e = 0
                    if L > 0:
                        if r < topk:
                            i = int(topk_idx[b, h, r])
                            if 0 <= i <= t // block_size:
                                a, e = i * block_size, min(i * block_size + block_size, L)
                        else:
                            a = max(0, t - window) + (r - topk) * piece
                            e = min(a + piece, L)
                    a, e = max(a, shard_lo), min(e, shard_hi)
                    if a < e:
                        lo[b, h, r] = int(seq_row0[b]) + a - shard_lo
                        hi[b, h, r] = int(seq_row0[b]) + e - shard_lo
        return lo, hi
