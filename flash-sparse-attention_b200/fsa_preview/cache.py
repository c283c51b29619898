"""Pre-allocated KV cache for one-step NSA decode.

The reference concatenates the whole cache with the new token on every step
(fsa_preview/module/fsa_decode.py:84-85, :127-132).  Here the cache is allocated once at its full
length ([batch, capacity] rows per GPU, sized for HBM) and a step appends in place with index
copies that need no host synchronisation:

* ``k`` (rotated) and ``v``: this GPU's slice [tok_lo, tok_hi) of every sequence;
* ``cmp_k`` (rotated at positions c * stride) and ``cmp_v``: compressed tokens [cmp_lo, cmp_hi);
* ``k_tail`` / ``v_tail``: the last ``kernel_size`` un-rotated K and V rows of every sequence as a
  ring — the incremental compressor's input window (fsa_preview/ops/linear_compress_decode.py:14-76,
  fed with raw tokens as the reference's own test does, test/test_cmp_attn_decode.py:150-210).

With the KV sequence sharded, every rank sees the same new token, keeps the same ring, computes the
same compressed token, and only the owner of a position writes it.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from fsa_preview.ops.decode import Shard


class DecodeCache:
    def __init__(self, batch: int, max_len: int, num_kv_heads: int, head_dim: int, kernel_size: int, kernel_stride: int,
                 dtype=torch.bfloat16, device="cuda", shard: Optional[Shard] = None):
        self.B, self.max_len, self.Hk, self.D = batch, max_len, num_kv_heads, head_dim
        self.ks, self.stride = kernel_size, kernel_stride
        self.shard = shard or Shard()
        s = self.shard
        self.cap = max(min(max_len, s.tok_hi) - s.tok_lo, 0)
        max_cmp = (max_len - kernel_size) // kernel_stride + 1 if max_len >= kernel_size else 0
        self.cmp_cap = max(min(max_cmp, s.cmp_hi) - s.cmp_lo, 0)
        # one extra row at the end of each buffer swallows the writes of non-owners
        mk = lambda rows: torch.zeros((rows + 1, num_kv_heads, head_dim), dtype=dtype, device=device)
        self.k, self.v = mk(batch * self.cap), mk(batch * self.cap)
        self.cmp_k, self.cmp_v = mk(batch * self.cmp_cap), mk(batch * self.cmp_cap)
        self.k_tail, self.v_tail = mk(batch * kernel_size), mk(batch * kernel_size)
        self.seq_len = torch.zeros(batch, dtype=torch.int32, device=device)
        ar = torch.arange(batch, dtype=torch.int32, device=device)
        self.seq_row0 = ar * self.cap
        self.cmp_row0 = ar * self.cmp_cap
        self.tail_row0 = (ar * kernel_size).long()
        self.host_len = [0] * batch
        # True: always run the compressor with masked writes, so that every step issues the same launches (graph capture)
        self.always_compress = False

    # ---------------------------------------------------------------- bulk load after a prefill
    @torch.no_grad()
    def load(self, k_raw: torch.Tensor, k_rot: torch.Tensor, v: torch.Tensor, cmp_k_rot: torch.Tensor, cmp_v: torch.Tensor,
             seqlens: Sequence[int], cmp_seqlens: Sequence[int]):
        """Packed prefill tensors ([total, Hk, D], sequences back to back) -> cache.  Set-up path (host loop)."""
        s = self.shard
        ts = cs = 0
        for b, (L, C) in enumerate(zip(seqlens, cmp_seqlens)):
            assert L <= self.max_len
            a, e = min(s.tok_lo, L), min(s.tok_hi, L)
            if e > a:
                r0 = b * self.cap
                self.k[r0 : r0 + e - a] = k_rot[ts + a : ts + e]
                self.v[r0 : r0 + e - a] = v[ts + a : ts + e]
            a, e = min(s.cmp_lo, C), min(s.cmp_hi, C)
            if e > a:
                r0 = b * self.cmp_cap
                self.cmp_k[r0 : r0 + e - a] = cmp_k_rot[cs + a : cs + e]
                self.cmp_v[r0 : r0 + e - a] = cmp_v[cs + a : cs + e]
            for t in range(max(0, L - self.ks), L):
                self.k_tail[b * self.ks + t % self.ks] = k_raw[ts + t]
                self.v_tail[b * self.ks + t % self.ks] = v[ts + t]
            ts += L
            cs += C
            self.host_len[b] = L
        self.seq_len.copy_(torch.tensor(self.host_len, dtype=torch.int32))

    # ---------------------------------------------------------------- one token per sequence
    @torch.no_grad()
    def append(self, k_raw: torch.Tensor, k_rot: torch.Tensor, v: torch.Tensor, compress_key: torch.Tensor,
               compress_value: torch.Tensor, intra_block_pe: Optional[torch.Tensor],
               rope_fn: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None):
        """Append one token per sequence ([B, Hk, D] each) and, for the sequences whose new length completes a
        compression window, the new compressed token.  ``rope_fn(x [B,Hk,D], positions [B]) -> rotated x``."""
        s = self.shard
        t = self.seq_len.long()                                         # position of the new token
        own = (t >= s.tok_lo) & (t < s.tok_hi)
        dummy = self.k.shape[0] - 1
        rows = torch.where(own, self.seq_row0.long() + t - s.tok_lo, torch.full_like(t, dummy))
        self.k.index_copy_(0, rows, k_rot)
        self.v.index_copy_(0, rows, v)
        ring = self.tail_row0 + t % self.ks
        self.k_tail.index_copy_(0, ring, k_raw)
        self.v_tail.index_copy_(0, ring, v)
        self.seq_len += 1
        new_host = [L + 1 for L in self.host_len]
        self.host_len = new_host
        if not self.always_compress and not any(L >= self.ks and (L - self.ks) % self.stride == 0 for L in new_host):
            return
        n = t + 1
        emit = (n >= self.ks) & ((n - self.ks) % self.stride == 0)
        m = torch.clamp((n - self.ks) // self.stride, min=0)             # index of the compressed token
        order = (n % self.ks)[:, None] + torch.arange(self.ks, device=t.device)[None, :]
        idx = self.tail_row0[:, None] + order % self.ks                  # ring rows, oldest first
        H, D = self.Hk, self.D
        xk = self.k_tail[idx].permute(2, 0, 1, 3).reshape(H, self.B, self.ks * D)    # [Hk, B, ks*D]
        xv = self.v_tail[idx].permute(2, 0, 1, 3).reshape(H, self.B, self.ks * D)
        ck = torch.bmm(xk, compress_key).transpose(0, 1)                 # [B, Hk, D]
        cv = torch.bmm(xv, compress_value).transpose(0, 1)
        if intra_block_pe is not None:
            ck = ck + torch.einsum("hD,hDd->hd", intra_block_pe.reshape(H, self.ks * D), compress_key).unsqueeze(0)
        if rope_fn is not None:
            ck = rope_fn(ck.contiguous(), m * self.stride)
        cown = emit & (m >= s.cmp_lo) & (m < s.cmp_hi)
        cdummy = self.cmp_k.shape[0] - 1
        crow = torch.where(cown, self.cmp_row0.long() + m - s.cmp_lo, torch.full_like(m, cdummy))
        self.cmp_k.index_copy_(0, crow, ck.to(self.cmp_k.dtype))
        self.cmp_v.index_copy_(0, crow, cv.contiguous().to(self.cmp_v.dtype))
