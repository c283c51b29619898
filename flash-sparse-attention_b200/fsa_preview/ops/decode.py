"""Decode-step operators over the C ABI: partial attention over cache-row ranges, log-sum-exp merge,
top-k block selection for the decoded token, range construction.

``CudaDecodeOps`` is the only implementation the package ships; it raises when the sm_100a library
is missing or a tensor is not on a CUDA device.  The step logic in ``nsa_decode_attention`` takes the
operator set as an argument so that the sharding protocol can be exercised by CPU ranks in tests.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from fsa import _lib

OUT_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


class CudaDecodeOps:
    """Thin wrappers: allocate outputs with torch, pass raw pointers to the library."""

    @staticmethod
    def _need_cuda(t):
        if not t.is_cuda:
            raise RuntimeError("the sm_100a decode kernels need CUDA tensors (there is no CPU fallback)")

    def attn_partial(self, q, k, v, rng_lo, rng_hi, chunk, nchunk, sm_scale, want_scores=False, rpp=1):
        """q [B,Hq,D]; k, v [rows,Hk,D]; rng_* [B,Hk,R] int32.  ``rpp`` consecutive ranges share one partial.  Returns
        o_part [B,Hq,P,D] fp32, ml [B,Hq,P,2] with P = ceil(R/rpp)*nchunk, scores [B,Hk,chunk*nchunk] fp32 or None."""
        self._need_cuda(q)
        B, Hq, D = q.shape
        Hk = k.shape[1]
        R = rng_lo.shape[-1]
        P = -(-R // rpp) * nchunk
        assert k.stride(2) == 1 and k.stride(1) == D and v.stride() == k.stride() and q.is_contiguous()
        o_part = torch.empty((B, Hq, P, D), dtype=torch.float32, device=q.device)
        ml = torch.empty((B, Hq, P, 2), dtype=torch.float32, device=q.device)
        ld = chunk * nchunk
        scores = torch.empty((B, Hk, ld), dtype=torch.float32, device=q.device) if want_scores else None
        with torch.cuda.device(q.device):
            rc = _lib.lib().fsa_decode_attn_partial(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), k.shape[0], k.stride(0), _lib.ptr(rng_lo), _lib.ptr(rng_hi), B, Hq, Hk, D, R, rpp, chunk,
                nchunk, _lib.DTYPE_CODE[q.dtype], float(sm_scale), _lib.ptr(o_part), _lib.ptr(ml), _lib.ptr(scores), ld,
                _lib.current_stream(q.device))
        _lib.check(rc, "fsa_decode_attn_partial")
        return o_part, ml, scores

    def lse_merge(self, o_part, ml, out_dtype, p0=0, pn=None):
        """o_part [..., P, D] fp32, ml [..., P, 2] -> o [..., D] in out_dtype, lse [...] (log2 units); merges the
        partials p0 .. p0+pn-1 of every row (all by default)."""
        self._need_cuda(o_part)
        *lead, P, D = o_part.shape
        rows = math.prod(lead)
        pn = P - p0 if pn is None else pn
        assert o_part.is_contiguous() and ml.is_contiguous() and 0 <= p0 and p0 + pn <= P
        o = torch.empty((*lead, D), dtype=out_dtype, device=o_part.device)
        lse = torch.empty(tuple(lead), dtype=torch.float32, device=o_part.device)
        with torch.cuda.device(o_part.device):
            rc = _lib.lib().fsa_lse_merge(o_part.data_ptr() + p0 * D * 4, ml.data_ptr() + p0 * 8, rows, pn, P, D, OUT_CODE[out_dtype],
                                          _lib.ptr(o), _lib.ptr(lse), _lib.current_stream(o_part.device))
        _lib.check(rc, "fsa_lse_merge")
        return o, lse

    def select_topk(self, scores, ld, shard_len, shard_stride, lse, seq_len, num_cmp, num_kv_heads, kernel_size, kernel_stride,
                    block_size, init_blocks, local_blocks, topk, max_blocks):
        self._need_cuda(scores)
        B, Hq = lse.shape
        out = torch.empty((B, num_kv_heads, topk), dtype=torch.int32, device=scores.device)
        with torch.cuda.device(scores.device):
            rc = _lib.lib().fsa_decode_select_topk(
                _lib.ptr(scores), ld, shard_len, shard_stride, _lib.ptr(lse), _lib.ptr(seq_len), _lib.ptr(num_cmp), B, Hq,
                num_kv_heads, kernel_size, kernel_stride, block_size, init_blocks, local_blocks, topk, max_blocks, _lib.ptr(out),
                _lib.current_stream(scores.device))
        _lib.check(rc, "fsa_decode_select_topk")
        return out

    def cmp_ranges(self, seq_len, cmp_row0, num_kv_heads, kernel_size, kernel_stride, cmp_lo, cmp_hi):
        """num_cmp [B] and the compressed-cache row range [B, Hk, 1] of this GPU's visible compressed tokens."""
        self._need_cuda(seq_len)
        B = seq_len.numel()
        num_cmp = torch.empty(B, dtype=torch.int32, device=seq_len.device)
        lo = torch.empty((B, num_kv_heads, 1), dtype=torch.int32, device=seq_len.device)
        hi = torch.empty_like(lo)
        with torch.cuda.device(seq_len.device):
            rc = _lib.lib().fsa_decode_cmp_ranges(_lib.ptr(seq_len), _lib.ptr(cmp_row0), B, num_kv_heads, kernel_size, kernel_stride,
                                                  cmp_lo, min(cmp_hi, 2**31 - 1), _lib.ptr(num_cmp), _lib.ptr(lo), _lib.ptr(hi),
                                                  _lib.current_stream(seq_len.device))
        _lib.check(rc, "fsa_decode_cmp_ranges")
        return num_cmp, lo, hi

    def finish(self, o_part, ml, num_sel, num_win, o_cmp, gate):
        """Merge the selected ([0, num_sel)) and window ([num_sel, num_sel + num_win)) partials of ``o_part [B,Hq,P,D]``
        and mix the three branches with ``gate [B, 3]``: one launch, returns ``[B, Hq, D]`` in o_cmp's dtype."""
        self._need_cuda(o_part)
        B, Hq, P, D = o_part.shape
        assert o_part.is_contiguous() and ml.is_contiguous() and o_cmp.is_contiguous() and num_sel + num_win <= P
        gate = gate.to(o_cmp.dtype).contiguous()
        out = torch.empty_like(o_cmp)
        with torch.cuda.device(o_part.device):
            rc = _lib.lib().fsa_decode_finish(_lib.ptr(o_part), _lib.ptr(ml), B * Hq, num_sel, num_win, P, D, Hq,
                                              _lib.DTYPE_CODE[o_cmp.dtype], _lib.ptr(o_cmp), _lib.ptr(gate), _lib.ptr(out),
                                              _lib.current_stream(o_part.device))
        _lib.check(rc, "fsa_decode_finish")
        return out

    def ranges(self, topk_idx, seq_len, seq_row0, num_kv_heads, topk, block_size, window, piece, num_pieces, shard_lo, shard_hi):
        self._need_cuda(seq_len)
        B = seq_len.numel()
        R = topk + num_pieces
        lo = torch.empty((B, num_kv_heads, R), dtype=torch.int32, device=seq_len.device)
        hi = torch.empty_like(lo)
        with torch.cuda.device(seq_len.device):
            rc = _lib.lib().fsa_decode_ranges(_lib.ptr(topk_idx), _lib.ptr(seq_len), _lib.ptr(seq_row0), B, num_kv_heads, topk,
                                              block_size, window, piece, num_pieces, shard_lo, shard_hi, _lib.ptr(lo), _lib.ptr(hi),
                                              _lib.current_stream(seq_len.device))
        _lib.check(rc, "fsa_decode_ranges")
        return lo, hi


@dataclass
class Shard:
    """What one GPU holds when the KV sequence is split: tokens [tok_lo, tok_hi) and compressed tokens
    [cmp_lo, cmp_hi) of EVERY sequence.  One GPU: everything."""
    tok_lo: int = 0
    tok_hi: int = 2**31 - 1
    cmp_lo: int = 0
    cmp_hi: int = 2**31 - 1
    rank: int = 0
    world: int = 1
    group: object = None


def shard_plan(max_len: int, kernel_size: int, kernel_stride: int, rank: int, world: int, group=None, align: int = 64) -> Shard:
    """Contiguous equal slices of the token axis (multiples of ``align`` tokens) and of the compressed axis."""
    per = -(-max_len // world)
    per = -(-per // align) * align
    max_cmp = (max_len - kernel_size) // kernel_stride + 1 if max_len >= kernel_size else 0
    cper = max(-(-max_cmp // world), 1)
    cper = -(-cper // 4) * 4
    return Shard(rank * per, (rank + 1) * per, rank * cper, (rank + 1) * cper, rank, world, group)


def _pack(*tensors: torch.Tensor) -> torch.Tensor:
    return torch.cat([t.reshape(-1) for t in tensors])


def _unpack(gathered: torch.Tensor, world: int, *like: torch.Tensor):
    """``gathered [world * n]`` (every rank's packed buffer) -> per tensor a view ``[world, *shape]``."""
    out = gathered.view(world, -1)
    views, off = [], 0
    for t in like:
        views.append(out[:, off : off + t.numel()].reshape(world, *t.shape))
        off += t.numel()
    return views


def _all_gather(flat: torch.Tensor, shard: Shard) -> torch.Tensor:
    import torch.distributed as dist

    out = torch.empty((shard.world * flat.numel(),), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, flat, group=shard.group)
    return out


def _merge_gathered(ops, o_all, lse_all, out_dtype):
    """Second-level merge across GPUs: every rank contributed its normalised fp32 output ``[W, ..., D]`` and its lse
    ``[W, ...]``; a rank with no visible key has lse = -inf and weight 0."""
    nd = o_all.dim()
    o_part = o_all.permute(*range(1, nd - 1), 0, nd - 1).contiguous()         # [..., W, D]
    m = lse_all.permute(*range(1, nd - 1), 0)
    ml = torch.stack([m, torch.isfinite(m).to(torch.float32)], dim=-1).contiguous()
    return ops.lse_merge(o_part, ml, out_dtype)


class DecodeStepPlan:
    """The decode step cut at its two exchanges.  One GPU: ``part1`` -> ``part2`` -> ``part3`` back to back.  KV sequence
    sharded: after ``part1`` and after ``part2`` every rank all-gathers one packed fp32 buffer (``self.flat1`` /
    ``self.flat2``) and hands the gathered buffer to the next part.  Each part is free of host synchronisation and of
    collectives, so it can be captured in a CUDA graph of its own while the two collectives stay ordinary launches."""

    def __init__(self, *, kernel_size, kernel_stride, block_size, topk, init_blocks, local_blocks, window_size, max_len,
                 sm_scale=None, shard: Optional[Shard] = None, ops=None, cmp_chunk: int = 1024):
        self.ks, self.stride, self.bs, self.topk = kernel_size, kernel_stride, block_size, topk
        self.init_blocks, self.local_blocks, self.window, self.max_len = init_blocks, local_blocks, window_size, max_len
        self.sm_scale, self.shard, self.ops, self.cmp_chunk = sm_scale, shard or Shard(), ops or CudaDecodeOps(), cmp_chunk
        s = self.shard
        max_cmp = (max_len - kernel_size) // kernel_stride + 1 if max_len >= kernel_size else 0
        # every rank must size its score rows alike (they are all-gathered): the shard WIDTH, not what this rank holds of it
        cmp_local = max(min(max_cmp, s.cmp_hi - s.cmp_lo), 1)
        self.nchunk = -(-cmp_local // cmp_chunk)
        self.ld = cmp_chunk * self.nchunk
        self.max_blocks = -(-max_len // block_size)
        self.npieces = -(-(window_size + 1) // block_size)
        # ranges per partial: the largest power of two <= 16 that divides top-k (a partial never mixes selected blocks and
        # window pieces); longer chains per CTA keep the three-stage K/V ring busy (measured: 0.096 ms at 4, 0.077 at 16)
        self.rpp = next(r for r in (16, 8, 4, 2, 1) if topk % r == 0)

    # compressed branch on this GPU's compressed rows
    def part1(self, q, cmp_k, cmp_v, seq_len, cmp_row0):
        ops, s = self.ops, self.shard
        Hk = cmp_k.shape[1]
        scale = self.sm_scale if self.sm_scale is not None else q.shape[-1] ** -0.5
        # compressed token c is visible when its window ends at or before t (c*stride + ks - 1 <= t)
        self.num_cmp, lo_c, hi_c = ops.cmp_ranges(seq_len, cmp_row0, Hk, self.ks, self.stride, s.cmp_lo, s.cmp_hi)
        o_part, ml, self.scores = ops.attn_partial(q, cmp_k, cmp_v, lo_c, hi_c, self.cmp_chunk, self.nchunk, scale, want_scores=True)
        if s.world == 1:
            self.o_cmp, self.lse_cmp = ops.lse_merge(o_part, ml, q.dtype)
            return None
        self.o_loc, self.lse_loc = ops.lse_merge(o_part, ml, torch.float32)
        self.flat1 = _pack(self.o_loc, self.lse_loc, self.scores)
        return self.flat1

    # top-k of the decoded row, selected blocks + sliding window on this GPU's rows
    def part2(self, q, k, v, seq_len, seq_row0, gathered1=None, gate=None):
        """``gate [B, 3]`` (one GPU only): skip the two merges and return the gate-mixed output of the three branches
        from one fused launch instead (``self.mixed``)."""
        ops, s = self.ops, self.shard
        Hk = k.shape[1]
        scale = self.sm_scale if self.sm_scale is not None else q.shape[-1] ** -0.5
        if s.world == 1:
            scores, shard_len, shard_stride = self.scores, self.ld, 0
        else:
            o_all, lse_all, scores = _unpack(gathered1, s.world, self.o_loc, self.lse_loc, self.scores)   # scores stay shard-major
            self.o_cmp, self.lse_cmp = _merge_gathered(ops, o_all, lse_all, q.dtype)
            shard_len, shard_stride = s.cmp_hi - s.cmp_lo, scores.stride(0)
        self.topk_idx = ops.select_topk(scores, self.ld, shard_len, shard_stride, self.lse_cmp, seq_len, self.num_cmp, Hk, self.ks,
                                        self.stride, self.bs, self.init_blocks, self.local_blocks, self.topk, self.max_blocks)
        lo, hi = ops.ranges(self.topk_idx, seq_len, seq_row0, Hk, self.topk, self.bs, self.window, self.bs, self.npieces,
                            s.tok_lo, s.tok_hi)
        o_part, ml, _ = ops.attn_partial(q, k, v, lo, hi, self.bs, 1, scale, rpp=self.rpp)
        if gate is not None and s.world == 1:
            self.mixed = ops.finish(o_part, ml, self.topk // self.rpp, -(-self.npieces // self.rpp), self.o_cmp, gate)
            return None
        first = torch.float32 if s.world > 1 else q.dtype
        self.o_sel, self.lse_sel = ops.lse_merge(o_part, ml, first, 0, self.topk // self.rpp)
        self.o_win, self.lse_win = ops.lse_merge(o_part, ml, first, self.topk // self.rpp, -(-self.npieces // self.rpp))
        if s.world == 1:
            return None
        self.o_both, self.lse_both = torch.stack([self.o_sel, self.o_win]), torch.stack([self.lse_sel, self.lse_win])
        self.flat2 = _pack(self.o_both, self.lse_both)
        return self.flat2

    def part3(self, q, gathered2=None):
        s = self.shard
        if s.world > 1:
            o_all, lse_all = _unpack(gathered2, s.world, self.o_both, self.lse_both)      # [W, 2, B, Hq, (D)]
            both, lse_both = _merge_gathered(self.ops, o_all, lse_all, q.dtype)
            self.o_sel, self.o_win, self.lse_sel, self.lse_win = both[0], both[1], lse_both[0], lse_both[1]
        return self.o_cmp, self.o_sel, self.o_win, self.lse_cmp, self.lse_sel, self.lse_win, self.topk_idx


def nsa_decode_attention(
    q: torch.Tensor,                 # [B, Hq, D] (already rotated)
    k: torch.Tensor, v: torch.Tensor,            # cache rows [rows, Hk, D] of this GPU (k rotated)
    cmp_k: torch.Tensor, cmp_v: torch.Tensor,    # compressed cache rows of this GPU
    seq_len: torch.Tensor,           # [B] int32: tokens per sequence INCLUDING the decoded one
    seq_row0: torch.Tensor,          # [B] int32: cache row of token shard.tok_lo of each sequence
    cmp_row0: torch.Tensor,          # [B] int32: compressed-cache row of compressed token shard.cmp_lo
    *, kernel_size: int, kernel_stride: int, block_size: int, topk: int, init_blocks: int, local_blocks: int,
    window_size: int, max_len: int, sm_scale: Optional[float] = None, shard: Optional[Shard] = None, ops=None,
    cmp_chunk: int = 1024,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """The three NSA branches for ONE new token per sequence; the token is the last of its sequence and gets
    what the prefill path gives that row.  Returns (o_cmp, o_sel, o_win [B,Hq,D], lse_cmp, lse_sel, lse_win
    [B,Hq] log2 units, topk_idx [B,Hk,T]).  ``max_len`` (host int) bounds every sequence length."""
    plan = DecodeStepPlan(kernel_size=kernel_size, kernel_stride=kernel_stride, block_size=block_size, topk=topk,
                          init_blocks=init_blocks, local_blocks=local_blocks, window_size=window_size, max_len=max_len,
                          sm_scale=sm_scale, shard=shard, ops=ops, cmp_chunk=cmp_chunk)
    flat1 = plan.part1(q, cmp_k, cmp_v, seq_len, cmp_row0)
    g1 = _all_gather(flat1, plan.shard) if flat1 is not None else None
    flat2 = plan.part2(q, k, v, seq_len, seq_row0, g1)
    g2 = _all_gather(flat2, plan.shard) if flat2 is not None else None
    return plan.part3(q, g2)


def nsa_decode_mixed(q, k, v, cmp_k, cmp_v, seq_len, seq_row0, cmp_row0, gate, **kw):
    """One-GPU decode step ending in the gate mix: ``g0 o_cmp + g1 o_sel + g2 o_win`` ``[B, Hq, D]`` and the top-k ids.
    Same arguments as ``nsa_decode_attention`` plus ``gate [B, 3]`` (after the sigmoid); the selected / window merges
    and the mix run as one kernel."""
    plan = DecodeStepPlan(**kw)
    assert plan.shard.world == 1, "the fused finish is the one-GPU path; sharded steps merge across ranks first"
    plan.part1(q, cmp_k, cmp_v, seq_len, cmp_row0)
    plan.part2(q, k, v, seq_len, seq_row0, None, gate=gate)
    return plan.mixed, plan.topk_idx
