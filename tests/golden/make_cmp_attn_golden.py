"""Generate golden vectors for the compressed branch and the block selection from the reference's OWN kernels.

Runs, on the CPU through Triton's interpreter (``TRITON_INTERPRET=1``, fp16 inputs because the interpreter's bf16 dot
product is broken in Triton 3.6):

* ``CompressedAttention.apply`` forward and backward (nsa_ref/ops/compressed_attention.py:762-829);
* ``_get_attention_score`` per KV head, sliced the way the layer's path slices it (:833-1003, :1280-1283);
* ``_transform_score_kernel`` (:1007-1084) launched as ``transform_score`` launches it (:1087-1158) but with the tap
  weights made on the host (``torch.histc`` of an int64 tensor, :1115, does not exist on the CPU; the weights are the
  histogram of i + j for i < kernel_size/stride, j < block_size/stride);
* the top-k tail (:1307-1313): bf16 cast, ``topk(sorted=False)``, ascending sort, mask of non-causal ids.

The compressed keys/values are random tensors (the reference's ``linear_compress`` is hard-wired to CUDA,
nsa_ref/ops/linear_compress.py:340, and the attention does not care where they come from).

Usage (needs the reference checkout; not needed to run the tests):
    python tests/golden/make_cmp_attn_golden.py /path/to/reference
Writes tests/golden/cmp_attn_case*.npz
"""
import math
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_cmp_attn_golden.py <checkout of Relaxed-System-Lab/Flash-Sparse-Attention>")
sys.path.append(sys.argv[1])

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402

from nsa_ref.ops.compressed_attention import (  # noqa: E402
    CompressedAttention,
    _get_attention_score,
    _transform_score_kernel,
)

CASES = [
    # name, seqlens, Hk, G, d, kernel_size, stride, block_size, topk, seed
    ("case0", [300], 2, 2, 64, 32, 16, 64, 4, 2000),
    ("case1", [200, 20, 141], 1, 4, 128, 32, 16, 64, 3, 2001),     # a sequence shorter than one window: no compressed token
    ("case2", [97, 260], 2, 1, 64, 32, 16, 32, 5, 2002),           # block_size 32: taps [1, 2, 1]
]


def tap_weights(kernel_size, stride, block_size):
    a, b = kernel_size // stride, block_size // stride
    w = torch.zeros(a + b - 1)
    for i in range(a):
        for j in range(b):
            w[i + j] += 1
    return w


for name, seqlens, Hk, G, d, ks, st, bs, topk, seed in CASES:
    g = torch.Generator().manual_seed(seed)
    N, Hq = sum(seqlens), Hk * G
    clens = [(L - ks) // st + 1 if L >= ks else 0 for L in seqlens]
    Nc = sum(clens)
    rnd = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).to(torch.float16)
    q, ck, cv, do = rnd(N, Hq, d), rnd(Nc, Hk, d), rnd(Nc, Hk, d), rnd(N, Hq, d)
    cu_q = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(np.cumsum(clens)), dtype=torch.int32)
    max_q, max_k = max(seqlens), max(clens)
    scale = 1.0 / math.sqrt(d)

    qr, kr, vr = (x.clone().requires_grad_(True) for x in (q, ck, cv))
    o, lse = CompressedAttention.apply(qr, kr, vr, ks, st, cu_q, cu_k, max_q, max_k, scale)
    o.backward(do)
    dq, dk, dv = qr.grad, kr.grad, vr.grad

    max_blocks = math.ceil(max_q / bs)
    w = tap_weights(ks, st, bs)
    scores, block_scores, ids = [], [], []
    q_idx = torch.cat([torch.arange(L) for L in seqlens]) // bs
    for h in range(Hk):
        score = _get_attention_score(q[:, h * G : (h + 1) * G], ck[:, h : h + 1], lse.detach()[h * G : (h + 1) * G], ks, st,
                                     cu_q, cu_k, max_q, max_k, scale)              # [1, N, max_k]
        block_score = torch.zeros(1, N, max_blocks, dtype=torch.float32)
        BQ, BK_, BO = 16, min(128, triton.next_power_of_2(max_blocks)), triton.next_power_of_2(w.numel())
        grid = (1 * len(seqlens), triton.cdiv(N, BQ), triton.cdiv(max_blocks, BK_))
        _transform_score_kernel[grid](
            score, block_score, w, cu_q, 1, w.numel(), score.shape[-1], max_blocks, ks // st - 1, bs, bs // st, 1, 2,
            score.stride(0), score.stride(1), score.stride(2), block_score.stride(0), block_score.stride(1),
            block_score.stride(2), TOTAL_QUERY_LEN=N, BLOCK_SIZE_Q=BQ, BLOCK_SIZE_K=BK_, BLOCK_SIZE_O=BO)
        t = min(topk, max_blocks)
        idx = block_score.to(torch.bfloat16).topk(t, dim=-1, sorted=False).indices.sort(-1).values
        idx[idx > q_idx[None, :, None]] = -1
        scores.append(score[0]); block_scores.append(block_score[0]); ids.append(idx[0].to(torch.int32))

    np.savez_compressed(
        os.path.join(HERE, f"cmp_attn_{name}.npz"),
        q=q.numpy(), ck=ck.numpy(), cv=cv.numpy(), do=do.numpy(), cu_q=cu_q.numpy(), cu_k=cu_k.numpy(),
        kernel_size=np.int32(ks), kernel_stride=np.int32(st), block_size=np.int32(bs), topk=np.int32(topk),
        num_kv_heads=np.int32(Hk), sm_scale=np.float32(scale),
        o=o.detach().numpy(), lse=lse.detach().numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
        score=torch.stack(scores).numpy(), block_score=torch.stack(block_scores).numpy(), topk_idx=torch.stack(ids).numpy(),
    )
    print(name, "done", tuple(o.shape), float(o.float().abs().max()))
