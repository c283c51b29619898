"""Generate golden vectors for selected attention from the reference's OWN kernels.

Runs ``_topk_sparse_attention_fwd`` / ``_topk_sparse_attention_bwd``
(nsa_ref/ops/topk_sparse_attention.py:814, :908) on the CPU through Triton's interpreter
(``TRITON_INTERPRET=1``).  Inputs are fp16 because the interpreter's bf16 dot product is
broken in Triton 3.6; the values are drawn as bf16 N(0,1) first, which fp16 represents exactly.

Usage (needs the reference checkout; not needed to run the tests):
    python tests/golden/make_sel_attn_golden.py /path/to/reference
Writes tests/golden/sel_attn_case*.npz
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "flash-sparse-attention_b200"))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_sel_attn_golden.py <checkout of Relaxed-System-Lab/Flash-Sparse-Attention>")
ref_root = sys.argv[1]
sys.path.append(ref_root)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from fsa.synthetic import make_cu_seqlens, make_qkv, make_topk_idx  # noqa: E402
from nsa_ref.ops.topk_sparse_attention import (  # noqa: E402
    _topk_sparse_attention_bwd,
    _topk_sparse_attention_fwd,
)

CASES = [
    # name, seqlens, Hk, G, d, B_K, T, seed
    ("case0", [256], 2, 2, 128, 64, 4, 1000),
    ("case1", [100, 156], 2, 1, 64, 32, 3, 1001),
    ("case2", [70, 1, 129], 1, 4, 128, 64, 16, 1002),
]

for name, seqlens, Hk, G, d, B_K, T, seed in CASES:
    N = sum(seqlens)
    cu = make_cu_seqlens(seqlens)
    q, k, v, do = make_qkv(N, Hk * G, Hk, d, seed, dtype=torch.bfloat16)
    q, k, v, do = (x.to(torch.float16) for x in (q, k, v, do))
    idx = make_topk_idx(seqlens, Hk, T, B_K, seed)
    scale = 1.0 / (d ** 0.5)
    mx = max(seqlens)
    o, lse = _topk_sparse_attention_fwd(q, k, v, idx, B_K, cu, cu, mx, mx, scale)
    dq, dk, dv = _topk_sparse_attention_bwd(o, do, lse, q, k, v, idx, B_K, cu, cu, mx, mx, scale)
    np.savez_compressed(
        os.path.join(HERE, f"sel_attn_{name}.npz"),
        q=q.numpy(), k=k.numpy(), v=v.numpy(), do=do.numpy(), topk_idx=idx.numpy(), cu_seqlens=cu.numpy(),
        block_size=np.int32(B_K), sm_scale=np.float32(scale),
        o=o.numpy(), lse=lse.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
    )
    print(name, "done", o.shape, float(o.float().abs().max()))
