"""The CPU oracle against vectors produced by the reference's own kernels
(tests/golden/make_sel_attn_golden.py ran nsa_ref's _topk_sparse_attention_fwd/_bwd through
Triton's CPU interpreter, fp16)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle.sel_attn_oracle import (
    attended_key_count,
    check_topk_idx_wellformed,
    sel_attn_forward,
    sel_attn_forward_backward,
)
from fsa.synthetic import make_cu_seqlens, make_topk_idx

CASES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "sel_attn_case*.npz")))


def _load(path):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files if z[k].ndim > 0}
    return t, int(z["block_size"]), float(z["sm_scale"])


def test_golden_files_present():
    assert len(CASES) >= 3


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p) for p in CASES])
def test_oracle_matches_reference_kernels(path):
    t, bs, scale = _load(path)
    check_topk_idx_wellformed(t["topk_idx"], t["cu_seqlens"], bs)
    o, lse, dq, dk, dv = sel_attn_forward_backward(
        t["q"], t["k"], t["v"], t["do"], t["topk_idx"], bs, t["cu_seqlens"], scale
    )
    # reference kernels compute in fp16 with fp32 accumulation: tolerances are the
    # measured fp16 rounding levels of those kernels (outputs ~1e-3, grads a few e-3)
    assert (o - t["o"].float()).abs().max() < 2e-3
    assert (lse - t["lse"]).abs().max() < 2e-5
    assert (dq - t["dq"].float()).abs().max() < 4e-3
    assert (dk - t["dk"].float()).abs().max() < 8e-3
    assert (dv - t["dv"].float()).abs().max() < 8e-3


def test_lse_is_log2_of_softmax_denominator():
    torch.manual_seed(0)
    N, Hk, G, d, bs, T = 130, 1, 2, 64, 32, 2
    q, k, v = torch.randn(N, Hk * G, d), torch.randn(N, Hk, d), torch.randn(N, Hk, d)
    cu = make_cu_seqlens([N])
    idx = make_topk_idx([N], Hk, T, bs, 3)
    o, lse = sel_attn_forward(q, k, v, idx, bs, cu)
    # brute force for a few tokens
    for t in (0, 31, 32, 77, 129):
        blocks = [b for b in idx[0, t].tolist() if b >= 0]
        keys = [j for b in blocks for j in range(b * bs, min((b + 1) * bs, N)) if j <= t]
        s = (q[t, 1] @ k[keys, 0].T) / d ** 0.5
        ref_lse = torch.logsumexp(s, 0) * 1.4426950408889634
        ref_o = torch.softmax(s, 0) @ v[keys, 0]
        assert abs(float(lse[1, t] - ref_lse)) < 1e-4
        assert (o[t, 1] - ref_o).abs().max() < 1e-5


def test_generator_contract_and_key_count():
    seqlens = [300, 64, 1000]
    bs, T, Hk = 64, 16, 2
    idx = make_topk_idx(seqlens, Hk, T, bs, 7)
    cu = make_cu_seqlens(seqlens)
    check_topk_idx_wellformed(idx, cu, bs)
    start = 0
    for L in seqlens:
        for t in sorted({0, min(63, L - 1), min(64, L - 1), L - 1}):
            row = idx[0, start + t].tolist()
            valid = [x for x in row if x >= 0]
            b = t // bs
            assert valid == sorted(set(valid))
            assert 0 in valid and b in valid
            assert len(valid) == min(T, b + 1)
        start += L
    # closed form of the attended-key count for one sequence, one head
    L = 1000
    idx1 = make_topk_idx([L], 1, T, bs, 1)
    P = attended_key_count(idx1, make_cu_seqlens([L]), bs, 1)
    exp = sum((min(T, t // bs + 1) - 1) * bs + t % bs + 1 for t in range(L))
    assert P == exp
