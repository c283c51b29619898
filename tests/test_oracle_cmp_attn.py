"""The CPU oracles of the compressed branch and of the block selection against vectors produced by the reference's
own kernels (tests/golden/make_cmp_attn_golden.py ran CompressedAttention, _get_attention_score and
_transform_score_kernel of nsa_ref/ops/compressed_attention.py through Triton's CPU interpreter, fp16), and against the
reference's top-k tail run on those block scores."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import nsa_layer_oracle as orc
from oracle.range_attn_oracle import compressed_attention, with_grads

CASES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "cmp_attn_case*.npz")))
LOG2E = 1.4426950408889634


def _load(path):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files if z[k].ndim > 0}
    s = {k: z[k].item() for k in z.files if z[k].ndim == 0}
    return t, s


def test_golden_files_present():
    assert len(CASES) >= 3


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p) for p in CASES])
def test_compressed_attention_oracle_matches_reference_kernels(path):
    t, s = _load(path)
    o, lse, dq, dk, dv = with_grads(compressed_attention, t["q"], t["ck"], t["cv"], t["do"], s["kernel_size"], s["kernel_stride"],
                                    t["cu_q"], t["cu_k"], s["sm_scale"])
    # rows that see no compressed key: o = 0, lse = -inf on both sides
    assert torch.equal(torch.isinf(lse), torch.isinf(t["lse"]))
    fin = ~torch.isinf(lse)
    assert fin.any() and (~fin).any()
    # the reference kernels compute in fp16 with fp32 accumulation (levels as in test_oracle_sel_attn.py)
    assert (o - t["o"].float()).abs().max() < 2e-3
    assert (lse[fin] - t["lse"][fin]).abs().max() < 2e-5
    assert (dq - t["dq"].float()).abs().max() < 4e-3
    # dk / dv sum over every query of the sequence and reach magnitudes of 10 and more, where one fp16 ulp is 7.8e-3
    for mine, ref in ((dk, t["dk"].float()), (dv, t["dv"].float())):
        assert (mine - ref).abs().max() < 8e-3 * max(1.0, float(ref.abs().max()) / 4)


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p) for p in CASES])
def test_score_and_block_score_oracle_match_reference_kernels(path):
    t, s = _load(path)
    ks, st, bs, T, Hk = s["kernel_size"], s["kernel_stride"], s["block_size"], s["topk"], s["num_kv_heads"]
    q, ck, lse = t["q"].float(), t["ck"].float(), t["lse"]
    G = q.shape[1] // Hk
    cu_q, cu_k = t["cu_q"].tolist(), t["cu_k"].tolist()
    max_q = max(b - a for a, b in zip(cu_q[:-1], cu_q[1:]))
    max_blocks = -(-max_q // bs)
    t_out = min(T, max_blocks)
    ties = rows = 0
    for h in range(Hk):
        for b in range(len(cu_q) - 1):
            qs, qe, c0, c1 = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
            L, n = qe - qs, c1 - c0
            qk = q[qs:qe, h * G] @ ck[c0:c1, h].t() if n > 0 else torch.zeros(L, 0)
            ids = orc.select_topk_ref(qk, lse[h * G, qs:qe], L, n, s["sm_scale"], ks, st, bs, 1, 2, max_blocks, T)
            for tt in range(L):
                nvis = min((tt - (ks - 1)) // st + 1, n) if tt >= ks - 1 else 0
                p = torch.zeros(n)
                if nvis > 0:
                    p[:nvis] = torch.exp2(qk[tt, :nvis] * (s["sm_scale"] * LOG2E) - lse[h * G, qs + tt])
                # probabilities (score_kernel, :897-912): zero outside the visible keys
                ref_p = t["score"][h, qs + tt, :n]
                assert (p - ref_p).abs().max() < 2e-6 if n else True
                # block scores (_transform_score_kernel): same +inf pattern, same values
                mine = orc.block_scores_ref(p, tt, ks, st, bs, 1, 2)                      # bf16-rounded, causal blocks only
                ref_bs = t["block_score"][h, qs + tt, : tt // bs + 1]
                assert torch.equal(torch.isinf(mine), torch.isinf(ref_bs))
                f = ~torch.isinf(ref_bs)
                assert (mine[f] - ref_bs[f].to(torch.bfloat16).float()).abs().max() <= 2 ** -7 * max(1e-6, float(ref_bs[f].abs().max())) if f.any() else True
                # ids: identical wherever the reference's own choice is unambiguous (torch.topk leaves the order of tied
                # scores unspecified; the oracle breaks ties towards the lower block id)
                rows += 1
                sc = ref_bs.to(torch.bfloat16).float().sort(descending=True).values
                if sc.numel() > t_out and float(sc[t_out - 1]) == float(sc[t_out]):
                    ties += 1
                    continue
                if not torch.equal(mine.isinf(), ref_bs.isinf()) or (mine[f] != ref_bs[f].to(torch.bfloat16).float()).any():
                    continue   # a last-bit difference in a probability moved a score across a bf16 boundary
                assert torch.equal(ids[tt], t["topk_idx"][h, qs + tt]), (h, b, tt)
    assert rows > 0 and ties < rows // 2
