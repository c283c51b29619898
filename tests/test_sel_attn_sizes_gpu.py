"""Selected attention at the benchmark configurations' full sizes against the CPU oracle.

The small-shape tests (test_sel_attn_gpu.py) cannot show what only long tile lists show: tile
schedules that wrap, blocks selected by thousands of tokens, accumulators flushed many times.
Here the kernels run the BASELINE configurations as stated and the oracle checks
  * config 0 (1 x 8192 tokens, 4 KV heads, G = 1): the whole forward;
  * config 1 (4 x 16384, 4 KV heads, G = 2): forward and backward of one complete sequence for
    two of its KV heads -- dq on every token, dk / dv on every row (sequences and KV heads are
    independent, so the oracle runs on that sequence alone);
  * config 2 (1 x 65536, G in {1, 4, 16} at d = 128 and G = 2 at d = 256): o, lse and dq of the
    last 1024 tokens (rows that see blocks all over the sequence), plus identities on dk / dv.

Tolerances are those of test_sel_attn_gpu.py (bf16 in/out against fp32): max-abs <= 2e-2 *
max(1, |ref|max / 2), mean-abs <= 1e-3 * the same scale, lse <= 1e-4.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fsa.ops.FSA_topk_sparse_attention import sel_attn_bwd, sel_attn_fwd
from fsa.synthetic import make_cu_seqlens, make_qkv, make_topk_idx
from oracle.sel_attn_oracle import sel_attn_forward_rows, sel_attn_forward, sel_attn_forward_backward_chunked

DEV = "cuda:0"


def _tol_ok(got, ref, name):
    err = (got.float().cpu() - ref).abs()
    scale = max(1.0, float(ref.abs().max()) / 2.0)
    assert float(err.max()) <= 2e-2 * scale, f"{name}: max-abs {float(err.max()):.3e} (ref max {float(ref.abs().max()):.2f})"
    assert float(err.mean()) <= 1e-3 * scale, f"{name}: mean-abs {float(err.mean()):.3e}"


def test_config0_forward_matches_oracle():
    seqlens, Hk, G, d, bs, T = [8192], 4, 1, 128, 64, 16
    N = sum(seqlens)
    q, k, v = make_qkv(N, Hk * G, Hk, d, 42, with_do=False)
    idx = make_topk_idx(seqlens, Hk, T, bs, 42)
    cu = make_cu_seqlens(seqlens)
    scale = d ** -0.5
    o, lse, _ = sel_attn_fwd(q.to(DEV), k.to(DEV), v.to(DEV), idx.to(DEV), bs, cu.to(DEV), scale, check_status=True)
    o_ref, lse_ref = sel_attn_forward(q, k, v, idx, bs, cu, scale, token_chunk=256)
    _tol_ok(o, o_ref, "o")
    assert float((lse.cpu() - lse_ref).abs().max()) <= 1e-4


def test_config1_backward_of_one_sequence_matches_oracle():
    seqlens, Hk, G, d, bs, T = [16384] * 4, 4, 2, 128, 64, 16
    N = sum(seqlens)
    q, k, v, do = make_qkv(N, Hk * G, Hk, d, 43)
    idx = make_topk_idx(seqlens, Hk, T, bs, 43)
    cu = make_cu_seqlens(seqlens)
    scale = d ** -0.5
    qc, kc, vc, dc, ic, cc = (x.to(DEV) for x in (q, k, v, do, idx, cu))
    o, lse, ws = sel_attn_fwd(qc, kc, vc, ic, bs, cc, scale, check_status=True)
    dq, dk, dv = sel_attn_bwd(qc, kc, vc, o, lse, dc, ic, bs, cc, scale, ws, check_status=True)
    s, e = 2 * 16384, 3 * 16384          # third sequence
    cu1 = make_cu_seqlens([e - s])
    for h in (0, 3):                     # KV heads are independent: check the first and the last
        hq = slice(h * G, (h + 1) * G)
        o_r, lse_r, dq_r, dk_r, dv_r = sel_attn_forward_backward_chunked(
            q[s:e, hq], k[s:e, h : h + 1], v[s:e, h : h + 1], do[s:e, hq], idx[h : h + 1, s:e], bs, cu1, scale, token_chunk=512)
        _tol_ok(o[s:e, hq], o_r, f"o head {h}")
        assert float((lse[hq, s:e].cpu() - lse_r).abs().max()) <= 1e-4
        _tol_ok(dq[s:e, hq], dq_r, f"dq head {h}")
        _tol_ok(dk[s:e, h : h + 1], dk_r, f"dk head {h}")
        _tol_ok(dv[s:e, h : h + 1], dv_r, f"dv head {h}")


@pytest.mark.parametrize("G,d", [(1, 128), (4, 128), (16, 128), (2, 256)])
def test_config2_tail_rows_match_oracle(G, d):
    seqlens, Hk, bs, T = [65536], 4, 64, 16
    N = sum(seqlens)
    q, k, v, do = make_qkv(N, Hk * G, Hk, d, 44 + G)
    idx = make_topk_idx(seqlens, Hk, T, bs, 44)
    cu = make_cu_seqlens(seqlens)
    scale = d ** -0.5
    qc, kc, vc, dc, ic, cc = (x.to(DEV) for x in (q, k, v, do, idx, cu))
    o, lse, ws = sel_attn_fwd(qc, kc, vc, ic, bs, cc, scale, check_status=True)
    dq, dk, dv = sel_attn_bwd(qc, kc, vc, o, lse, dc, ic, bs, cc, scale, ws, check_status=True)
    del qc, kc, vc, dc, ws
    # rows of the last 1024 tokens, first and last KV head
    c0, c1 = N - 1024, N
    kf, vf = k.float(), v.float()
    for h in (0, Hk - 1):
        hq = slice(h * G, (h + 1) * G)
        o_parts, lse_parts, dq_parts = [], [], []
        for r0 in range(c0, c1, 256):
            qf = q[r0 : r0 + 256, hq].float().requires_grad_(True)
            o_r, lse_r = sel_attn_forward_rows(qf, kf[:, h : h + 1], vf[:, h : h + 1], idx[h : h + 1], bs, r0, r0 + 256, scale)
            (gq,) = torch.autograd.grad(o_r, qf, do[r0 : r0 + 256, hq].float())
            o_parts.append(o_r.detach()); lse_parts.append(lse_r.detach()); dq_parts.append(gq)
        _tol_ok(o[c0:c1, hq], torch.cat(o_parts, 0), f"o head {h}")
        assert float((lse[hq, c0:c1].cpu() - torch.cat(lse_parts, 1)).abs().max()) <= 1e-4
        _tol_ok(dq[c0:c1, hq], torch.cat(dq_parts, 0), f"dq head {h}")
    # dk / dv over the whole sequence: rows of P sum to one, so the column sums of dV equal those of dO summed over
    # the group; dS rows sum to zero, so every key's dk is finite and the total is bounded by |dO| |V|
    assert torch.isfinite(dq.float()).all() and torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()
    lhs = dv.float().sum(0).cpu()                                        # [Hk, d]
    rhs = do.float().sum(0).view(Hk, G, d).sum(1)
    assert float((lhs - rhs).abs().max()) <= 2e-2 * float(rhs.abs().max()) + 0.5 * G
