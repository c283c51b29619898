"""Compressed-branch and sliding-window attention on the GPU against the CPU oracle.
Tolerances as in test_sel_attn_gpu.py (bf16 in/out vs fp32 oracle)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fsa.ops.range_attention import compressed_attention_core, sliding_window_attention
from fsa.synthetic import make_cu_seqlens
from oracle import range_attn_oracle as orc

DEV = "cuda:0"


def _tol_ok(got, ref, name):
    err = (got.float().cpu() - ref).abs()
    scale = max(1.0, float(ref.abs().max()) / 2.0)
    assert float(err.max()) <= 2e-2 * scale, f"{name}: max-abs {float(err.max()):.3e} (ref max {float(ref.abs().max()):.2f})"
    assert float(err.mean()) <= 1e-3 * scale, f"{name}: mean-abs {float(err.mean()):.3e}"


def _lse_ok(lse, ref):
    fin = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert float((lse.cpu()[fin] - ref[fin]).abs().max()) <= 1e-4


@pytest.mark.parametrize("seqlens,Hk,G,d,W", [([700, 45, 300], 2, 2, 128, 128), ([1500], 1, 4, 128, 512), ([333], 2, 1, 64, 64),
                                              ([33, 70, 5, 128] * 10, 1, 4, 128, 64),
                                              ([400, 90], 1, 2, 256, 100)])       # head_dim 256: the block-major forward and backward
def test_sliding_window(seqlens, Hk, G, d, W):
    N = sum(seqlens)
    g = torch.Generator().manual_seed(N + W)
    q = torch.randn(N, Hk * G, d, generator=g).to(torch.bfloat16)
    k = torch.randn(N, Hk, d, generator=g).to(torch.bfloat16)
    v = torch.randn(N, Hk, d, generator=g).to(torch.bfloat16)
    do = torch.randn(N, Hk * G, d, generator=g).to(torch.bfloat16)
    cu = make_cu_seqlens(seqlens)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = orc.with_grads(orc.sliding_window_attention, q, k, v, do, cu, W)
    qc, kc, vc = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    o, lse = sliding_window_attention(qc, kc, vc, cu.to(DEV), W)
    o.backward(do.to(DEV))
    _tol_ok(o, o_ref, "o")
    _lse_ok(lse, lse_ref)
    _tol_ok(qc.grad, dq_ref, "dq")
    _tol_ok(kc.grad, dk_ref, "dk")
    _tol_ok(vc.grad, dv_ref, "dv")


@pytest.mark.parametrize("seqlens,Hk,G,d,ks,stride", [([2000, 20, 777], 2, 2, 128, 32, 16), ([4096], 1, 4, 128, 32, 16), ([500], 1, 1, 64, 16, 8)])
def test_compressed_branch(seqlens, Hk, G, d, ks, stride):
    N = sum(seqlens)
    cmp_lens = [max((L - ks) // stride + 1, 0) if L >= ks else 0 for L in seqlens]
    Nc = sum(cmp_lens)
    g = torch.Generator().manual_seed(N + ks)
    q = torch.randn(N, Hk * G, d, generator=g).to(torch.bfloat16)
    ck = torch.randn(Nc, Hk, d, generator=g).to(torch.bfloat16)
    cv = torch.randn(Nc, Hk, d, generator=g).to(torch.bfloat16)
    do = torch.randn(N, Hk * G, d, generator=g).to(torch.bfloat16)
    cu_q, cu_k = make_cu_seqlens(seqlens), make_cu_seqlens(cmp_lens)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = orc.with_grads(orc.compressed_attention, q, ck, cv, do, ks, stride, cu_q, cu_k)
    qc, kc, vc = (x.to(DEV).requires_grad_(True) for x in (q, ck, cv))
    o, lse = compressed_attention_core(qc, kc, vc, ks, stride, cu_q.to(DEV), cu_k.to(DEV), max(cmp_lens))
    o.backward(do.to(DEV))
    _tol_ok(o, o_ref, "o")
    _lse_ok(lse, lse_ref)
    _tol_ok(qc.grad, dq_ref, "dq")
    _tol_ok(kc.grad, dk_ref, "dk")
    _tol_ok(vc.grad, dv_ref, "dv")


@pytest.mark.parametrize("seqlens,Hk,G,d,W,dtype,qscale", [
    ([300, 41], 1, 3, 128, 100, torch.bfloat16, 1.0),       # 40 tokens per tile: 120 of the 128 tile rows are used
    ([513], 2, 8, 128, 64, torch.bfloat16, 1.0),
    ([260, 90], 1, 16, 64, 200, torch.float16, 1.0),        # 8 tokens per tile
    ([1200], 1, 2, 128, 1024, torch.bfloat16, 6.0),         # logits of magnitude ~70: the reference max of a row is raised
                                                            # while the accumulator already holds products (rescale in TMEM)
    ([900], 2, 4, 64, 300, torch.bfloat16, 5.0),
    ([5, 130, 64, 1, 257, 33] * 4, 2, 4, 128, 96, torch.bfloat16, 1.0),    # many short sequences: most tiles are partial
    ([17, 40, 3, 64, 129] * 14, 1, 2, 128, 50, torch.bfloat16, 1.0),       # 70 sequences: the tile lookup walks them 32 at a time
])
def test_query_major_forward_shapes(seqlens, Hk, G, d, W, dtype, qscale):
    """Forward of the query-tile-major kernel on group sizes / dtypes / logit ranges beyond the cases above, with q as a
    strided view of a fused projection (token stride > heads * d)."""
    N = sum(seqlens)
    g = torch.Generator().manual_seed(3 * N + W)
    fused = (torch.randn(N, 2 * Hk * G * d, generator=g) * qscale).to(dtype)
    q = fused[:, Hk * G * d :].view(N, Hk * G, d)
    k = torch.randn(N, Hk, d, generator=g).to(dtype)
    v = torch.randn(N, Hk, d, generator=g).to(dtype)
    cu = make_cu_seqlens(seqlens)
    o_ref, lse_ref = orc.sliding_window_attention(q.float(), k.float(), v.float(), cu, W)
    o, lse = sliding_window_attention(fused.to(DEV)[:, Hk * G * d :].view(N, Hk * G, d), k.to(DEV), v.to(DEV), cu.to(DEV), W)
    _tol_ok(o, o_ref, "o")
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert float((lse.cpu()[fin] - lse_ref[fin]).abs().max()) <= 1e-4 * max(1.0, float(lse_ref[fin].abs().max()))


def test_query_major_forward_rows_without_keys():
    """Tokens whose range is empty (kv_hi < kv_lo) get o = 0 and lse = -inf, also when a whole tile sees nothing."""
    from fsa.ops.range_attention import range_attention

    N, Hk, G, d = 400, 1, 2, 128
    g = torch.Generator().manual_seed(9)
    q = torch.randn(N, Hk * G, d, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(N, Hk, d, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(N, Hk, d, generator=g).to(torch.bfloat16).to(DEV)
    cu = make_cu_seqlens([N]).to(DEV)
    tok = torch.arange(N, dtype=torch.int32, device=DEV)
    hi = tok.clone()
    hi[:130] = -1                      # the first two tiles (64 tokens each) see nothing, the third partly
    hi[300:310] = -1
    lo = torch.clamp(tok - 50, min=0)
    o, lse = range_attention(q, k, v, cu, cu, lo, hi, (50 + 1 + 63) // 64 + 1)
    dead = hi < 0
    assert float(o[dead].abs().max()) == 0 and bool(torch.isinf(lse[:, dead]).all())
    # the rest against plain softmax attention over the same ranges
    qf, kf, vf = q.float().cpu(), k.float().cpu(), v.float().cpu()
    for t in (130, 200, 299, 310, 399):
        a, b = int(lo[t]), int(hi[t])
        for hq in range(Hk * G):
            s = (kf[a : b + 1, hq // G] @ qf[t, hq]) / d ** 0.5
            ref = torch.softmax(s, 0) @ vf[a : b + 1, hq // G]
            assert float((o[t, hq].float().cpu() - ref).abs().max()) <= 2e-2


@pytest.mark.parametrize("branch", ["window", "compressed"])
def test_query_major_kernels_at_full_length(branch):
    """One 32768-token sequence with the layer's group size (the length of the layer benchmark's sequences): o, lse and dq
    of sampled tokens against closed-form fp32 attention over the token's range; dv through the identity
    sum_rows(dv) = sum over tokens and heads of dO (every softmax row sums to one)."""
    from fsa.ops.range_attention import compressed_attention_core, sliding_window_attention

    L, Hk, G, d = 32768, 2, 4, 128
    g = torch.Generator().manual_seed(77)
    q = torch.randn(L, Hk * G, d, generator=g).to(torch.bfloat16)
    do = torch.randn(L, Hk * G, d, generator=g).to(torch.bfloat16)
    cu = make_cu_seqlens([L])
    if branch == "window":
        W = 512
        k = torch.randn(L, Hk, d, generator=g).to(torch.bfloat16)
        v = torch.randn(L, Hk, d, generator=g).to(torch.bfloat16)
        rng = lambda t: (max(0, t - W), t)
        qc, kc, vc = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
        o, lse = sliding_window_attention(qc, kc, vc, cu.to(DEV), W)
    else:
        ks, st = 32, 16
        nc = (L - ks) // st + 1
        k = torch.randn(nc, Hk, d, generator=g).to(torch.bfloat16)
        v = torch.randn(nc, Hk, d, generator=g).to(torch.bfloat16)
        rng = lambda t: (0, min((t - ks + 1) // st, nc - 1) if t >= ks - 1 else -1)
        qc, kc, vc = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
        o, lse = compressed_attention_core(qc, kc, vc, ks, st, cu.to(DEV), make_cu_seqlens([nc]).to(DEV), nc)
    o.backward(do.to(DEV))
    oc, lc, dqc = o.detach().float().cpu(), lse.float().cpu(), qc.grad.float().cpu()
    kf, vf, qf, dof = k.float(), v.float(), q.float(), do.float()
    scale = d ** -0.5
    toks = [0, 1, 30, 31, 32, 63, 64, 511, 512, 513, 4095, 4096, 20000, L - 2, L - 1] + torch.randint(0, L, (60,), generator=g).tolist()
    for t in toks:
        a, b = rng(t)
        for hq in (0, 3, 5):
            h = hq // G
            if b < a:
                assert float(oc[t, hq].abs().max()) == 0 and lc[hq, t] == float("-inf") and float(dqc[t, hq].abs().max()) == 0
                continue
            s = (kf[a : b + 1, h] @ qf[t, hq]) * scale
            p = torch.softmax(s, 0)
            o_ref = p @ vf[a : b + 1, h]
            lse_ref = torch.logsumexp(s, 0) * 1.4426950408889634
            dp = vf[a : b + 1, h] @ dof[t, hq]
            ds = p * (dp - (o_ref * dof[t, hq]).sum()) * scale
            dq_ref = ds @ kf[a : b + 1, h]
            assert float((oc[t, hq] - o_ref).abs().max()) <= 2e-2 * max(1.0, float(o_ref.abs().max()))
            assert abs(float(lc[hq, t] - lse_ref)) <= 1e-3
            assert float((dqc[t, hq] - dq_ref).abs().max()) <= 2e-2 * max(1.0, float(dq_ref.abs().max()))
    # dv: every probability row sums to one, so the column sums of dv equal those of dO over the tokens that see a key
    seen = torch.tensor([rng(t)[1] >= rng(t)[0] for t in range(L)])
    want = dof[seen].reshape(-1, Hk, G, d).sum((0, 2))
    got = vc.grad.float().cpu().sum(0)
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max()) + 2.0


def test_fp16_forward_and_backward():
    """fp16 inputs through the query-tile-major forward / dQ kernels and the block-major dK/dV kernel."""
    seqlens, Hk, G, d, W = [300, 130], 2, 4, 128, 100
    N = sum(seqlens)
    g = torch.Generator().manual_seed(21)
    q, do = (torch.randn(N, Hk * G, d, generator=g).to(torch.float16) for _ in range(2))
    k, v = (torch.randn(N, Hk, d, generator=g).to(torch.float16) for _ in range(2))
    cu = make_cu_seqlens(seqlens)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = orc.with_grads(orc.sliding_window_attention, q, k, v, do, cu, W)
    qc, kc, vc = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    o, lse = sliding_window_attention(qc, kc, vc, cu.to(DEV), W)
    o.backward(do.to(DEV))
    _tol_ok(o, o_ref, "o")
    _lse_ok(lse, lse_ref)
    _tol_ok(qc.grad, dq_ref, "dq")
    _tol_ok(kc.grad, dk_ref, "dk")
    _tol_ok(vc.grad, dv_ref, "dv")


def test_sliding_window_against_flash_attn():
    """The sliding-window branch against the very call the reference makes (fsa/module/fsa.py:149-159):
    ``flash_attn_varlen_func(q, k, v, cu, cu, max, max, causal=True, window_size=(W, -1))`` of the third-party
    flash-attn package (2.8.3 in this image), forward and backward, bf16 on both sides.  Skipped where that package has no
    kernel for the GPU."""
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"flash_attn not importable: {e}")
    seqlens, Hk, G, d, W = [700, 45, 300, 1111], 2, 4, 128, 512
    N = sum(seqlens)
    g = torch.Generator().manual_seed(31)
    q, do = (torch.randn(N, Hk * G, d, generator=g).to(torch.bfloat16).to(DEV) for _ in range(2))
    k, v = (torch.randn(N, Hk, d, generator=g).to(torch.bfloat16).to(DEV) for _ in range(2))
    cu = make_cu_seqlens(seqlens).to(DEV)
    qr, kr, vr = (x.clone().requires_grad_(True) for x in (q, k, v))
    try:
        o_ref = flash_attn_varlen_func(qr, kr, vr, cu, cu, max(seqlens), max(seqlens), causal=True, window_size=(W, -1))
        o_ref.backward(do)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"flash_attn does not run on this GPU: {type(e).__name__}")
    qc, kc, vc = (x.clone().requires_grad_(True) for x in (q, k, v))
    o, _ = sliding_window_attention(qc, kc, vc, cu, W)
    o.backward(do)
    # two bf16 implementations of the same function: each rounds its output once
    for name, got, ref in (("o", o, o_ref), ("dq", qc.grad, qr.grad), ("dk", kc.grad, kr.grad), ("dv", vc.grad, vr.grad)):
        err = (got.float() - ref.float()).abs()
        scale = max(1.0, float(ref.float().abs().max()) / 2.0)
        assert float(err.max()) <= 3e-2 * scale, f"{name}: max-abs {float(err.max()):.3e}"
        assert float(err.mean()) <= 1.5e-3 * scale, f"{name}: mean-abs {float(err.mean()):.3e}"


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_shapes_forward_backward(seed):
    """Seeded random problems (sequence counts and lengths, group sizes incl. those that leave tile rows unused, head
    sizes, windows shorter and longer than a K/V tile, both dtypes) through both branches against the oracle."""
    rnd = torch.Generator().manual_seed(1000 + seed)
    ri = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=rnd))
    G = [1, 2, 3, 4, 6, 8, 16][ri(0, 6)]
    Hk = ri(1, 2)
    d = [64, 128][ri(0, 1)]
    dtype = [torch.bfloat16, torch.float16][ri(0, 1)]
    seqlens = [ri(1, 400) for _ in range(ri(1, 5))]
    N = sum(seqlens)
    q, do = (torch.randn(N, Hk * G, d, generator=rnd).to(dtype) for _ in range(2))
    cu = make_cu_seqlens(seqlens)
    if seed % 2 == 0:
        W = ri(1, 300)
        k, v = (torch.randn(N, Hk, d, generator=rnd).to(dtype) for _ in range(2))
        ref = orc.with_grads(orc.sliding_window_attention, q, k, v, do, cu, W)
        qc, kc, vc = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
        o, lse = sliding_window_attention(qc, kc, vc, cu.to(DEV), W)
    else:
        ks, st = [(32, 16), (16, 8), (32, 32)][ri(0, 2)]
        cmp_lens = [(L - ks) // st + 1 if L >= ks else 0 for L in seqlens]
        if sum(cmp_lens) == 0:
            seqlens[0] += ks
            N = sum(seqlens)
            q, do = (torch.randn(N, Hk * G, d, generator=rnd).to(dtype) for _ in range(2))
            cu = make_cu_seqlens(seqlens)
            cmp_lens = [(L - ks) // st + 1 if L >= ks else 0 for L in seqlens]
        Nc = sum(cmp_lens)
        k, v = (torch.randn(Nc, Hk, d, generator=rnd).to(dtype) for _ in range(2))
        cu_k = make_cu_seqlens(cmp_lens)
        ref = orc.with_grads(orc.compressed_attention, q, k, v, do, ks, st, cu, cu_k)
        qc, kc, vc = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
        o, lse = compressed_attention_core(qc, kc, vc, ks, st, cu.to(DEV), cu_k.to(DEV), max(cmp_lens))
    o.backward(do.to(DEV))
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = ref
    tag = f"seed {seed}: G={G} Hk={Hk} d={d} {dtype} seqlens={seqlens}"
    _tol_ok(o, o_ref, "o " + tag)
    _lse_ok(lse, lse_ref)
    _tol_ok(qc.grad, dq_ref, "dq " + tag)
    _tol_ok(kc.grad, dk_ref, "dk " + tag)
    _tol_ok(vc.grad, dv_ref, "dv " + tag)
