"""GPU parity of the one-step decode: each device operator against its CPU restatement, the whole step against the
decode oracle (= prefill row t), the layer's decode step against the prefill layer's last row, and the
reference-signature forward against the stateful step."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fsa.module.fsa import FlashSparseAttention  # noqa: E402
from fsa.module.rope import RopeConfig  # noqa: E402
from fsa.ops.linear_compress import compressed_seqlens, linear_compress  # noqa: E402
from fsa_preview.module import FlashSparseAttentionDecode, FlashSparseAttentionDecodeKernel, GraphedStep  # noqa: E402
from fsa_preview.ops import _compressed_attention_decode, _topk_sparse_attention_decode  # noqa: E402
from fsa_preview.ops.decode import CudaDecodeOps  # noqa: E402
from oracle.decode_oracle import OracleDecodeOps, decode_branches_ref  # noqa: E402

DEV = "cuda:0"


def _close(got, ref, what, max_tol=2e-2, mean_tol=1e-3):
    got, ref = got.float().cpu(), ref.float().cpu()
    scale = max(1.0, float(ref.detach().abs().max()) / 2)
    err = (got - ref).abs()
    assert float(err.max()) <= max_tol * scale, f"{what}: max-abs {float(err.max()):.3e}"
    assert float(err.mean()) <= mean_tol * scale, f"{what}: mean-abs {float(err.mean()):.3e}"


@pytest.mark.parametrize("G,D,dtype", [(1, 128, torch.bfloat16), (2, 128, torch.bfloat16), (4, 128, torch.bfloat16),
                                       (8, 64, torch.float16), (16, 128, torch.bfloat16), (4, 64, torch.bfloat16)])
def test_attn_partial_and_merge(G, D, dtype):
    torch.manual_seed(G * 100 + D)
    B, Hk, R, chunk, nchunk, rows = 3, 2, 3, 32, 3, 400
    Hq = Hk * G
    q = torch.randn(B, Hq, D).to(dtype)
    k = torch.randn(rows, Hk, D).to(dtype)
    v = torch.randn(rows, Hk, D).to(dtype)
    lo = torch.randint(0, rows - chunk * nchunk, (B, Hk, R), dtype=torch.int32)
    ln = torch.randint(0, chunk * nchunk + 1, (B, Hk, R), dtype=torch.int32)
    lo[0, 0, 1] = -1                                                    # an empty range
    ln[1, 1, 0] = 0                                                     # a zero-length range
    ln[2, 0, 2] = 1
    hi = torch.where(lo >= 0, lo + ln, lo)
    ref_o, ref_ml, ref_s = OracleDecodeOps().attn_partial(q, k, v, lo, hi, chunk, nchunk, D ** -0.5, want_scores=True)
    ops = CudaDecodeOps()
    o, ml, s = ops.attn_partial(q.to(DEV), k.to(DEV), v.to(DEV), lo.to(DEV), hi.to(DEV), chunk, nchunk, D ** -0.5, want_scores=True)
    torch.cuda.synchronize()
    live = ref_ml[..., 1] > 0
    assert torch.equal((ml[..., 1] > 0).cpu(), live)
    torch.testing.assert_close(ml.cpu()[live], ref_ml[live], rtol=1e-4, atol=1e-4)
    # P is rounded to the input type before P V (as the prefill kernels and the reference do): bf16-sized errors
    torch.testing.assert_close(o.cpu()[live], ref_o[live], rtol=2e-2, atol=3e-2)
    for b in range(B):
        for h in range(Hk):
            n = int(hi[b, h, 0] - lo[b, h, 0]) if lo[b, h, 0] >= 0 else 0
            torch.testing.assert_close(s[b, h, :n].cpu(), ref_s[b, h, :n], rtol=1e-4, atol=1e-4)
    for p0, pn in ((0, None), (2, 4)):
        go, glse = ops.lse_merge(o, ml, dtype, p0, pn)
        ro, rlse = OracleDecodeOps().lse_merge(ref_o, ref_ml, torch.float32, p0, pn)
        _close(go, ro, "merged o")
        fin = torch.isfinite(rlse)
        assert torch.equal(torch.isfinite(glse).cpu(), fin)
        torch.testing.assert_close(glse.cpu()[fin], rlse[fin], rtol=1e-4, atol=1e-4)


def test_decode_status_word_is_clean():
    from ctypes import byref, c_int

    from fsa import _lib

    st = c_int(-1)
    _lib.check(_lib.lib().fsa_decode_read_status(byref(st)), "fsa_decode_read_status")
    assert st.value == 0


@pytest.mark.parametrize("G,D,chunk,nchunk", [(4, 128, 512, 2), (16, 128, 256, 3), (2, 64, 192, 2), (8, 64, 64, 1)])
def test_attn_partial_long_chunks(G, D, chunk, nchunk):
    """Chunks of several 64-key pipeline stages (more stages than the ring holds), ragged tails."""
    torch.manual_seed(G + D + chunk)
    B, Hk, R, rows = 2, 2, 2, 3000
    Hq = Hk * G
    q = torch.randn(B, Hq, D).to(torch.bfloat16)
    k = torch.randn(rows, Hk, D).to(torch.bfloat16)
    v = torch.randn(rows, Hk, D).to(torch.bfloat16)
    lo = torch.randint(0, rows - chunk * nchunk, (B, Hk, R), dtype=torch.int32)
    ln = torch.randint(1, chunk * nchunk + 1, (B, Hk, R), dtype=torch.int32)
    ln[0, 0, 0] = chunk * nchunk
    lo[1, 1, 1] = rows - 37                                             # a range that ends at the last row of the tensor
    ln[1, 1, 1] = 37
    hi = lo + ln
    ref_o, ref_ml, ref_s = OracleDecodeOps().attn_partial(q, k, v, lo, hi, chunk, nchunk, D ** -0.5, want_scores=True)
    ops = CudaDecodeOps()
    o, ml, s = ops.attn_partial(q.to(DEV), k.to(DEV), v.to(DEV), lo.to(DEV), hi.to(DEV), chunk, nchunk, D ** -0.5, want_scores=True)
    go, glse = ops.lse_merge(o, ml, torch.float32)
    ro, rlse = OracleDecodeOps().lse_merge(ref_o, ref_ml, torch.float32)
    _close(go, ro, "merged o")
    torch.testing.assert_close(glse.cpu(), rlse, rtol=1e-4, atol=1e-4)
    for b in range(B):
        for h in range(Hk):
            n = int(ln[b, h, 0])
            torch.testing.assert_close(s[b, h, :n].cpu(), ref_s[b, h, :n], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("rpp,R", [(2, 5), (4, 8), (4, 25)])
def test_attn_partial_ranges_per_partial(rpp, R):
    """Several ranges folded into one partial (one online softmax over their keys), empty ranges in between."""
    torch.manual_seed(rpp * 10 + R)
    B, Hk, G, D, rows, piece = 2, 2, 4, 128, 2000, 64
    Hq = Hk * G
    q = torch.randn(B, Hq, D).to(torch.bfloat16)
    k = torch.randn(rows, Hk, D).to(torch.bfloat16)
    v = torch.randn(rows, Hk, D).to(torch.bfloat16)
    lo = torch.randint(0, rows - piece, (B, Hk, R), dtype=torch.int32)
    ln = torch.randint(1, piece + 1, (B, Hk, R), dtype=torch.int32)
    lo[0, 0, 1] = -1
    lo[1, 1, :rpp] = -1                                                  # a partial with no key at all
    hi = torch.where(lo >= 0, lo + ln, lo)
    ref_o, ref_ml, _ = OracleDecodeOps().attn_partial(q, k, v, lo, hi, piece, 1, D ** -0.5, rpp=rpp)
    ops = CudaDecodeOps()
    o, ml, _ = ops.attn_partial(q.to(DEV), k.to(DEV), v.to(DEV), lo.to(DEV), hi.to(DEV), piece, 1, D ** -0.5, rpp=rpp)
    assert o.shape == ref_o.shape
    live = ref_ml[..., 1] > 0
    assert torch.equal((ml[..., 1] > 0).cpu(), live)
    torch.testing.assert_close(ml.cpu()[live], ref_ml[live], rtol=1e-4, atol=1e-4)
    go, glse = ops.lse_merge(o, ml, torch.float32)
    ro, rlse = OracleDecodeOps().lse_merge(ref_o, ref_ml, torch.float32)
    _close(go, ro, "merged o")
    torch.testing.assert_close(glse.cpu(), rlse, rtol=1e-4, atol=1e-4)


def test_select_topk_and_ranges_bit_exact():
    torch.manual_seed(7)
    B, Hk, G, ks, st, BK, T, W = 5, 2, 2, 32, 16, 64, 6, 100
    seq_len = torch.tensor([1, 40, 700, 1500, 2048], dtype=torch.int32)
    ncmp = torch.clamp((seq_len - ks) // st + 1, min=0).to(torch.int32)
    ld = 128
    scores = torch.randn(B, Hk, ld) * 3
    lse = torch.randn(B, Hk * G) + 6
    max_blocks = 2048 // BK
    ref = OracleDecodeOps().select_topk(scores, ld, ld, 0, lse, seq_len, ncmp, Hk, ks, st, BK, 1, 2, T, max_blocks)
    ops = CudaDecodeOps()
    got = ops.select_topk(scores.to(DEV), ld, ld, 0, lse.to(DEV), seq_len.to(DEV), ncmp.to(DEV), Hk, ks, st, BK, 1, 2, T, max_blocks)
    assert torch.equal(got.cpu(), ref)
    # shard-major scores (two shards of 64 compressed tokens) give the same ids
    sh = torch.stack([scores[..., :64], scores[..., 64:]]).contiguous()
    got2 = ops.select_topk(sh.to(DEV), 64, 64, B * Hk * 64, lse.to(DEV), seq_len.to(DEV), ncmp.to(DEV), Hk, ks, st, BK, 1, 2, T, max_blocks)
    assert torch.equal(got2.cpu(), ref)
    row0 = torch.arange(B, dtype=torch.int32) * 3000
    for s_lo, s_hi in ((0, 2**31 - 1), (0, 1024), (1024, 2048)):
        npieces = -(-(W + 1) // BK)
        rl, rh = OracleDecodeOps().ranges(ref, seq_len, row0, Hk, T, BK, W, BK, npieces, s_lo, s_hi)
        gl, gh = ops.ranges(ref.to(DEV), seq_len.to(DEV), row0.to(DEV), Hk, T, BK, W, BK, npieces, s_lo, s_hi)
        assert torch.equal(gl.cpu(), rl) and torch.equal(gh.cpu(), rh)


@pytest.mark.parametrize("max_len", [400, 40000, 131136, 160000])
def test_select_topk_long_rows_bit_exact(max_len):
    """Rows of up to 2500 candidate blocks (the benchmark's cache length and beyond) against the oracle on identical
    scores."""
    torch.manual_seed(max_len)
    B, Hk, G, ks, st, BK, T = 2, 1, 2, 32, 16, 64, 16
    seq_len = torch.tensor([max_len, max(max_len // 3, 33)], dtype=torch.int32)
    ncmp = torch.clamp((seq_len - ks) // st + 1, min=0).to(torch.int32)
    ld = int(ncmp.max()) + 5
    scores = torch.randn(B, Hk, ld) * 2
    lse = torch.full((B, Hk * G), 8.0)
    max_blocks = -(-max_len // BK)
    ref = OracleDecodeOps().select_topk(scores, ld, ld, 0, lse, seq_len, ncmp, Hk, ks, st, BK, 1, 2, T, max_blocks)
    got = CudaDecodeOps().select_topk(scores.to(DEV), ld, ld, 0, lse.to(DEV), seq_len.to(DEV), ncmp.to(DEV), Hk, ks, st, BK, 1, 2, T,
                                      max_blocks)
    assert torch.equal(got.cpu(), ref)


CFG = dict(kernel_size=32, kernel_stride=16, block_size=64, topk=4, init_blocks=1, local_blocks=2, window_size=100)


def _branch_check(q, ks_, vs_, cks, cvs, got, cfg):
    ref = decode_branches_ref(q.float().cpu(), ks_, vs_, cks, cvs, cfg)
    same = (got[6].cpu() == ref[6]).float().mean().item()
    assert same >= 0.97, f"top-k ids agree on {same:.3f} only"
    ref = decode_branches_ref(q.float().cpu(), ks_, vs_, cks, cvs, cfg, topk_idx=got[6].cpu())
    for i, name in enumerate(("o_cmp", "o_sel", "o_win")):
        _close(got[i], ref[i], name)
        fin = torch.isfinite(ref[3 + i])
        assert torch.equal(torch.isfinite(got[3 + i]).cpu(), fin)
        torch.testing.assert_close(got[3 + i].cpu()[fin], ref[3 + i][fin], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("G", [1, 4])
def test_decode_kernel_module_steps(G):
    """Cache prefilled with ragged lengths (one shorter than a compression window, one crossing windows), then
    several steps; every step's branches against the decode oracle on the full token history."""
    torch.manual_seed(11 + G)
    Hk, D, steps = 2, 128, 18
    Hq = Hk * G
    seqlens = [300, 7, 31, 1000]
    B = len(seqlens)
    mod = FlashSparseAttentionDecodeKernel(Hq * D, Hq, Hk, D, **CFG).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        for p in (mod.compress_key, mod.compress_value, mod.intra_block_pe):
            p.copy_(torch.randn_like(p) * 0.05)
        mod.gate[0].weight.copy_(torch.randn_like(mod.gate[0].weight) * 0.02)
    k = [torch.randn(L + steps, Hk, D).to(torch.bfloat16) for L in seqlens]
    v = [torch.randn(L + steps, Hk, D).to(torch.bfloat16) for L in seqlens]
    ks, st = CFG["kernel_size"], CFG["kernel_stride"]
    cache = mod.new_cache(B, 1100, device=DEV)
    kp = torch.cat([x[:L] for x, L in zip(k, seqlens)]).to(DEV)
    vp = torch.cat([x[:L] for x, L in zip(v, seqlens)]).to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32, device=DEV)
    ck, _ = linear_compress(kp, mod.compress_key, cu, ks, st, mod.intra_block_pe, seqlens)
    cv, _ = linear_compress(vp, mod.compress_value, cu, ks, st, None, seqlens)
    cache.load(kp, kp, vp, ck, cv, seqlens, compressed_seqlens(seqlens, ks, st))
    from fsa_preview.ops.decode import nsa_decode_attention

    for s in range(steps):
        q = torch.randn(B, Hq, D).to(torch.bfloat16).to(DEV)
        kn = torch.stack([x[L + s] for x, L in zip(k, seqlens)]).to(DEV)
        vn = torch.stack([x[L + s] for x, L in zip(v, seqlens)]).to(DEV)
        out = mod.step(q, kn, vn, cache)
        assert out.shape == (B, Hq * D)
        got = nsa_decode_attention(q, cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0, cache.cmp_row0,
                                   max_len=cache.max_len, **CFG)
        if s % 6 in (0, 1) or s == steps - 1:
            lens = [L + s + 1 for L in seqlens]
            ks_ = [x[:L] for x, L in zip(k, lens)]
            vs_ = [x[:L] for x, L in zip(v, lens)]
            cuL = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
            ckf, ccu = linear_compress(torch.cat(ks_).to(DEV), mod.compress_key, cuL, ks, st, mod.intra_block_pe, lens)
            cvf, _ = linear_compress(torch.cat(vs_).to(DEV), mod.compress_value, cuL, ks, st, None, lens)
            ccu = ccu.tolist()
            cks = [ckf[ccu[b] : ccu[b + 1]].detach().cpu() for b in range(B)]
            cvs = [cvf[ccu[b] : ccu[b + 1]].detach().cpu() for b in range(B)]
            _branch_check(q, ks_, vs_, cks, cvs, got, CFG)
            gate = mod.gate(q.view(B, -1)).float()
            mix = gate[:, 0:1, None] * got[0].float() + gate[:, 1:2, None] * got[1].float() + gate[:, 2:3, None] * got[2].float()
            _close(out, mix.flatten(1), "gate mix")
    assert cache.host_len == [L + steps for L in seqlens]


def test_decode_layer_equals_prefill_last_row():
    """decode(t) == prefill row t: the decode layer after a prefill of L tokens, stepping token L, against the
    prefill layer run on L + 1 tokens."""
    torch.manual_seed(5)
    hidden, Hq, Hk, D = 256, 4, 2, 128
    cfg = dict(kernel_size=32, kernel_stride=16, block_size=64, topk=4, init_blocks=1, local_blocks=2, window_size=64)
    rope = RopeConfig(max_position_embeddings=4096, head_dim=D, rope_theta=500000.0)
    pre = FlashSparseAttention(hidden, Hq, Hk, D, rope_config=rope, **cfg).to(DEV).to(torch.bfloat16)
    dec = FlashSparseAttentionDecode(hidden, Hq, Hk, D, rope_config=rope, **cfg).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        for p in pre.parameters():
            p.copy_(torch.randn_like(p) * 0.05)
    dec.load_state_dict(pre.state_dict())
    seqlens = [257, 40, 640]
    B = len(seqlens)
    xs = [torch.randn(L + 2, hidden).to(torch.bfloat16).to(DEV) for L in seqlens]
    cache = dec.new_cache(B, 1024, device=DEV)
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32, device=DEV)
    dec.prefill_cache(cache, torch.cat([x[:L] for x, L in zip(xs, seqlens)]), cu, seqlens)
    for s in range(2):
        y = dec.step(torch.stack([x[L + s] for x, L in zip(xs, seqlens)]), cache)
        lens = [L + s + 1 for L in seqlens]
        cuL = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
        with torch.no_grad():
            full = pre(torch.cat([x[:L] for x, L in zip(xs, lens)]), cuL)
        last = (cuL[1:] - 1).long()
        assert torch.equal(dec.last_topk_idx.transpose(0, 1), pre.last_topk_idx[:, last])
        _close(y, full[last], f"decode step {s} vs prefill row")
    # the stateless reference signature on one sequence gives the same row
    L = seqlens[0] + 2
    x = xs[0]
    k_raw = dec.proj_k(x[: L - 1]).view(-1, Hk, D)
    v_raw = dec.proj_v(x[: L - 1]).view(-1, Hk, D)
    cu1 = torch.tensor([0, L - 1], dtype=torch.int32, device=DEV)
    ck, _ = linear_compress(k_raw, dec.compress_key, cu1, cfg["kernel_size"], cfg["kernel_stride"], dec.intra_block_pe, [L - 1])
    cv, _ = linear_compress(v_raw, dec.compress_value, cu1, cfg["kernel_size"], cfg["kernel_stride"], None, [L - 1])
    y1 = dec(x[L - 1 : L], torch.tensor([0, 1], dtype=torch.int32, device=DEV), torch.tensor([0, L], dtype=torch.int32, device=DEV),
             k_raw, v_raw, ck, cv)
    _close(y1, y[0:1], "stateless forward vs step")


def test_reference_named_ops():
    torch.manual_seed(3)
    B, Hk, G, D, ks, st, BK, T = 2, 2, 2, 128, 32, 16, 64, 4
    Hq = Hk * G
    lens = [500, 90]
    k = [torch.randn(L, Hk, D).to(torch.bfloat16) for L in lens]
    v = [torch.randn(L, Hk, D).to(torch.bfloat16) for L in lens]
    clens = compressed_seqlens(lens, ks, st)
    ck = [torch.randn(n, Hk, D).to(torch.bfloat16) for n in clens]
    cv = [torch.randn(n, Hk, D).to(torch.bfloat16) for n in clens]
    q = torch.randn(B, Hq, D).to(torch.bfloat16)
    cfg = dict(kernel_size=ks, kernel_stride=st, block_size=BK, topk=T, init_blocks=1, local_blocks=2, window_size=64)
    cuq = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    cuk = torch.tensor([0, lens[0], sum(lens)], dtype=torch.int32, device=DEV)
    cuc = torch.tensor([0, clens[0], sum(clens)], dtype=torch.int32, device=DEV)
    t = torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=DEV)
    o, idx = _compressed_attention_decode(q.to(DEV), torch.cat(ck).to(DEV), torch.cat(cv).to(DEV), ks, st, BK, T, cuq, cuc, 1, max(clens),
                                          None, 1, 2, query_start_index=t)
    ref = decode_branches_ref(q.float(), k, v, ck, cv, cfg)
    _close(o, ref[0], "o_cmp")
    assert (idx.transpose(0, 1).cpu() == ref[6]).float().mean() >= 0.9
    o_sel = _topk_sparse_attention_decode(q.to(DEV), torch.cat(k).to(DEV), torch.cat(v).to(DEV), idx, BK, cuq, cuk, 1, max(lens))
    ref = decode_branches_ref(q.float(), k, v, ck, cv, cfg, topk_idx=idx.transpose(0, 1).cpu())
    _close(o_sel, ref[1], "o_sel")


def test_graphed_step_matches_eager_step():
    """The captured step replays to the same outputs and cache state as the eager step, across a compression boundary."""
    torch.manual_seed(21)
    Hk, G, D, steps = 2, 4, 128, 20
    Hq = Hk * G
    seqlens = [100, 45, 31]
    B = len(seqlens)
    mod = FlashSparseAttentionDecodeKernel(Hq * D, Hq, Hk, D, **CFG).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(torch.randn_like(p) * 0.05)
    ks, st = CFG["kernel_size"], CFG["kernel_stride"]
    kp = torch.randn(sum(seqlens), Hk, D).to(torch.bfloat16).to(DEV)
    vp = torch.randn(sum(seqlens), Hk, D).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32, device=DEV)
    ck, _ = linear_compress(kp, mod.compress_key, cu, ks, st, mod.intra_block_pe, seqlens)
    cv, _ = linear_compress(vp, mod.compress_value, cu, ks, st, None, seqlens)
    caches = []
    for _ in range(2):
        c = mod.new_cache(B, 256, device=DEV)
        c.load(kp, kp, vp, ck.detach(), cv.detach(), seqlens, compressed_seqlens(seqlens, ks, st))
        caches.append(c)
    ins = [torch.randn(steps, B, H, D).to(torch.bfloat16).to(DEV) for H in (Hq, Hk, Hk)]
    graphed = GraphedStep(mod.step, caches[1], [x[0] for x in ins])
    for s in range(steps):
        a = mod.step(ins[0][s], ins[1][s], ins[2][s], caches[0])
        b = graphed(ins[0][s], ins[1][s], ins[2][s])
        assert torch.equal(a, b), f"step {s}"
    assert torch.equal(caches[0].seq_len, caches[1].seq_len) and caches[0].host_len == caches[1].host_len
    for n in ("k", "v", "cmp_k", "cmp_v"):
        x, y = getattr(caches[0], n), getattr(caches[1], n)
        assert torch.equal(x[:-1], y[:-1]), n
