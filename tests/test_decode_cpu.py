"""CPU tests of the decode row: the decode oracle against the prefill oracles (row t = L - 1), the incremental
compressor against the prefill compressor, the cache + step logic on the CPU restatement of the device operators,
and the KV-sequence sharding protocol on two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from fsa.ops.linear_compress import compressed_seqlens
from fsa.ops.linear_compress import linear_compress_gemm as linear_compress   # CPU tensors: the library-GEMM formulation
from fsa_preview.cache import DecodeCache
from fsa_preview.ops.compat import _linear_compress_decode
from fsa_preview.ops.decode import Shard, nsa_decode_attention, shard_plan
from oracle.decode_oracle import OracleDecodeOps, decode_branches_ref
from oracle.nsa_layer_oracle import LOG2E, select_topk_ref
from oracle.range_attn_oracle import compressed_attention as cmp_attn_ref
from oracle.range_attn_oracle import sliding_window_attention as win_attn_ref
from oracle.sel_attn_oracle import sel_attn_forward

CFG = dict(kernel_size=16, kernel_stride=8, block_size=16, topk=4, init_blocks=1, local_blocks=2, window_size=24)


def _rand_seqs(seqlens, Hk, d, seed):
    g = torch.Generator().manual_seed(seed)
    k = [torch.randn(L, Hk, d, generator=g) for L in seqlens]
    v = [torch.randn(L, Hk, d, generator=g) for L in seqlens]
    return k, v


def _compress(xs, w, ks, st):
    out = []
    for x in xs:
        n = (x.shape[0] - ks) // st + 1 if x.shape[0] >= ks else 0
        H, d = x.shape[1], x.shape[2]
        rows = [torch.einsum("khd,hkde->he", x[c * st : c * st + ks], w.view(H, ks, d, d)) for c in range(n)]
        out.append(torch.stack(rows) if rows else x.new_zeros((0, H, d)))
    return out


def test_decode_oracle_equals_prefill_oracle_last_row():
    torch.manual_seed(0)
    Hq, Hk, d = 4, 2, 16
    seqlens = [70, 9, 33]
    ks, st, BK, T, W = (CFG[n] for n in ("kernel_size", "kernel_stride", "block_size", "topk", "window_size"))
    k, v = _rand_seqs(seqlens, Hk, d, 1)
    wk, wv = torch.randn(Hk, ks * d, d) * 0.1, torch.randn(Hk, ks * d, d) * 0.1
    ck, cv = _compress(k, wk, ks, st), _compress(v, wv, ks, st)
    q_full = torch.randn(sum(seqlens), Hq, d)
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32)
    clens = [c.shape[0] for c in ck]
    ccu = torch.tensor([0] + list(torch.tensor(clens).cumsum(0)), dtype=torch.int32)
    last = (cu[1:] - 1).long()
    oc, osel, ow, lc, ls, lw, idx = decode_branches_ref(q_full[last], k, v, ck, cv, CFG)
    # prefill oracles over the whole batch, last row of every sequence
    K, V, CK, CV = torch.cat(k), torch.cat(v), torch.cat(ck), torch.cat(cv)
    o_ref, lse_ref = cmp_attn_ref(q_full, CK, CV, ks, st, cu, ccu)
    torch.testing.assert_close(oc, o_ref[last], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lc, lse_ref[:, last].t(), rtol=1e-5, atol=1e-5)
    G = Hq // Hk
    for b, L in enumerate(seqlens):
        qs, cs = int(cu[b]), int(ccu[b])
        for h in range(Hk):
            qk = q_full[qs : qs + L, h * G] @ CK[cs : cs + clens[b], h].t() if clens[b] else torch.zeros(L, 0)
            ids = select_topk_ref(qk, lse_ref[h * G, qs : qs + L], L, clens[b], d ** -0.5, ks, st, BK, 1, 2, -(-max(seqlens) // BK), T)
            assert ids[L - 1].tolist() == idx[b, h].tolist()
    topk_full = torch.zeros(Hk, sum(seqlens), T, dtype=torch.int32)
    topk_full[:, :, 1:] = -1
    topk_full[:, last] = idx.transpose(0, 1)
    o_ref, lse_ref = sel_attn_forward(q_full, K, V, topk_full, BK, cu)
    torch.testing.assert_close(osel, o_ref[last], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ls, lse_ref[:, last].t(), rtol=1e-5, atol=1e-5)
    o_ref, lse_ref = win_attn_ref(q_full, K, V, cu, W)
    torch.testing.assert_close(ow, o_ref[last], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lw, lse_ref[:, last].t(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("L", [31, 32, 33, 48, 64, 65])
def test_incremental_compressor_matches_prefill(L):
    """prefill(L) == prefill(L-1) + one decode step of the compressor (the reference's own check,
    test/test_cmp_attn_decode.py:212-232, which states rtol 1e-4 / atol 1e-5)."""
    torch.manual_seed(L)
    H, d, ks, st = 2, 16, 32, 16
    x = torch.randn(L, H, d).to(torch.bfloat16)
    w = (torch.randn(H, ks * d, d) * 0.05).to(torch.bfloat16)
    pe = (torch.randn(H, ks, d) * 0.05).to(torch.bfloat16)
    cu = torch.tensor([0, L], dtype=torch.int32)
    full, _ = linear_compress(x, w, cu, ks, st, pe, [L])
    prev, _ = linear_compress(x[: L - 1], w, torch.tensor([0, L - 1], dtype=torch.int32), ks, st, pe, [L - 1])
    nbuf = min(ks - 1, L - 1)
    new = _linear_compress_decode(x[L - 1 :], w, ks, st, pe, L - 1, x[L - 1 - nbuf : L - 1])
    got = torch.cat([prev, new], 0) if new is not None else prev
    assert got.shape == full.shape
    assert (new is not None) == (L >= ks and (L - ks) % st == 0)
    torch.testing.assert_close(got.float(), full.float(), rtol=1e-4, atol=1e-5)


def _make_problem(seed, seqlens, Hq, Hk, d, steps):
    g = torch.Generator().manual_seed(seed)
    ks = CFG["kernel_size"]
    B = len(seqlens)
    k = [torch.randn(L + steps, Hk, d, generator=g).to(torch.bfloat16) for L in seqlens]
    v = [torch.randn(L + steps, Hk, d, generator=g).to(torch.bfloat16) for L in seqlens]
    q = torch.randn(steps, B, Hq, d, generator=g).to(torch.bfloat16)
    wk = (torch.randn(Hk, ks * d, d, generator=g) * 0.1).to(torch.bfloat16)
    wv = (torch.randn(Hk, ks * d, d, generator=g) * 0.1).to(torch.bfloat16)
    pe = (torch.randn(Hk, ks, d, generator=g) * 0.1).to(torch.bfloat16)
    return q, k, v, wk, wv, pe


def _run_steps(shard, seqlens, steps, q, k, v, wk, wv, pe, max_len, always_compress=False):
    """Prefill a cache from the first L_b tokens, then decode ``steps`` tokens; returns the branch outputs per step."""
    ks, st = CFG["kernel_size"], CFG["kernel_stride"]
    B, Hk, d = len(seqlens), k[0].shape[1], k[0].shape[2]
    cache = DecodeCache(B, max_len, Hk, d, ks, st, torch.bfloat16, "cpu", shard)
    cache.always_compress = always_compress
    kp = torch.cat([x[:L] for x, L in zip(k, seqlens)])
    vp = torch.cat([x[:L] for x, L in zip(v, seqlens)])
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32)
    ck, _ = linear_compress(kp, wk, cu, ks, st, pe, seqlens)
    cv, _ = linear_compress(vp, wv, cu, ks, st, None, seqlens)
    cache.load(kp, kp, vp, ck, cv, seqlens, compressed_seqlens(seqlens, ks, st))
    outs = []
    for s in range(steps):
        kn = torch.stack([x[L + s] for x, L in zip(k, seqlens)])
        vn = torch.stack([x[L + s] for x, L in zip(v, seqlens)])
        cache.append(kn, kn, vn, wk, wv, pe, None)
        outs.append(nsa_decode_attention(q[s], cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0,
                                         cache.cmp_row0, max_len=max_len, shard=shard, ops=OracleDecodeOps(), cmp_chunk=8, **CFG))
    return outs


def _expected(seqlens, steps, q, k, v, wk, wv, pe):
    ks, st = CFG["kernel_size"], CFG["kernel_stride"]
    exp = []
    for s in range(steps):
        lens = [L + s + 1 for L in seqlens]
        ks_ = [x[:L] for x, L in zip(k, lens)]
        vs_ = [x[:L] for x, L in zip(v, lens)]
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
        ck, ccu = linear_compress(torch.cat(ks_), wk, cu, ks, st, pe, lens)
        cv, _ = linear_compress(torch.cat(vs_), wv, cu, ks, st, None, lens)
        cks = [ck[int(ccu[b]) : int(ccu[b + 1])] for b in range(len(lens))]
        cvs = [cv[int(ccu[b]) : int(ccu[b + 1])] for b in range(len(lens))]
        exp.append(decode_branches_ref(q[s].float(), ks_, vs_, cks, cvs, CFG))
    return exp


def _compare(outs, exp):
    for got, ref in zip(outs, exp):
        assert got[6].tolist() == ref[6].tolist()                       # top-k ids bit-exact
        for i in range(3):
            torch.testing.assert_close(got[i].float(), ref[i], rtol=2e-2, atol=2e-2)
            fin = torch.isfinite(ref[3 + i])
            assert torch.equal(torch.isfinite(got[3 + i]), fin)
            torch.testing.assert_close(got[3 + i][fin], ref[3 + i][fin], rtol=1e-4, atol=1e-4)


def test_cache_and_step_logic_single_rank():
    seqlens, steps = [37, 5, 64], 6
    q, k, v, wk, wv, pe = _make_problem(3, seqlens, 4, 2, 16, steps)
    outs = _run_steps(None, seqlens, steps, q, k, v, wk, wv, pe, max_len=80)
    _compare(outs, _expected(seqlens, steps, q, k, v, wk, wv, pe))


def test_masked_compressor_path_matches_conditional_path():
    """The launch-invariant append (compressor always runs, masked writes: what a captured step uses) leaves the same
    cache and gives the same outputs as the append that skips the compressor when no window completes."""
    seqlens, steps = [37, 5, 64], 10
    q, k, v, wk, wv, pe = _make_problem(8, seqlens, 4, 2, 16, steps)
    a = _run_steps(None, seqlens, steps, q, k, v, wk, wv, pe, max_len=96)
    b = _run_steps(None, seqlens, steps, q, k, v, wk, wv, pe, max_len=96, always_compress=True)
    for x, y in zip(a, b):
        for i in range(7):
            assert torch.equal(x[i], y[i])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # max_len chosen so that the two ranks hold different numbers of 8-token score chunks (12 and 7 compressed tokens)
        seqlens, steps, max_len = [37, 5, 64, 18], 6, 160
        q, k, v, wk, wv, pe = _make_problem(5, seqlens, 4, 2, 16, steps)
        shard = shard_plan(max_len, CFG["kernel_size"], CFG["kernel_stride"], rank, world, group=None, align=16)
        outs = _run_steps(shard, seqlens, steps, q, k, v, wk, wv, pe, max_len)
        _compare(outs, _expected(seqlens, steps, q, k, v, wk, wv, pe))
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback

        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def test_kv_sequence_sharding_two_gloo_ranks():
    """Each rank stores half of every sequence's tokens and compressed tokens; partial outputs are merged by LSE after
    an all-gather and every rank must reproduce the unsharded result, top-k ids included."""
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert all(ret.get(r) == "ok" for r in range(world)), dict(ret)
