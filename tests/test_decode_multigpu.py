"""KV-sequence sharded decode on two GPUs (NCCL): every rank must reproduce the unsharded result.  Skipped on a
one-GPU box; the CPU twin of this test (gloo, CPU restatement of the device operators) is in test_decode_cpu.py."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

CFG = dict(kernel_size=32, kernel_stride=16, block_size=64, topk=4, init_blocks=1, local_blocks=2, window_size=100)


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from fsa.ops.linear_compress import compressed_seqlens, linear_compress
        from fsa_preview.cache import DecodeCache
        from fsa_preview.ops.decode import nsa_decode_attention, shard_plan
        from oracle.decode_oracle import decode_branches_ref

        g = torch.Generator().manual_seed(9)
        Hk, G, D, steps, max_len = 2, 4, 128, 5, 1280
        Hq = Hk * G
        seqlens = [700, 45, 1200, 130]
        B = len(seqlens)
        ks, st = CFG["kernel_size"], CFG["kernel_stride"]
        k = [torch.randn(L + steps, Hk, D, generator=g).to(torch.bfloat16) for L in seqlens]
        v = [torch.randn(L + steps, Hk, D, generator=g).to(torch.bfloat16) for L in seqlens]
        q = torch.randn(steps, B, Hq, D, generator=g).to(torch.bfloat16)
        wk = (torch.randn(Hk, ks * D, D, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        wv = (torch.randn(Hk, ks * D, D, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        shard = shard_plan(max_len, ks, st, rank, world, align=64)
        cache = DecodeCache(B, max_len, Hk, D, ks, st, torch.bfloat16, dev, shard)
        kp = torch.cat([x[:L] for x, L in zip(k, seqlens)]).to(dev)
        vp = torch.cat([x[:L] for x, L in zip(v, seqlens)]).to(dev)
        cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32, device=dev)
        ck, _ = linear_compress(kp, wk, cu, ks, st, None, seqlens)
        cv, _ = linear_compress(vp, wv, cu, ks, st, None, seqlens)
        cache.load(kp, kp, vp, ck, cv, seqlens, compressed_seqlens(seqlens, ks, st))
        for s in range(steps):
            kn = torch.stack([x[L + s] for x, L in zip(k, seqlens)]).to(dev)
            vn = torch.stack([x[L + s] for x, L in zip(v, seqlens)]).to(dev)
            cache.append(kn, kn, vn, wk, wv, None, None)
            got = nsa_decode_attention(q[s].to(dev), cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0,
                                       cache.cmp_row0, max_len=max_len, shard=shard, **CFG)
            lens = [L + s + 1 for L in seqlens]
            ks_ = [x[:L] for x, L in zip(k, lens)]
            vs_ = [x[:L] for x, L in zip(v, lens)]
            cuL = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
            ckf, ccu = linear_compress(torch.cat(ks_).to(dev), wk, cuL, ks, st, None, lens)
            cvf, _ = linear_compress(torch.cat(vs_).to(dev), wv, cuL, ks, st, None, lens)
            ccu = ccu.tolist()
            cks = [ckf[ccu[b] : ccu[b + 1]].cpu() for b in range(B)]
            cvs = [cvf[ccu[b] : ccu[b + 1]].cpu() for b in range(B)]
            ref = decode_branches_ref(q[s].float(), ks_, vs_, cks, cvs, CFG, topk_idx=got[6].cpu())
            assert (got[6].cpu() == ref[6]).float().mean() >= 0.97
            for i in range(3):
                err = (got[i].float().cpu() - ref[i]).abs()
                scale = max(1.0, float(ref[i].abs().max()) / 2)           # bf16 outputs: the tolerance follows the magnitude
                assert float(err.max()) <= 2e-2 * scale and float(err.mean()) <= 1e-3 * scale, (s, i, float(err.max()), float(err.mean()))
                fin = torch.isfinite(ref[3 + i])
                torch.testing.assert_close(got[3 + i].cpu()[fin], ref[3 + i][fin], rtol=1e-4, atol=1e-4)
        # the step as three CUDA graphs around its two all-gathers gives the same outputs as the launch-by-launch step
        from fsa_preview.module import GraphedShardedAttention
        from fsa_preview.ops.decode import DecodeStepPlan

        qd = q[steps - 1].to(dev)
        plan = DecodeStepPlan(max_len=max_len, shard=shard, **CFG)
        graphed = GraphedShardedAttention(plan, qd, cache, lambda oc, os_, ow: torch.stack([oc, os_, ow]))
        for _ in range(2):
            out = graphed()
        torch.cuda.synchronize()
        for i in range(3):
            assert torch.equal(out[i], got[i]), f"graphed sharded step: branch {i} differs"
        ret[rank] = "ok"
    except Exception:  # noqa: BLE001
        import traceback

        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_decode_two_gpus():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    assert all(ret.get(r) == "ok" for r in range(world)), dict(ret)
