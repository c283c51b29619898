"""RoPE, gate mix, top-k block selection and the whole FlashSparseAttention layer on the GPU against the CPU oracle."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from fsa import _lib
from fsa.module.fsa import FlashSparseAttention, RopeConfig
from fsa.module.rope import RotaryEmbedding, compute_inv_freq
from fsa.ops.compressed_attention import select_topk_blocks
from fsa.ops.gate import gate_mix
from fsa.synthetic import make_cu_seqlens
from oracle import nsa_layer_oracle as orc

DEV = "cuda:0"


def test_rope_forward_backward():
    seqlens, H, d = [100, 37, 260], 3, 128
    N = sum(seqlens)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(N, H, d, generator=g).to(torch.bfloat16)
    cfg = RopeConfig(head_dim=d)
    rope = RotaryEmbedding(cfg).to(DEV)
    cu = make_cu_seqlens(seqlens).to(DEV)
    for start, stride in ((0, 1), (0, 16)):
        xc = x.to(DEV).requires_grad_(True)
        y = rope(xc, cu, start=start, stride=stride)
        ref = orc.rope_ref(x, compute_inv_freq(cfg), seqlens, start, stride)
        assert float((y.float().cpu() - ref).abs().max()) <= 2e-2
        # the rotation is orthogonal: backward of y.sum-like cotangent equals the inverse rotation
        dy = torch.randn(N, H, d, generator=g).to(torch.bfloat16)
        y.backward(dy.to(DEV))
        xf = x.float().requires_grad_(True)
        orc_y = orc.rope_ref(xf, compute_inv_freq(cfg), seqlens, start, stride)
        orc_y.backward(dy.float())
        assert float((xc.grad.float().cpu() - xf.grad).abs().max()) <= 3e-2


def test_gate_mix_forward_backward():
    N, H, d = 333, 4, 128
    g = torch.Generator().manual_seed(2)
    a, b, c = (torch.randn(N, H, d, generator=g).to(torch.bfloat16) for _ in range(3))
    gate = torch.rand(N, 3, generator=g).to(torch.bfloat16)
    dout = torch.randn(N, H, d, generator=g).to(torch.bfloat16)
    ts = [t.to(DEV).requires_grad_(True) for t in (gate, a, b, c)]
    out = gate_mix(*ts)
    out.backward(dout.to(DEV))
    fs = [t.float().requires_grad_(True) for t in (gate, a, b, c)]
    ref = fs[0][:, 0:1, None] * fs[1] + fs[0][:, 1:2, None] * fs[2] + fs[0][:, 2:3, None] * fs[3]
    ref.backward(dout.float())
    assert float((out.float().cpu() - ref).abs().max()) <= 3e-2
    for t, f, tol in zip(ts, fs, (0.5, 2e-2, 2e-2, 2e-2)):
        assert float((t.grad.float().cpu() - f.grad).abs().max()) <= tol * max(1.0, float(f.grad.abs().max()) / 16)


def test_topk_selection_bit_exact_on_exact_scores():
    """Scores that are exact powers of two in every implementation: the ids must be identical to the oracle's."""
    L, Hk, G, d = 700, 2, 2, 64
    ks, st, bs, T = 32, 16, 64, 6
    ncmp = (L - ks) // st + 1
    g = torch.Generator().manual_seed(3)
    # raw products such that qk * scale * log2e is a small negative integer: build the fp32 product tensor directly
    scale = 1.0 / (1.4426950408889634)          # scale * log2e == 1 up to rounding; use integers below
    qk = -torch.randint(0, 12, (Hk, L, ncmp), generator=g).float()
    lse = torch.zeros(Hk * G, L)
    max_blocks = math.ceil(L / bs)
    out = torch.empty((Hk, L, min(T, max_blocks)), dtype=torch.int32, device=DEV)
    ld = (ncmp + 3) // 4 * 4
    qk_pad = torch.zeros(Hk, L, ld)
    qk_pad[:, :, :ncmp] = qk
    qk_dev, lse_dev = qk_pad.to(DEV), lse.to(DEV)
    rc = _lib.lib().fsa_select_topk_seq(_lib.ptr(qk_dev), ld, _lib.ptr(lse_dev), L, 0, L, ncmp, Hk, G, scale, ks, st, bs, 1, 2,
                                        max_blocks, out.shape[-1], _lib.ptr(out), None)
    assert rc == 0
    torch.cuda.synchronize()
    for h in range(Hk):
        ref = orc.select_topk_ref(qk[h], lse[h * G], L, ncmp, scale, ks, st, bs, 1, 2, max_blocks, T)
        assert torch.equal(out[h].cpu(), ref)


CFG = dict(hidden_size=256, num_q_heads=4, num_kv_heads=2, head_dim=128, kernel_size=32, kernel_stride=16, block_size=64,
           topk=6, init_blocks=1, local_blocks=2, window_size=128)


def test_layer_forward_backward_against_oracle():
    torch.manual_seed(5)
    seqlens = [600, 50, 330]
    N = sum(seqlens)
    rope_cfg = RopeConfig(head_dim=CFG["head_dim"])
    layer = FlashSparseAttention(**CFG, rope_config=rope_cfg)
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.05)
    layer = layer.to(DEV).to(torch.bfloat16)
    x = torch.randn(N, CFG["hidden_size"]).to(torch.bfloat16)
    cu = make_cu_seqlens(seqlens)
    xc = x.to(DEV).requires_grad_(True)
    y = layer(xc, cu.to(DEV), seqlens=seqlens)
    params = {k: v.detach().float().cpu() for k, v in layer.named_parameters()}
    # (1) the oracle's own top-k ids agree with the layer's on almost every (head, token): they are chosen from
    #     bf16-rounded scores, so a last-bit difference in a probability can swap two near-tied blocks
    y_ref, idx_ref, _ = orc.layer_forward_ref(params, x, seqlens, CFG, compute_inv_freq(rope_cfg))
    idx_gpu = layer.last_topk_idx.cpu()
    agree = (idx_gpu == idx_ref).all(-1).float().mean()
    assert float(agree) >= 0.97, f"top-k rows identical: {float(agree):.4f}"
    # (2) with the layer's ids fed to the oracle the outputs must match to bf16 accuracy
    y_ref2, _, _ = orc.layer_forward_ref(params, x, seqlens, CFG, compute_inv_freq(rope_cfg), topk_idx=idx_gpu)
    err = (y.detach().float().cpu() - y_ref2).abs()
    ref_scale = float(y_ref2.abs().mean())
    assert float(err.mean()) <= 2e-2 * ref_scale, f"mean err {float(err.mean()):.3e} vs mean |y| {ref_scale:.3e}"
    assert float(err.max()) <= 1e-1 * float(y_ref2.abs().max())
    # gradients flow to every parameter and to x, finite
    y.backward(torch.randn_like(y))
    assert torch.isfinite(xc.grad.float()).all()
    for n, p in layer.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad.float()).all(), n
        assert float(p.grad.float().abs().max()) > 0, n
