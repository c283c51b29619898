"""Host-side NSA pieces that need no GPU: rotary frequencies against the transformers golden vector,
linear_compress_gemm (the library-GEMM formulation of the compressor) against the loop oracle, the top-k oracle's tie rule."""
import os

import numpy as np
import torch

from fsa.module.rope import RopeConfig, compute_inv_freq
from fsa.ops.linear_compress import compressed_seqlens
from fsa.ops.linear_compress import linear_compress_gemm as linear_compress   # CPU tensors: the library-GEMM formulation (the backward of the kernel path)
from oracle.nsa_layer_oracle import linear_compress_ref, topk_from_block_scores

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_llama3_inv_freq_matches_transformers_golden():
    gold = torch.from_numpy(np.load(os.path.join(GOLDEN, "rope_llama3_inv_freq.npy")))
    assert torch.equal(compute_inv_freq(RopeConfig()), gold)
    # "default" type: plain theta^(-2i/d)
    plain = compute_inv_freq(RopeConfig(rope_scaling=None, head_dim=64, rope_theta=10000.0))
    assert torch.allclose(plain, 1.0 / (10000.0 ** (torch.arange(0, 64, 2).float() / 64)))


def test_linear_compress_matches_loop_oracle_and_grads():
    torch.manual_seed(0)
    seqlens, H, d, ks, st = [70, 10, 33], 2, 16, 16, 8
    N = sum(seqlens)
    x = torch.randn(N, H, d).to(torch.bfloat16)
    w = (torch.randn(H, ks * d, d) * 0.1).to(torch.bfloat16)
    pe = torch.randn(H, ks, d).to(torch.bfloat16)
    cu = torch.tensor([0, 70, 80, 113], dtype=torch.int32)
    assert compressed_seqlens(seqlens, ks, st) == [7, 0, 3]
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y, ycu = linear_compress(xr, wr, cu, ks, st, pe, seqlens=seqlens)
    y_ref, lens = linear_compress_ref(x, w, seqlens, ks, st, pe)
    assert ycu.tolist() == [0, 7, 7, 10] and lens == [7, 0, 3]
    assert (y.float() - y_ref).abs().max() < 0.15            # bf16 output of a 256-term product
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    yf, _ = linear_compress_ref_autograd(xf, wf, seqlens, ks, st)
    yf = yf + torch.einsum("hD,hDd->hd", pe.float().reshape(H, -1), wf).unsqueeze(0)
    yf.backward(dy.float())
    assert (xr.grad.float() - xf.grad).abs().max() < 0.05 * float(xf.grad.abs().max()) + 0.05
    assert (wr.grad.float() - wf.grad).abs().max() < 0.05 * float(wf.grad.abs().max()) + 0.05


def linear_compress_ref_autograd(x, w, seqlens, ks, st):
    H, d = x.shape[1], x.shape[2]
    outs, start = [], 0
    for L in seqlens:
        n = (L - ks) // st + 1 if L >= ks else 0
        for c in range(n):
            win = x[start + c * st : start + c * st + ks]
            outs.append(torch.einsum("khd,hkde->he", win, w.view(H, ks, d, d)))
        start += L
    return torch.stack(outs, 0), None


def test_topk_tie_rule():
    bs = torch.tensor([float("inf"), 0.5, 0.5, 0.25, float("inf")])
    assert topk_from_block_scores(bs, 3) == [0, 1, 4]
    assert topk_from_block_scores(bs, 4) == [0, 1, 2, 4]
    assert topk_from_block_scores(torch.tensor([float("inf")]), 3) == [0, -1, -1]
