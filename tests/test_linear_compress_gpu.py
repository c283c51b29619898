"""The K/V compressor on the GPU (fsa_linear_compress_fwd / fsa_linear_compress_bwd through the operator) against the CPU oracle
(oracle.nsa_layer_oracle.linear_compress_ref, which restates nsa_ref/ops/linear_compress.py:113-131, :334-346, :495-502).

Tolerance: the kernel accumulates in fp32 and rounds once to the activation dtype (twice with the bias, as the reference
does); against the fp32 oracle max-abs <= 2e-2 * max(1, |ref|max / 2), mean-abs <= 1e-3 * the same scale."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fsa.ops.linear_compress import linear_compress, linear_compress_gemm
from fsa.synthetic import make_cu_seqlens
from oracle.nsa_layer_oracle import linear_compress_ref

DEV = "cuda:0"


def _tol_ok(got, ref, name):
    err = (got.float().cpu() - ref).abs()
    scale = max(1.0, float(ref.abs().max()) / 2.0)
    assert float(err.max()) <= 2e-2 * scale, f"{name}: max-abs {float(err.max()):.3e} (ref max {float(ref.abs().max()):.2f})"
    assert float(err.mean()) <= 1e-3 * scale, f"{name}: mean-abs {float(err.mean()):.3e}"


@pytest.mark.parametrize("seqlens,H,d,ks,st,dtype,with_pe", [
    ([300, 20, 1000], 2, 128, 32, 16, torch.bfloat16, True),       # a sequence shorter than one window
    ([2100], 3, 128, 32, 16, torch.bfloat16, False),               # more than one tile of 128 windows
    ([257, 513], 2, 64, 32, 16, torch.float16, True),
    ([31], 1, 128, 32, 16, torch.bfloat16, True),                  # no window at all
    ([700], 2, 128, 64, 32, torch.bfloat16, True),
    ([1500, 40, 333], 2, 128, 16, 16, torch.bfloat16, False),      # non-overlapping windows: every token in one window
    ([900, 2300], 1, 64, 64, 16, torch.bfloat16, True),            # every token in four windows
    ([5000, 4200], 2, 128, 32, 16, torch.float16, False),          # many 128-window tiles in the dW reduction
])
def test_forward_backward_matches_oracle(seqlens, H, d, ks, st, dtype, with_pe):
    N = sum(seqlens)
    g = torch.Generator().manual_seed(7 + N)
    # x as the layer produces it: a strided view of a fused projection output
    fused = torch.randn(N, 2 * H * d, generator=g).to(dtype)
    w = (torch.randn(H, ks * d, d, generator=g) * 0.02).to(dtype)
    pe = (torch.randn(H, ks, d, generator=g) * 0.5).to(dtype) if with_pe else None
    x = fused[:, H * d :].view(N, H, d)
    cu = make_cu_seqlens(seqlens)
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    pf = pe.float().requires_grad_(True) if with_pe else None
    y_ref, lens = linear_compress_ref(xf, wf, seqlens, ks, st, pf)
    fc = fused.to(DEV).requires_grad_(True)
    wc = w.to(DEV).requires_grad_(True)
    pc = pe.to(DEV).requires_grad_(True) if with_pe else None
    y, y_cu = linear_compress(fc[:, H * d :].view(N, H, d), wc, cu.to(DEV), ks, st, pc, seqlens)
    assert y_cu.tolist() == [0] + list(torch.tensor(lens).cumsum(0).tolist())
    assert y.shape == y_ref.shape
    if y.numel() == 0:
        return
    _tol_ok(y, y_ref.detach(), "y")
    # the library-GEMM formulation agrees too (same inputs, same rounding points)
    y2, _ = linear_compress_gemm(x.to(DEV), w.to(DEV), cu.to(DEV), ks, st, pe.to(DEV) if with_pe else None, seqlens)
    assert float((y.float() - y2.float()).abs().max()) <= 2e-2 * max(1.0, float(y_ref.abs().max()) / 2)
    dy = torch.randn(y.shape, generator=g).to(dtype)
    y.backward(dy.to(DEV))
    y_ref.backward(dy.float())
    _tol_ok(fc.grad[:, H * d :].reshape(N, H, d), xf.grad, "dx")
    assert float(fc.grad[:, : H * d].abs().max()) == 0
    gw = wc.grad.float().cpu()
    assert float((gw - wf.grad).norm()) <= 2e-2 * float(wf.grad.norm()), "dw"
    if with_pe:
        assert float((pc.grad.float().cpu() - pf.grad).norm()) <= 3e-2 * float(pf.grad.norm()), "dpe"


def test_backward_is_bit_reproducible():
    """No atomics: two backward passes on the same inputs give the same bits (the reference's do not, :275, :292)."""
    seqlens, H, d, ks, st = [3000, 777], 2, 128, 32, 16
    N = sum(seqlens)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(N, H, d, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(H, ks * d, d, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    cu = make_cu_seqlens(seqlens).to(DEV)
    grads = []
    for _ in range(2):
        xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y, _ = linear_compress(xr, wr, cu, ks, st, None, seqlens)
        gy = torch.Generator().manual_seed(6)
        y.backward(torch.randn(y.shape, generator=gy).to(torch.bfloat16).to(DEV))
        grads.append((xr.grad.clone(), wr.grad.clone()))
    assert torch.equal(grads[0][0], grads[1][0]) and torch.equal(grads[0][1], grads[1][1])


def test_kernels_match_reference_generated_vectors():
    """Forward (with the PE bias), dx and dW against the vectors the reference's own Triton kernels produced
    (tests/golden/linear_compress_case*.npz; head_dim 64 cases run on the kernels of this library)."""
    import glob
    import os

    import numpy as np

    paths = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "linear_compress_case*.npz")))
    assert len(paths) == 3
    ran = 0
    for path in paths:
        z = np.load(path)
        x, w, dy = (torch.from_numpy(z[k]) for k in ("x", "w", "dy"))
        if x.shape[-1] not in (64, 128):
            continue
        ran += 1
        pe = torch.from_numpy(z["pe"]) if z["pe"].size else None
        cu = torch.from_numpy(z["cu"])
        seqlens = (cu[1:] - cu[:-1]).tolist()
        ks, st = int(z["kernel_size"]), int(z["kernel_stride"])
        xc, wc = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
        with torch.no_grad():
            yb, y_cu = linear_compress(xc, wc, cu.to(DEV), ks, st, pe.to(DEV) if pe is not None else None, seqlens)
        assert y_cu.tolist() == z["y_cu"].tolist()
        assert float((yb.float().cpu() - torch.from_numpy(z["y"]).float()).abs().max()) <= 1.6e-2
        # the vectors' dx / dW are those of the two kernels (no bias path)
        y, _ = linear_compress(xc, wc, cu.to(DEV), ks, st, None, seqlens)
        assert float((y.float().cpu() - torch.from_numpy(z["y_nobias"]).float()).abs().max()) <= 8e-3
        y.backward(dy.to(DEV))
        dx_ref, dw_ref = torch.from_numpy(z["dx"]).float(), torch.from_numpy(z["dw"]).float()
        assert float((xc.grad.float().cpu() - dx_ref).abs().max()) <= 8e-3 * max(1.0, float(dx_ref.abs().max()))
        assert float((wc.grad.float().cpu() - dw_ref).norm()) <= 2e-3 * float(dw_ref.norm())
    assert ran == 2
