"""The fused gate path (gate projection + sigmoid + mix of the three branches, fsa/module/fsa.py:162-171) against the
separate torch modules it replaces, forward and backward.

Tolerance: the kernels round where the modules round (the Linear's output, the sigmoid, the mixed output; in the backward
d(gate), the sigmoid's backward, dx and dW), so results agree to rounding: outputs and da/db/dc within 2 bf16 ulps of the
value's magnitude, dx / dW within 2e-2 relative L2 (their 3-term / N-term sums are accumulated in a different order)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fsa.ops.gate import gate_mix, gate_proj_mix

DEV = "cuda:0"


@pytest.mark.parametrize("N,hidden,H,d,dtype", [(300, 256, 4, 64, torch.bfloat16), (1000, 1024, 8, 128, torch.bfloat16),
                                                (77, 512, 2, 128, torch.float16), (5000, 4096, 32, 128, torch.bfloat16)])
def test_gate_proj_mix_matches_modules(N, hidden, H, d, dtype):
    g = torch.Generator().manual_seed(N + hidden)
    x = torch.randn(N, hidden, generator=g).to(dtype).to(DEV)
    w = (torch.randn(3, hidden, generator=g) * hidden ** -0.5).to(dtype).to(DEV)
    a, b, c, dout = (torch.randn(N, H, d, generator=g).to(dtype).to(DEV) for _ in range(4))
    # reference: the modules of the layer
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ar, br, cr = (t.clone().requires_grad_(True) for t in (a, b, c))
    gate = torch.sigmoid(torch.nn.functional.linear(xr, wr))
    ref = gate[:, 0, None, None] * ar + gate[:, 1, None, None] * br + gate[:, 2, None, None] * cr
    ref.backward(dout)
    xf, wf = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    af, bf, cf = (t.clone().requires_grad_(True) for t in (a, b, c))
    out = gate_proj_mix(xf, wf, af, bf, cf)
    out.backward(dout)
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10

    def close(got, want, name, mag=None):
        err = (got.float() - want.float()).abs()
        mag = want.float().abs() if mag is None else mag
        lim = 4 * ulp * mag.clamp_min(0.05)
        assert bool((err <= lim).all()), f"{name}: max err {float(err.max()):.3e}"

    # the modules round every product and every partial sum of the mix, the kernel rounds once: a few ulps of the
    # largest term, not of the (possibly cancelling) sum
    close(out, ref, "out", a.float().abs() + b.float().abs() + c.float().abs())
    close(af.grad, ar.grad, "da"); close(bf.grad, br.grad, "db"); close(cf.grad, cr.grad, "dc")
    for got, want, name in ((xf.grad, xr.grad, "dx"), (wf.grad, wr.grad, "dw")):
        rel = float((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-6))
        assert rel <= 2e-2, f"{name}: relative L2 {rel:.3e}"
    # two runs give the same bits (no atomics)
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    out2 = gate_proj_mix(xg, wg, a, b, c)
    out2.backward(dout)
    assert torch.equal(out2, out) and torch.equal(xg.grad, xf.grad) and torch.equal(wg.grad, wf.grad)
