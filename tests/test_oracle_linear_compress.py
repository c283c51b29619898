"""The compressor oracle (oracle.nsa_layer_oracle.linear_compress_ref) against vectors made by the reference's own Triton
kernels (linear_compress_fwd_kernel / linear_compress_bwd_kernel, nsa_ref/ops/linear_compress.py:28-292, launched as
LinearCompress launches them; generator: tests/golden/make_linear_compress_golden.py).

Tolerances: the reference computes in fp16 with fp32 accumulation and rounds y, dx and dW to fp16: |y| <= 8 gives an
output rounding of 4e-3, dW values of magnitude 16 one of 8e-3; the oracle is fp32 throughout."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle.nsa_layer_oracle import linear_compress_ref

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = sorted(glob.glob(os.path.join(HERE, "golden", "linear_compress_case*.npz")))


def load(path):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files}
    t["seqlens"] = (t["cu"][1:] - t["cu"][:-1]).tolist()
    t["ks"], t["st"] = int(z["kernel_size"]), int(z["kernel_stride"])
    t["pe"] = t["pe"] if t["pe"].numel() else None
    return t


def test_fixtures_present():
    assert len(CASES) == 3


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_oracle_matches_reference_kernels(path):
    t = load(path)
    x = t["x"].float().requires_grad_(True)
    w = t["w"].float().requires_grad_(True)
    y_nb, lens = linear_compress_ref(x, w, t["seqlens"], t["ks"], t["st"], None)
    assert [0] + list(np.cumsum(lens)) == t["y_cu"].tolist()
    assert float((y_nb - t["y_nobias"].float()).abs().max()) <= 6e-3
    y, _ = linear_compress_ref(t["x"].float(), t["w"].float(), t["seqlens"], t["ks"], t["st"], t["pe"].float() if t["pe"] is not None else None)
    assert float((y - t["y"].float()).abs().max()) <= 1.2e-2          # product and bias are rounded separately in the reference
    y_nb.backward(t["dy"].float())
    assert float((x.grad - t["dx"].float()).abs().max()) <= 4e-3 * max(1.0, float(t["dx"].float().abs().max()))
    assert float((w.grad - t["dw"].float()).abs().max()) <= 1e-3 * max(1.0, float(t["dw"].float().abs().max())) + 8e-3
