"""Golden vectors for the K/V compressor from the reference's OWN Triton kernels, run on the CPU through Triton's
interpreter (``TRITON_INTERPRET=1``, fp16 inputs: the interpreter's bf16 dot product is broken in Triton 3.6).

``LinearCompress.forward`` allocates one tensor with ``device="cuda"`` (nsa_ref/ops/linear_compress.py:340), so the
autograd function cannot run without a GPU; its two kernels can.  This script launches ``linear_compress_fwd_kernel`` and
``linear_compress_bwd_kernel`` exactly as ``LinearCompress.forward`` / ``.backward`` launch them (:334-398, :401-470: same
grids, strides, block sizes, fp32 dx / dw buffers then cast), with CPU tensors, and adds the position-embedding bias with
the wrapper's own expression (:497-501).

Usage (needs the reference checkout; not needed to run the tests):
    python tests/golden/make_linear_compress_golden.py /path/to/reference
Writes tests/golden/linear_compress_case*.npz
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_linear_compress_golden.py <checkout of Relaxed-System-Lab/Flash-Sparse-Attention>")
sys.path.append(sys.argv[1])

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
from einops import einsum, rearrange  # noqa: E402

from nsa_ref.ops.linear_compress import IS_HOPPER_GPU, linear_compress_bwd_kernel, linear_compress_fwd_kernel  # noqa: E402

CASES = [
    # name, seqlens, H, d, kernel_size, stride, with_pe, seed
    ("case0", [150], 2, 64, 32, 16, True, 3000),
    ("case1", [100, 20, 75], 1, 64, 32, 16, False, 3001),     # a sequence shorter than one window
    ("case2", [90], 2, 32, 16, 16, True, 3002),               # non-overlapping windows
]

for name, seqlens, H, d, ks, st, with_pe, seed in CASES:
    g = torch.Generator().manual_seed(seed)
    N = sum(seqlens)
    x = torch.randn(N, H, d, generator=g).to(torch.float16)
    w = (torch.randn(H, ks * d, d, generator=g) * 0.05).to(torch.float16)
    pe = (torch.randn(H, ks, d, generator=g) * 0.5).to(torch.float16) if with_pe else None
    cu = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int32)
    B = len(seqlens)
    sl = cu[1:] - cu[:-1]
    y_sl = torch.floor((sl - ks) / st).to(torch.int32) + 1
    y_sl[sl < ks] = 0
    y_cu = torch.cat([torch.zeros(1, dtype=torch.int32), torch.cumsum(y_sl, 0)]).to(torch.int32)
    y = torch.zeros(int(y_cu[-1]), H, d, dtype=x.dtype)
    bks = max(16, triton.next_power_of_2(ks))
    bhd = 8 if IS_HOPPER_GPU else 4
    bhD, bos = 32, 64
    w4 = w.reshape(H, ks, d, d).contiguous()
    grid = (B * H, triton.cdiv(int(y_sl.max()), bos), triton.cdiv(d, bhD))
    linear_compress_fwd_kernel[grid](x, y, w4, cu, y_cu, x.stride(0), x.stride(1), x.stride(2), w4.stride(0), w4.stride(1), w4.stride(2),
                                     w4.stride(3), y.stride(0), y.stride(1), y.stride(2), H, ks, st, d, d, bos, bks, bhd, bhD)
    dy = torch.randn(y.shape, generator=g).to(torch.float16)
    dx = torch.zeros(N, H, d, dtype=torch.float32)
    dw = torch.zeros(H, ks, d, d, dtype=torch.float32)
    grid = (B * H, triton.cdiv(int(y_sl.max()), bos), triton.cdiv(d, bhD) * triton.cdiv(d, bhd))
    linear_compress_bwd_kernel[grid](dx, dy, dw, x, w4, cu, y_cu, x.stride(0), x.stride(1), x.stride(2), w4.stride(0), w4.stride(1),
                                     w4.stride(2), w4.stride(3), dx.stride(0), dx.stride(1), dx.stride(2), dw.stride(0), dw.stride(1),
                                     dw.stride(2), dw.stride(3), dy.stride(0), dy.stride(1), dy.stride(2), H, d // bhd, ks, st, d, d,
                                     bks, bhd, bhD, bos)
    dx16, dw16 = dx.to(x.dtype), rearrange(dw.to(x.dtype), "n k d D -> n (k d) D")
    y_out = y
    if pe is not None:
        bias = einsum(rearrange(pe, "h k d -> h (k d)"), w, "h D, h D d -> h d")
        y_out = y + bias.unsqueeze(0)
    np.savez_compressed(os.path.join(HERE, f"linear_compress_{name}.npz"), x=x.numpy(), w=w.numpy(),
                        pe=(pe.numpy() if pe is not None else np.zeros(0, np.float16)), cu=cu.numpy(), y_cu=y_cu.numpy(),
                        kernel_size=np.int32(ks), kernel_stride=np.int32(st), y_nobias=y.numpy(), y=y_out.numpy(), dy=dy.numpy(),
                        dx=dx16.numpy(), dw=dw16.numpy())
    print(name, "done", tuple(y.shape), float(y.float().abs().max()), float(dx.abs().max()), float(dw.abs().max()))
