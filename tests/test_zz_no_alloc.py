"""fsa_sel_fwd_static: the forward for callers that cannot allocate device memory.

Some host programs hand all GPU memory to their own arena when they start, or must not risk
the synchronisation and the late failure an allocation can cause while they serve requests;
they have no workspace to pass.  This entry point keeps its scratch in a fixed array inside the
library instead.  The test calls it through the C ABI, twice in a row on different problems
(the array keeps the first call's contents), and checks each result against the ordinary
entry point, which works in caller-owned workspaces.  It also checks the size limit.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
from ctypes import byref, c_int

import pytest
import torch

pytestmark = pytest.mark.gpu

from fsa import _lib
from fsa.ops.FSA_topk_sparse_attention import sel_attn_fwd
from fsa.synthetic import make_cu_seqlens, make_qkv, make_topk_idx

DEV = "cuda:0"


def _static_fwd(q, k, v, idx, bs, cu, scale, o=None, lse=None):
    L = _lib.lib()
    N, Hq, D = q.shape
    Hk, T, B = k.shape[1], idx.shape[-1], cu.numel() - 1
    o = torch.empty_like(q) if o is None else o
    lse = torch.empty(Hq, N, dtype=torch.float32, device=q.device) if lse is None else lse
    rc = L.fsa_sel_fwd_static(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(idx), _lib.ptr(cu), N, B, Hq, Hk, D, T, bs,
        _lib.DTYPE_CODE[q.dtype], q.stride(0), q.stride(1), k.stride(0), v.stride(0), float(scale),
        _lib.ptr(o), o.stride(0), o.stride(1), _lib.ptr(lse), _lib.current_stream(q.device))
    return rc, o, lse


def _problem(seqlens, Hk, G, d, bs, T, seed):
    N = sum(seqlens)
    q, k, v = make_qkv(N, Hk * G, Hk, d, seed, with_do=False)
    idx = make_topk_idx(seqlens, Hk, T, bs, seed)
    cu = make_cu_seqlens(seqlens)
    return [x.to(DEV) for x in (q, k, v, idx, cu)]


def _static_status():
    st = c_int(-1)
    rc = _lib.lib().fsa_read_status(None, _lib.current_stream(torch.device(DEV)), byref(st))
    return rc, st.value


def test_static_forward_matches_workspace_forward_twice():
    with torch.cuda.device(DEV):
        # differently shaped problems back to back in the one shared array: a large one, a small one with another
        # head layout (its words land where the first left tile records, entries and positions), then the large one
        # again -- every call must be independent of what the previous one left behind
        shapes = (([1500, 548], 2, 2, 128, 64, 8, 21), ([300, 212], 1, 4, 128, 64, 16, 22), ([1500, 548], 2, 2, 128, 64, 8, 21))
        for i, (seqlens, Hk, G, d, bs, T, seed) in enumerate(shapes):
            q, k, v, idx, cu = _problem(seqlens, Hk, G, d, bs, T, seed)
            scale = d ** -0.5
            o_ref, lse_ref, _ = sel_attn_fwd(q, k, v, idx, bs, cu, scale, check_status=True)
            o = torch.empty_like(q)
            lse = torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc, o, lse = _static_fwd(q, k, v, idx, bs, cu, scale, o, lse)
            assert rc == 0, _lib.lib().fsa_error_string(rc)
            rc, st = _static_status()          # synchronises the stream
            assert rc == 0 and st == 0, f"device status {st}"
            if i > 0:
                # outputs were allocated before the reading and the first call has loaded every kernel: a call that
                # allocates nothing leaves the device's free memory where it was
                assert torch.cuda.mem_get_info()[0] == free_before
            assert float((o.float() - o_ref.float()).abs().max()) <= 2e-2
            assert float((lse - lse_ref).abs().max()) <= 1e-4


def test_static_forward_refuses_problems_beyond_its_array():
    with torch.cuda.device(DEV):
        q, k, v, idx, cu = _problem([16384], 4, 2, 128, 64, 16, 23)
        rc, _, _ = _static_fwd(q, k, v, idx, 64, cu, 128 ** -0.5)
        assert rc == _lib.FSA_ERR_STATIC_LIMIT
        assert b"static" in _lib.lib().fsa_error_string(rc)
