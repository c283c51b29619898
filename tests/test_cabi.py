"""The C-ABI library: loads, exports every symbol include/fsa_sm100.h declares, and its
host-only entry points (size queries, argument checks) behave.  No GPU needed."""
import os
import re
from ctypes import byref, c_int64

import pytest
import torch  # noqa: F401  (loads the CUDA runtime the library links against)

from fsa import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fsa_sm100.h")


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(fsa_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(L, n), f"{n} declared in fsa_sm100.h but not exported"
    # and the Python binding table covers the same set
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_strings():
    L = _lib.lib()
    assert L.fsa_version() >= 100
    assert L.fsa_error_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert len(L.fsa_error_string(code)) > 3


def test_workspace_queries():
    L = _lib.lib()
    n = c_int64(0)
    # config 1 of the benchmark: 64K tokens, 4 sequences, 8 q heads, 4 kv heads, T=16, BK=64
    assert L.fsa_sel_index_bytes(65536, 4, 8, 4, 16, 64, byref(n)) == 0
    entries = 4 * 65536 * 16 * 4   # one int per (kv head, token, slot): entry list and position map
    # plus room for one ragged tile per (kv head, window, block) key that may exist: O(N * Hk * T) ints all the same
    assert 2 * entries <= n.value < 5 * entries
    assert L.fsa_sel_fwd_scratch_bytes(65536, 4, 8, 4, 128, 16, 64, byref(n)) == 0
    assert n.value >= 65536 * 8 * 16 * 64 * 2  # at least bf16 partials
    assert L.fsa_sel_bwd_scratch_bytes(65536, 4, 8, 4, 128, 16, 64, byref(n)) == 0
    assert n.value > 0


def test_argument_checks_return_codes():
    L = _lib.lib()
    n = c_int64(0)
    assert L.fsa_sel_index_bytes(1024, 1, 3, 2, 16, 64, byref(n)) == _lib.FSA_ERR_BAD_ARG  # Hq % Hk != 0
    assert L.fsa_sel_index_bytes(1024, 1, 4, 2, 16, 48, byref(n)) == _lib.FSA_ERR_UNSUPPORTED  # block size
    assert L.fsa_sel_index_bytes(1024, 1, 4, 2, 65, 64, byref(n)) == _lib.FSA_ERR_UNSUPPORTED  # top-k > 64
    assert L.fsa_sel_index_bytes(-1, 1, 4, 2, 16, 64, byref(n)) == _lib.FSA_ERR_BAD_ARG
    with pytest.raises(ValueError):
        _lib.check(_lib.FSA_ERR_UNSUPPORTED, "x")
    with pytest.raises(_lib.FsaError):
        _lib.check(_lib.FSA_ERR_WORKSPACE, "x")


def test_operator_refuses_cpu_tensors():
    from fsa.ops import FSA_topk_sparse_attention

    q = torch.zeros(64, 2, 128, dtype=torch.bfloat16)
    k = torch.zeros(64, 1, 128, dtype=torch.bfloat16)
    idx = torch.zeros(1, 64, 2, dtype=torch.int32)
    cu = torch.tensor([0, 64], dtype=torch.int32)
    with pytest.raises(AssertionError):
        FSA_topk_sparse_attention(q, k, k, idx, 64, cu)
