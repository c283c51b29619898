"""A state_dict with the reference layer's parameter names and shapes loads into this layer unchanged.

The reference declares (fsa/module/fsa.py:44-59): proj_q / proj_k / proj_v / proj_o as bias-free nn.Linear,
compress_key / compress_value [num_kv_heads, head_dim * kernel_size, head_dim], intra_block_pe [num_kv_heads, kernel_size,
head_dim], gate = Sequential(Linear(hidden, 3, bias=False), Sigmoid) -> "gate.0.weight"; its rotary module keeps inv_freq
as a non-persistent buffer (nsa_ref/module/rope.py:79), so nothing of it is in the state_dict.  The decode modules of
fsa_preview declare the same parameters (fsa_preview/module/fsa_decode.py:12-60)."""
import torch

from fsa.module.fsa import FlashSparseAttention, RopeConfig
from fsa_preview.module import FlashSparseAttentionDecode, FlashSparseAttentionDecodeKernel

CFG = dict(hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=64, kernel_size=32, kernel_stride=16, block_size=64, topk=16,
           init_blocks=1, local_blocks=2, window_size=512)


def reference_shaped_state_dict(c, seed=0):
    g = torch.Generator().manual_seed(seed)
    hq, hk, d, ks, hid = c["num_q_heads"], c["num_kv_heads"], c["head_dim"], c["kernel_size"], c["hidden_size"]
    r = lambda *shape: torch.randn(*shape, generator=g)
    return {
        "proj_q.weight": r(hq * d, hid), "proj_k.weight": r(hk * d, hid), "proj_v.weight": r(hk * d, hid), "proj_o.weight": r(hid, hq * d),
        "compress_key": r(hk, d * ks, d), "compress_value": r(hk, d * ks, d), "intra_block_pe": r(hk, ks, d), "gate.0.weight": r(3, hid),
    }


def test_reference_state_dict_loads_strictly():
    sd = reference_shaped_state_dict(CFG)
    layer = FlashSparseAttention(**CFG, rope_config=RopeConfig(head_dim=CFG["head_dim"]))
    assert sorted(layer.state_dict().keys()) == sorted(sd.keys())
    missing, unexpected = layer.load_state_dict(sd, strict=True)
    assert not missing and not unexpected
    for k, v in sd.items():
        assert torch.equal(layer.state_dict()[k], v), k


def test_decode_modules_take_the_same_state_dict():
    sd = reference_shaped_state_dict(CFG, seed=1)
    args = (CFG["hidden_size"], CFG["num_q_heads"], CFG["num_kv_heads"], CFG["head_dim"])
    kw = {k: CFG[k] for k in ("kernel_size", "kernel_stride", "block_size", "topk", "init_blocks", "local_blocks", "window_size")}
    for cls in (FlashSparseAttentionDecode, FlashSparseAttentionDecodeKernel):
        try:
            mod = cls(*args, **kw, rope_config=RopeConfig(head_dim=CFG["head_dim"]))
        except TypeError:
            mod = cls(*args, **kw)
        own = mod.state_dict()
        shared = {k: v for k, v in sd.items() if k in own}
        assert shared, cls.__name__
        for k, v in shared.items():
            assert own[k].shape == v.shape, (cls.__name__, k)
        mod.load_state_dict(shared, strict=False)
        # every parameter of the module has a reference name (nothing is renamed)
        assert set(own.keys()) <= set(sd.keys()), (cls.__name__, sorted(set(own.keys()) - set(sd.keys())))
