"""Golden vector for the llama3 rotary frequencies: the output of the function the reference calls,
``transformers.modeling_rope_utils.ROPE_INIT_FUNCTIONS["llama3"]`` (call site nsa_ref/module/rope.py:76-78),
for the reference's default RopeConfig (rope.py:43-59).  Needs transformers; not needed to run the tests.

    python tests/golden/make_rope_golden.py
"""
import os

import numpy as np
from transformers import LlamaConfig
from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

cfg = LlamaConfig(hidden_size=4096, num_attention_heads=32, head_dim=128, max_position_embeddings=131072, rope_theta=500000.0,
                  rope_scaling={"factor": 8.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                                "original_max_position_embeddings": 8192, "rope_type": "llama3"})
inv, scaling = ROPE_INIT_FUNCTIONS["llama3"](cfg, "cpu")
assert scaling == 1.0
np.save(os.path.join(os.path.dirname(os.path.abspath(__file__)), "rope_llama3_inv_freq.npy"), inv.numpy())
print(inv[:4], inv[-4:])
