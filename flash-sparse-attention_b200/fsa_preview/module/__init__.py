from fsa_preview.module.fsa_decode import FlashSparseAttentionDecode  # noqa: F401
from fsa_preview.module.fsa_decode_kernel import FlashSparseAttentionDecodeKernel  # noqa: F401
from fsa_preview.module.graph import GraphedShardedAttention, GraphedStep  # noqa: F401
