from fsa_preview.ops.compat import (_compressed_attention_decode, _linear_compress_decode,  # noqa: F401
                                    _topk_sparse_attention_decode)
from fsa_preview.ops.decode import CudaDecodeOps, Shard, nsa_decode_attention, shard_plan  # noqa: F401

__all__ = [
    "_compressed_attention_decode",
    "_linear_compress_decode",
    "_topk_sparse_attention_decode",
    "nsa_decode_attention",
    "CudaDecodeOps",
    "Shard",
    "shard_plan",
]
