from fsa.ops.FSA_topk_sparse_attention import FSA_topk_sparse_attention

__all__ = ["FSA_topk_sparse_attention"]
