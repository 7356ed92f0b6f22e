"""blockrank_b200: B200-native BlockRank prefill attention and ranking-score extraction.

    from blockrank_b200 import register_cuda_blockrank_attention
    register_cuda_blockrank_attention()          # -> "cuda_blockrank"
    model.set_attn_implementation("cuda_blockrank")

All compute runs in libblockrank_b200.so (hand-written sm_100a kernels behind a
C ABI, include/blockrank_b200.h).  Importing this package does not load the
library; the first call that needs it does, and fails loudly if it is missing.
"""
from .attention import (ATTN_NAME, BlockSpans, cuda_blockrank_attention_forward, cuda_blockrank_attention_mask,
                        register_cuda_blockrank_attention)
from .collate import block_icr_collate_fn, packed_block_collate_fn
from .scores import doc_logits_from_mass, notebook_scores, signal_rows_from_labels, topk_documents

__all__ = ["ATTN_NAME", "BlockSpans", "cuda_blockrank_attention_forward", "cuda_blockrank_attention_mask",
           "register_cuda_blockrank_attention", "block_icr_collate_fn", "packed_block_collate_fn",
           "doc_logits_from_mass", "notebook_scores", "signal_rows_from_labels", "topk_documents"]
