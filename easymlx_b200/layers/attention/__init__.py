from ._performer import AttentionPerformer, PagedAttentionInputs, prepare_paged_attention_inputs

__all__ = ("AttentionPerformer", "PagedAttentionInputs", "prepare_paged_attention_inputs")
