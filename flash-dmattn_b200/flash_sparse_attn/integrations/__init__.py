"""Caller-side glue for HuggingFace-style attention modules (reference: flash_sparse_attn/integrations/)."""
from .flash_sparse_attention import flash_sparse_attention_forward  # noqa: F401
