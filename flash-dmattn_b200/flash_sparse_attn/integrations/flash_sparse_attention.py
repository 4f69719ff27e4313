"""`flash_sparse_attention_forward`: the attention-interface function a HuggingFace model registers for
`attn_implementation="flash_sparse_attn"` (reference: flash_sparse_attn/integrations/flash_sparse_attention.py:12-111).
Takes (B, H, S, d) tensors from the module, returns ((B, S, H, d), None)."""
from typing import Optional

import torch

from .modeling_flash_sparse_attention_utils import _flash_sparse_attention_forward


def _half_dtype_of(module: torch.nn.Module) -> Optional[torch.dtype]:
    """The dtype fp32 activations are cast back to: autocast's, else the pre-quantisation dtype, else the dtype of
    the module's first Linear weight (reference :79-88)."""
    if torch.is_autocast_enabled():
        return torch.get_autocast_gpu_dtype()
    config = getattr(module, "config", None)
    if config is not None and hasattr(config, "_pre_quantization_dtype"):
        return config._pre_quantization_dtype
    for layer in module.modules():
        if isinstance(layer, torch.nn.Linear):
            return layer.weight.dtype
    return None


def flash_sparse_attention_forward(
    module: torch.nn.Module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    attention_bias: Optional[torch.Tensor],
    scaling: Optional[float] = None,
    window_size: Optional[int] = None,
    softcap: Optional[float] = None,
    **kwargs,
):
    query_len, key_len = query.shape[2], key.shape[2]
    if any(dim == 0 for dim in query.shape):
        raise ValueError("FlashSparseAttention does not support inputs with a zero dimension; check the input "
                         "shapes or use SDPA instead.")
    query, key, value = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    target_dtype = _half_dtype_of(module) if query.dtype == torch.float32 else None
    is_causal = kwargs.pop("is_causal", None)
    if is_causal is None:
        is_causal = module.is_causal
    for dropped in ("output_attentions", "head_mask"):  # not supported by the fused path, as in the reference
        kwargs.pop(dropped, None)
    out = _flash_sparse_attention_forward(
        query, key, value, attention_mask, attention_bias,
        query_length=query_len, key_length=key_len, is_causal=is_causal, softmax_scale=scaling, softcap=softcap,
        window_size=window_size, target_dtype=target_dtype, implementation="flash_sparse_attn",
        layer_idx=getattr(module, "layer_idx", None), **kwargs)
    return out, None
