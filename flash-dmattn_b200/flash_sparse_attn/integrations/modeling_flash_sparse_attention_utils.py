"""The reference's HuggingFace glue
(flash_sparse_attn/integrations/modeling_flash_sparse_attention_utils.py:425-596): recast fp32 activations to the
model's half-precision dtype (:321-339), build the top-`window_size` mask from the bias only when the key length
exceeds the window (:570-583), and call `flash_sparse_attn_func`.

A 2-D padding mask (batch, seq_len) is handled without un-padding: the reference gathers the valid tokens, runs its
variable-length kernel with no bias and no dynamic mask, and pads the result with zeros (:511-536, `_upad_input`
:144-220). The same numbers come out of the dense operator when the padding mask is passed as a row-broadcast key
mask (B, 1, 1, Sk) -- valid tokens keep their order, so the causal test on padded positions equals the causal test
on gathered positions (for query_length < key_length under the left padding the reference assumes, :209-211) -- and
the padded query rows are zeroed afterwards. Few valid keys -> `flash_sparse_attn_func` takes its gathered-keys route.

Packed sequences given by position ids or cu_seqlens (:538-565, `_prepare_from_posids` :270-302) go through the
reference's varlen kernel as well. Here small packs (Tq x Tk up to `_PACKED_MASK_LIMIT` elements) run as ONE
sequence under a per-query visibility mask (same example, and causal inside the example with the bottom-right
alignment of its own lengths), which the full-range kernels skip tile by tile -- one launch however many examples
there are; larger packs go through `flash_sparse_attn_varlen_func`, which runs every example as a zero-copy slice.
"""
import os
from typing import Optional

import torch

from ..flash_sparse_attn_interface import flash_sparse_attn_func, flash_sparse_attn_varlen_func
from ..utils.mask import create_mask


def fsa_peft_integration_check(q, k, v, bias, target_dtype: Optional[torch.dtype] = None):
    """fp32 activations (PEFT keeps layer norms in fp32) go back to `target_dtype`; anything else passes through."""
    if target_dtype is not None and q.dtype == torch.float32:
        q, k, v = q.to(target_dtype), k.to(target_dtype), v.to(target_dtype)
        bias = bias.to(target_dtype) if bias is not None else None
    return q, k, v, bias


def _is_packed_sequence(position_ids: Optional[torch.Tensor], batch_size: int) -> bool:
    """Packed (padding-free) batches show up as one row of position ids that restarts from 0 somewhere
    (reference :279-296)."""
    if position_ids is None or position_ids.dim() != 2 or batch_size != 1 or position_ids.shape[1] < 2:
        return False
    expected = torch.arange(position_ids.shape[1], device=position_ids.device) + position_ids.min()
    return not bool((position_ids[0] == expected).all())


_PACKED_MASK_LIMIT = 1 << 24  # largest (Tq, Tk) visibility mask built for packed sequences; beyond: per-example calls


def _packed_visibility(cu_q: torch.Tensor, cu_k: torch.Tensor, total_q: int, total_k: int, causal: bool,
                       device) -> torch.Tensor:
    """(total_q, total_k) bool: query token i sees key token j iff both lie in the same example and, when causal,
    j_local <= i_local + len_k - len_q (the varlen kernels' bottom-right alignment per example). Tokens past the
    last boundary see nothing."""
    cu_q = cu_q.to(device=device, dtype=torch.int64)
    cu_k = cu_k.to(device=device, dtype=torch.int64)
    n = cu_q.numel() - 1
    tq = torch.arange(total_q, device=device)
    tk = torch.arange(total_k, device=device)
    sq = torch.bucketize(tq, cu_q[1:], right=True)   # example of each token; == n past the last boundary
    sk = torch.bucketize(tk, cu_k[1:], right=True)
    visible = (sq[:, None] == sk[None, :]) & (sq[:, None] < n) & (tq[:, None] >= cu_q[0]) & (tk[None, :] >= cu_k[0])
    if causal:
        sq_c = sq.clamp(max=n - 1)
        local_q = tq - cu_q[sq_c]
        local_k = tk - cu_k[sk.clamp(max=n - 1)]
        shift = (cu_k[1:] - cu_k[:-1] - (cu_q[1:] - cu_q[:-1]))[sq_c]
        visible &= local_k[None, :] <= (local_q + shift)[:, None]
    return visible


def _flash_sparse_attention_forward(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    attention_bias: Optional[torch.Tensor],
    query_length: int,
    key_length: int,
    is_causal: bool,
    position_ids: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    window_size: Optional[int] = None,
    softcap: Optional[float] = None,
    deterministic: Optional[bool] = None,
    cu_seq_lens_q: Optional[torch.LongTensor] = None,
    cu_seq_lens_k: Optional[torch.LongTensor] = None,
    max_length_q: Optional[int] = None,
    max_length_k: Optional[int] = None,
    target_dtype: Optional[torch.dtype] = None,
    implementation: Optional[str] = None,
    **kwargs,
):
    """query/key/value (B, S, H, d). Returns (B, Sq, H, d). Same argument list as the reference function."""
    if attention_mask is not None and attention_mask.dim() == 2 and attention_bias is not None:
        raise ValueError("If shape of attention_mask is (batch_size, seq_len), attention_bias has to be None.")
    padded = attention_mask is not None and attention_mask.dim() == 2
    packed_kwargs = all(x is not None for x in (cu_seq_lens_q, cu_seq_lens_k, max_length_q, max_length_k))
    packed = not padded and (packed_kwargs or _is_packed_sequence(position_ids, query_states.size(0)))

    query_states, key_states, value_states, attention_bias = fsa_peft_integration_check(
        query_states, key_states, value_states, attention_bias, target_dtype)
    if deterministic is None:
        deterministic = os.getenv("FLASH_SPARSE_ATTENTION_DETERMINISTIC", "0") == "1"

    if packed:
        if cu_seq_lens_q is None or cu_seq_lens_k is None:  # boundaries from the position ids (reference :241-251)
            flat = position_ids.reshape(-1)
            starts = (flat == 0).nonzero().view(-1).to(torch.int64)
            cu_seq_lens_q = cu_seq_lens_k = torch.cat(
                (starts, torch.tensor([flat.numel()], dtype=torch.int64, device=flat.device)))
        B = query_states.size(0)
        q1 = query_states.reshape(1, -1, query_states.size(-2), query_states.size(-1))
        k1 = key_states.reshape(1, -1, key_states.size(-2), key_states.size(-1))
        v1 = value_states.reshape(1, -1, value_states.size(-2), value_states.size(-1))
        if q1.size(1) * k1.size(1) > _PACKED_MASK_LIMIT:
            if max_length_q is None or max_length_k is None:
                max_length_q = int((cu_seq_lens_q[1:] - cu_seq_lens_q[:-1]).max())
                max_length_k = int((cu_seq_lens_k[1:] - cu_seq_lens_k[:-1]).max())
            out = flash_sparse_attn_varlen_func(q1[0], k1[0], v1[0], cu_seq_lens_q, cu_seq_lens_k, max_length_q,
                                                max_length_k, softmax_scale=softmax_scale, is_causal=is_causal,
                                                softcap=softcap, deterministic=deterministic)
            return out.view(B, -1, out.size(-2), out.size(-1))
        visible = _packed_visibility(cu_seq_lens_q, cu_seq_lens_k, q1.size(1), k1.size(1), is_causal, q1.device)
        out = flash_sparse_attn_func(q1, k1, v1, visible[None, None], None, softmax_scale=softmax_scale,
                                     is_causal=False, softcap=softcap, deterministic=deterministic)
        out = out[0] if isinstance(out, tuple) else out
        return out.view(B, -1, out.size(-2), out.size(-1))

    if padded:
        # static caches: k/v may be longer than the mask (reference :187-190)
        seq_len = attention_mask.shape[-1]
        if key_states.shape[1] > seq_len:
            key_states, value_states = key_states[:, :seq_len], value_states[:, :seq_len]
        key_valid = attention_mask.to(torch.bool)
        if query_length == key_states.shape[1]:
            query_valid = key_valid
        elif query_length == 1:
            query_valid = None
        else:
            query_valid = key_valid[:, -query_length:]  # left padding, as the reference assumes
        out = flash_sparse_attn_func(
            query_states, key_states, value_states, key_valid[:, None, None, :], None,
            softmax_scale=softmax_scale, is_causal=is_causal and query_length != 1,
            softcap=softcap, deterministic=deterministic)
        out = out[0] if isinstance(out, tuple) else out
        if query_valid is not None:
            out = torch.where(query_valid[:, :, None, None], out, torch.zeros((), dtype=out.dtype, device=out.device))
        return out

    if attention_bias is not None and window_size is not None and key_length > window_size:
        attention_mask = create_mask(
            attention_bias, attention_mask, batch_size=query_states.size(0), query_len=query_length,
            key_len=key_length, window_size=window_size, min_dtype=torch.finfo(attention_bias.dtype).min)
    out = flash_sparse_attn_func(
        query_states, key_states, value_states, attention_mask, attention_bias,
        softmax_scale=softmax_scale, is_causal=is_causal and query_length != 1,
        softcap=softcap, deterministic=deterministic)
    return out[0] if isinstance(out, tuple) else out
