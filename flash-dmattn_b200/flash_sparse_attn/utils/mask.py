"""`create_mask` with the reference's contract (flash_sparse_attn/utils/mask.py:163-240), computed by the
radix-select kernel behind `fdma_create_mask` instead of torch.topk + scatter_.

Differences a caller can observe: equal bias values at the selection threshold are taken in ascending key
order (torch.topk leaves that choice unspecified), and tensors must live on a CUDA device.
"""
import ctypes
from typing import NamedTuple, Optional

import torch

from .. import _lib

_TILE = 128


class KeptKeys(NamedTuple):
    """The selection of a row-broadcast dynamic mask as sorted positions instead of a bool tensor: what the
    reference's `topk_indices` returns (utils/mask.py:20-44), padded to a whole number of 128-key tiles.
    `flash_sparse_attn_func` accepts it in place of `attn_mask` and then never touches a bool mask."""

    key_pos: torch.Tensor    # int32 (Bm, Hm, Wp): ascending positions of the kept keys, INT32_MAX in unused slots
    count: torch.Tensor      # int32 (Bm, Hm): kept keys per row
    slot_mask: torch.Tensor  # bool (Bm, Hm, 1, Wp): slot < count
    seqlen_k: int            # number of keys the positions index into


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return {torch.bfloat16: _lib.FDMA_BF16, torch.float16: _lib.FDMA_FP16, torch.float32: _lib.FDMA_FP32}[t.dtype]
    except KeyError:
        raise RuntimeError(f"create_mask: unsupported bias dtype {t.dtype}") from None


def _launch(attention_bias, attention_mask, window_size, min_dtype, block_size, kind, positions="none"):
    """positions: "none" -> bool mask; "also" -> (bool mask, KeptKeys); "only" -> KeptKeys, no bool mask written."""
    bias = attention_bias.detach()
    if not bias.is_cuda:
        raise RuntimeError("create_mask: attention_bias must be a CUDA tensor (this build has no CPU path)")
    if bias.dim() != 4:
        raise RuntimeError("create_mask: attention_bias must have 4 dimensions")
    if bias.stride(-1) != 1:
        bias = bias.contiguous()
    pm = attention_mask
    if pm is not None:
        if pm.dtype != torch.bool:
            pm = pm.to(torch.bool)
        if pm.dim() != 4:
            raise RuntimeError("create_mask: attention_mask must have 2 or 4 dimensions")
        if pm.device != bias.device:
            raise RuntimeError("create_mask: attention_mask must be on the same device as attention_bias")
        if pm.stride(-1) != 1:
            pm = pm.contiguous()
    out_shape = torch.broadcast_shapes(bias.shape, pm.shape) if pm is not None else tuple(bias.shape)
    keys = out_shape[-1]
    if bias.shape[-1] != keys or (pm is not None and pm.shape[-1] != keys):
        # key-dimension broadcast is legal in torch but never used by callers; materialise it
        bias = bias.expand(*bias.shape[:-1], keys).contiguous()
        if pm is not None:
            pm = pm.expand(*pm.shape[:-1], keys).contiguous()
    if kind == _lib.MASK_TOPK and window_size > keys:
        raise RuntimeError("selected index k out of range")  # what torch.topk raises in the reference
    out = torch.empty(out_shape, dtype=torch.bool, device=bias.device) if positions not in ("only", "bits") else None
    want_bits = positions in ("bits", "bits_also")
    p = _lib.MaskParams()
    p.bias, p.premask = bias.data_ptr(), (pm.data_ptr() if pm is not None else None)
    p.out = out.data_ptr() if out is not None else None
    kept = None
    packed = None
    if want_bits:  # one bit per key (the kernel writes keys [0, keys); padding bits must be zero) + tile activity
        from ..packed import PackedMask

        words = (keys + _TILE - 1) // _TILE * (_TILE // 32)
        alloc = torch.empty if keys % _TILE == 0 else torch.zeros
        bits = alloc(tuple(out_shape[:3]) + (words,), dtype=torch.int32, device=bias.device)
        act = torch.empty(tuple(out_shape[:2]) + ((out_shape[2] + 127) // 128, (keys + _TILE - 1) // _TILE),
                          dtype=torch.uint8, device=bias.device)
        p.bits, p.activity = bits.data_ptr(), act.data_ptr()
        packed = PackedMask(bits, act, keys)
    elif positions in ("also", "only"):
        cap = max(_TILE, (min(int(window_size), keys) + _TILE - 1) // _TILE * _TILE)
        lead = tuple(out_shape[:2]) if out_shape[2] == 1 else tuple(out_shape[:3])
        key_pos = torch.empty(lead + (cap,), dtype=torch.int32, device=bias.device)
        count = torch.empty(lead, dtype=torch.int32, device=bias.device)
        slot_mask = torch.empty(tuple(out_shape[:3]) + (cap,), dtype=torch.bool, device=bias.device)
        p.key_pos, p.count, p.slot_mask, p.capacity = key_pos.data_ptr(), count.data_ptr(), slot_mask.data_ptr(), cap
        kept = KeptKeys(key_pos, count, slot_mask, keys)

    def strides(t):
        return [0 if t.shape[i] == 1 else t.stride(i) for i in range(3)]

    p.bias_batch_stride, p.bias_head_stride, p.bias_row_stride = strides(bias)
    if pm is not None:
        p.pm_batch_stride, p.pm_head_stride, p.pm_row_stride = strides(pm)
    p.out_b, p.out_h, p.out_rows, p.keys = out_shape
    p.window = int(window_size) if window_size is not None else 0
    p.dtype = _dtype_code(bias)
    p.kind = kind
    p.block_size = int(block_size) if block_size is not None else 0
    p.min_value = float(min_dtype)
    lib = _lib.load()
    with torch.cuda.device(bias.device):
        stream = torch.cuda.current_stream(bias.device).cuda_stream
        status = lib.fdma_create_mask(ctypes.byref(p), stream)
        if want_bits and status == _lib.ERR_UNSUPPORTED:
            if positions == "bits":
                return None  # the caller builds the bool mask and packs it
            p.bits, p.activity, packed = None, None, None  # bool mask alone
            status = lib.fdma_create_mask(ctypes.byref(p), stream)
        _lib.check(status, "fdma_create_mask")
    if positions == "bits":
        return packed
    if positions == "bits_also":
        return out, packed
    if positions == "only":
        return kept
    return (out, kept) if positions == "also" else out


def topk_mask(attention_bias, attention_mask, window_size, min_dtype, block_size=None, **kwargs):
    """Top-`window_size` keys per row by bias value (reference: utils/mask.py:76-120)."""
    if block_size is not None and block_size <= 0:
        raise ValueError(f"block_size must be a positive integer, got {block_size}.")
    return _launch(attention_bias, attention_mask, window_size, min_dtype, block_size, _lib.MASK_TOPK)


def _topk_mask_with_positions(attention_bias, attention_mask, window_size, min_dtype):
    """Bool mask and, from the same kernel launch, the sorted positions of its kept keys."""
    return _launch(attention_bias, attention_mask, window_size, min_dtype, None, _lib.MASK_TOPK, positions="also")


def relu_mask(attention_bias, attention_mask, min_dtype, block_size=None, **kwargs):
    """Keys whose (pre-masked) bias is positive (reference: utils/mask.py:123-159)."""
    if block_size is not None and block_size <= 0:
        raise ValueError(f"block_size must be a positive integer, got {block_size}.")
    return _launch(attention_bias, attention_mask, 0, min_dtype, block_size, _lib.MASK_RELU)


def topk_indices(attention_bias: torch.Tensor, window_size: int, **kwargs) -> torch.Tensor:
    """Sorted indices of the top-`window_size` keys of a (batch, kv_heads, key_len) bias
    (reference: utils/mask.py:20-44), derived from the selection kernel's mask."""
    b3 = attention_bias.detach()
    if window_size > b3.shape[-1]:
        raise RuntimeError("selected index k out of range")
    kept = _launch(b3.unsqueeze(2), None, window_size, float("-inf"), None, _lib.MASK_TOPK, positions="only")
    # the selection kernel writes the ascending positions itself; entries equal to -inf are never selected
    return kept.key_pos[..., :window_size].to(torch.int64)


def _reshape_padding_mask(attention_mask, batch_size, query_len, key_len):
    """2-D (B, Sk) / (B, Sq) padding masks -> (B, 1, 1, Sk), the latter left-padded with True (reference:
    utils/mask.py:198-218)."""
    if attention_mask is not None and attention_mask.dim() == 2:
        if attention_mask.shape[-1] == key_len:
            attention_mask = attention_mask.view(batch_size, 1, 1, key_len)
        elif attention_mask.shape[-1] == query_len:
            pad_len = key_len - query_len
            attention_mask = attention_mask.view(batch_size, 1, 1, query_len)
            if pad_len > 0:
                attention_mask = torch.nn.functional.pad(attention_mask, [pad_len, 0], value=True)
        else:
            raise ValueError(
                f"attention_mask shape {attention_mask.shape} is not compatible with key_len {key_len} "
                f"or query_len {query_len}."
            )
    return attention_mask


def create_mask(
    attention_bias: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    batch_size: int,
    query_len: int,
    key_len: int,
    window_size: int,
    min_dtype: float,
    block_size: Optional[int] = None,
    type: str = "topk",
) -> torch.Tensor:
    """Bool attention mask from the bias; same arguments and result shape as the reference's create_mask.

    attention_bias ({B|1}, {H|Hk|1}, {Sq|1}, Sk); attention_mask None, 4-D broadcastable to the bias, or
    2-D (B, Sk) / (B, Sq) padding mask (left-padded with True up to key_len). type "topk" keeps the
    window_size largest entries per row (never an entry equal to min_dtype); "relu" keeps bias > 0.
    block_size > 1 then replaces each block of keys by its majority vote.
    """
    attention_mask = _reshape_padding_mask(attention_mask, batch_size, query_len, key_len)
    if type == "topk":
        if block_size is not None and block_size <= 0:
            raise ValueError(f"block_size must be a positive integer, got {block_size}.")
        rows = attention_bias.shape[2] if attention_bias.dim() == 4 else 0
        if attention_mask is not None and attention_mask.dim() == 4:
            rows = max(rows, attention_mask.shape[2])
        if rows == 1 and (block_size is None or block_size <= 1) and 0 < window_size <= attention_bias.shape[-1]:
            # Row-broadcast selection: the same launch also writes the sorted positions of the kept keys. They ride
            # on the returned tensor as a cache that `flash_sparse_attn_func` uses to gather the kept keys without
            # re-reading the bool mask and without a device read-back; the tensor's version counter ties the cache
            # to the mask's current contents (any in-place edit invalidates it).
            mask, kept = _topk_mask_with_positions(attention_bias, attention_mask, window_size, min_dtype)
            mask._fdma_kept = (kept, mask._version)
            return mask
        if (rows > 1 and (block_size is None or block_size <= 1) and 0 < window_size <= attention_bias.shape[-1]
                and attention_bias.is_cuda and attention_bias.dim() == 4):
            # Per-query selection: the same launch also writes the mask as one bit per key, and a small kernel derives
            # the tile activity from the bits. Both ride on the returned tensor as a cache (tied to its version
            # counter like the position list above); `flash_sparse_attn_func` hands them to the kernels, which then
            # read an eighth of the mask bytes and need no activity pass of their own over the bool tensor.
            mask, packed = _launch(attention_bias, attention_mask, window_size, min_dtype, None, _lib.MASK_TOPK,
                                   positions="bits_also")
            if packed is not None:
                mask._fdma_packed = (packed, mask._version)
            return mask
        return topk_mask(attention_bias, attention_mask, window_size, min_dtype, block_size)
    if type == "relu":
        return relu_mask(attention_bias, attention_mask, min_dtype, block_size)
    raise ValueError(f"Unsupported mask type: {type}. Supported types are 'topk' and 'relu'.")


def create_kept_keys(
    attention_bias: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    batch_size: int,
    query_len: int,
    key_len: int,
    window_size: int,
    min_dtype: float,
) -> KeptKeys:
    """`create_mask(..., type="topk")` for a row-broadcast bias ({B|1}, {Hk|1}, 1, Sk), returned as the sorted
    positions of the kept keys (a `KeptKeys`) instead of a bool tensor: no (.., Sk) mask is written or read.
    Pass the result as `attn_mask` to `flash_sparse_attn_func`. Same selection as `create_mask`: the
    `window_size` largest entries per row, never an entry equal to `min_dtype`; `attention_mask` pre-masks keys
    (4-D broadcastable to the bias with one query row, or the 2-D padding forms `create_mask` takes)."""
    if attention_bias.dim() != 4 or attention_bias.shape[2] != 1:
        raise RuntimeError("create_kept_keys needs a row-broadcast bias of shape ({B|1}, {Hk|1}, 1, Sk)")
    attention_mask = _reshape_padding_mask(attention_mask, batch_size, query_len, key_len)
    if attention_mask is not None and attention_mask.shape[2] != 1:
        raise RuntimeError("create_kept_keys needs a pre-mask with one query row")
    return _launch(attention_bias, attention_mask, window_size, min_dtype, None, _lib.MASK_TOPK, positions="only")


def create_packed_mask(
    attention_bias: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    batch_size: int,
    query_len: int,
    key_len: int,
    window_size: int,
    min_dtype: float,
):
    """`create_mask(..., type="topk")` returned as a `packed.PackedMask` -- one bit per (query, key) and one activity
    byte per 128 x 128 tile -- instead of a bool tensor. Same selection as `create_mask` (the `window_size` largest
    entries per row, never an entry equal to `min_dtype`; `attention_mask` pre-masks keys). Pass the result as
    `attn_mask` to `flash_sparse_attn_func`. Meant for per-query biases (B, H, Sq, Sk), where the bool mask is as large
    as half the bias; for a row-broadcast bias `create_kept_keys` is the better form."""
    from ..packed import pack_mask

    attention_mask = _reshape_padding_mask(attention_mask, batch_size, query_len, key_len)
    packed = _launch(attention_bias, attention_mask, window_size, min_dtype, None, _lib.MASK_TOPK, positions="bits")
    if packed is None:  # a configuration the bit-writing kernel does not serve: bool mask first
        packed = pack_mask(_launch(attention_bias, attention_mask, window_size, min_dtype, None, _lib.MASK_TOPK))
    return packed
