"""Key compaction for row-broadcast dynamic masks.

When a mask keeps the same W of Sk keys for every query of a (batch, head) -- the usual shape of a dynamic mask
built from one importance row per head, ({B|1}, {Hk|1}, 1, Sk) -- the attention over all Sk keys equals the
attention over the W kept keys, as long as the causal test still sees the keys' original positions. This module
gathers K, V and the bias of the kept keys into dense (B, Wp, Hk, d) tensors, runs the attention kernels over them
with the position list, and scatters dK, dV and dBias back to their full shapes. Tiles are then W/128 per query
block instead of "every 128-key tile that holds at least one kept key", which for scattered keep-sets is the
difference between W/128 and Sk/128 tiles.

The reference's CUDA backend has no such path; its Triton prototype gathers the top-k keys per head in the same
way (flash_sparse_attn/flash_dmattn_triton.py:49-211). `flash_sparse_attn_func` takes this route by itself for the
mask shapes it fits (see `set_compaction`); `flash_sparse_attn_compact_func` asks for it explicitly.
"""
from typing import NamedTuple, Optional, Tuple

import ctypes
import torch

from . import _lib
from .flash_sparse_attn_interface import (_bsh, _check_inputs, _dtype_code, _fill_fwd, _raise_if_kernel_timed_out,
                                          _stream_ptr, round_multiple)

__all__ = ["CompactKeys", "compact_keys", "index_kept_keys", "gather_kept_keys", "scatter_kept_rows",
           "compact_forward", "compact_backward", "flash_sparse_attn_compact_func", "kept_keys_to_mask"]

_TILE = 128


class CompactKeys(NamedTuple):
    key: torch.Tensor          # (B, Wp, Hk, d)
    value: torch.Tensor        # (B, Wp, Hk, d)
    mask: torch.Tensor         # bool (Bm, Hm, 1, Wp): slot holds a kept key
    bias: Optional[torch.Tensor]  # (Bb, Hb, 1, Wp) or None
    key_pos: torch.Tensor      # int32 (Bm, Hm, Wp): ascending positions, INT32_MAX in unused slots
    count: torch.Tensor        # int32 (Bm, Hm): kept keys per row
    seqlen_k: int              # original number of keys


def _row_mask(attn_mask: torch.Tensor, B: int, Hk: int, Sk: int) -> torch.Tensor:
    if attn_mask.dtype != torch.bool or attn_mask.dim() != 4:
        raise RuntimeError("attn_mask must be a 4-D bool tensor")
    Bm, Hm, rows, keys = attn_mask.shape
    if rows != 1:
        raise RuntimeError("key compaction needs a row-broadcast mask: shape ({B|1}, {Hk|1}, 1, Sk)")
    if Bm not in (1, B) or Hm not in (1, Hk):
        raise RuntimeError("key compaction needs mask batch in {1, B} and mask heads in {1, num_heads_k}")
    if keys < Sk:
        raise RuntimeError("attn_mask has fewer keys than key")
    m = attn_mask[:, :, 0, :Sk]
    return m if m.stride(-1) == 1 else m.contiguous()


def _rows_params(src, dst, key_pos, b, heads, rows_full, cap, row_elems, src_strides, dst_strides):
    """fdma_rows_params for a gather (src full, dst compact) or a scatter (src compact, dst full)."""
    rp = _lib.RowsParams()
    rp.src, rp.dst, rp.key_pos = src.data_ptr(), dst.data_ptr(), key_pos.data_ptr()
    rp.key_pos_batch_stride = 0 if key_pos.shape[0] == 1 else key_pos.stride(0)
    rp.key_pos_head_stride = key_pos.stride(1)
    rp.src_batch_stride, rp.src_row_stride, rp.src_head_stride = src_strides
    rp.dst_batch_stride, rp.dst_row_stride, rp.dst_head_stride = dst_strides
    rp.b, rp.heads, rp.h_pos, rp.rows_full, rp.capacity, rp.row_elems = b, heads, key_pos.shape[1], rows_full, cap, row_elems
    rp.dtype = _dtype_code(src)
    return rp


def _rows_call(fn, src, dst, key_pos, b, heads, rows_full, cap, row_elems, src_strides, dst_strides, device):
    rp = _rows_params(src, dst, key_pos, b, heads, rows_full, cap, row_elems, src_strides, dst_strides)
    _lib.check(fn(ctypes.byref(rp), _stream_ptr(device)), fn.__name__)


def _bias_layout(attn_bias: torch.Tensor, key_pos: torch.Tensor, B: int):
    """Batch / head extents of the compacted bias: the bias' own, widened to the position list's where that varies."""
    Bb, Hb = attn_bias.shape[0], attn_bias.shape[1]
    Bm, Hm = key_pos.shape[0], key_pos.shape[1]
    if Bb not in (1, B):
        raise RuntimeError("attn_bias batch dimension must be 1 or batch_size")
    if attn_bias.shape[2] != 1:
        raise RuntimeError("key compaction needs a row-broadcast bias: shape ({B|1}, {H|Hk|1}, 1, Sk)")
    Bc, Hc = max(Bb, Bm), max(Hb, Hm)
    if Hc % Hm:
        raise RuntimeError("attn_bias heads must be a multiple of the mask heads")
    return Bc, Hc


def compact_keys(key: torch.Tensor, value: torch.Tensor, attn_mask: torch.Tensor,
                 attn_bias: Optional[torch.Tensor] = None, capacity: Optional[int] = None,
                 check_capacity: bool = True) -> CompactKeys:
    """Gathers the kept keys of a row-broadcast mask. `capacity` is the number of slots per row (rounded up to a
    multiple of 128); when omitted it is taken from the fullest mask row, which costs one device synchronisation.
    A row with more kept keys than `capacity` raises; that check reads the counts back (one synchronisation) and is
    skipped with check_capacity=False, for callers that know the bound holds."""
    B, Sk, Hk, d = key.shape
    m = _row_mask(attn_mask, B, Hk, Sk)
    key_pos, count, mask_c = index_kept_keys(m, capacity, check_capacity)
    k_c, v_c, bias_c = gather_kept_keys(key, value, attn_bias, key_pos)
    return CompactKeys(k_c, v_c, mask_c, bias_c, key_pos, count, Sk)


def index_kept_keys(m: torch.Tensor, capacity: Optional[int] = None, check_capacity: bool = True):
    """m: bool (Bm, Hm, Sk), keys contiguous. Returns key_pos (Bm,Hm,Wp) int32 (ascending positions of the kept
    keys, INT32_MAX in unused slots), count (Bm,Hm) int32 and the compact mask (Bm,Hm,1,Wp)."""
    lib = _lib.load()
    Bm, Hm, Sk = m.shape
    dev = m.device
    with torch.cuda.device(dev):
        if capacity is None:
            capacity = int(m.sum(dim=-1, dtype=torch.int32).max().item())
        cap = max(_TILE, round_multiple(int(capacity), _TILE))
        key_pos = torch.empty((Bm, Hm, cap), dtype=torch.int32, device=dev)
        count = torch.empty((Bm, Hm), dtype=torch.int32, device=dev)
        mask_c = torch.empty((Bm, Hm, 1, cap), dtype=torch.bool, device=dev)
        cp = _lib.CompactParams()
        cp.mask = m.data_ptr()
        cp.mask_batch_stride, cp.mask_head_stride = m.stride(0), m.stride(1)
        cp.b_mask, cp.h_mask, cp.seqlen_k, cp.capacity = Bm, Hm, Sk, cap
        cp.key_pos, cp.count, cp.mask_out = key_pos.data_ptr(), count.data_ptr(), mask_c.data_ptr()
        _lib.check(lib.fdma_compact_index(ctypes.byref(cp), _stream_ptr(dev)), "fdma_compact_index")
        if check_capacity and int(count.max().item()) > cap:
            raise RuntimeError(f"a mask row keeps more than capacity={cap} keys")
    return key_pos, count, mask_c


def gather_kept_keys(key, value, attn_bias, key_pos):
    """K, V (B,Sk,Hk,d) and bias ({B|1},{H|Hk|1},1,Sk) rows at key_pos (Bm,Hm,Wp) -> (B,Wp,Hk,d) x 2 and
    (Bc,Hc,1,Wp); slots whose position lies outside [0, Sk) come out as zeros."""
    lib = _lib.load()
    B, Sk, Hk, d = key.shape
    cap = key_pos.shape[-1]
    dev = key.device
    with torch.cuda.device(dev):
        key = key if key.stride(-1) == 1 else key.contiguous()
        value = value if value.stride(-1) == 1 else value.contiguous()
        k_c = torch.empty((B, cap, Hk, d), dtype=key.dtype, device=dev)
        v_c = torch.empty((B, cap, Hk, d), dtype=key.dtype, device=dev)
        for src, dst in ((key, k_c), (value, v_c)):
            _rows_call(lib.fdma_gather_rows, src, dst, key_pos, B, Hk, Sk, cap, d, _bsh(src), _bsh(dst), dev)
        bias_c = None
        if attn_bias is not None:
            Bc, Hc = _bias_layout(attn_bias, key_pos, B)
            bias_c = torch.empty((Bc, Hc, 1, cap), dtype=attn_bias.dtype, device=dev)
            sb = 0 if attn_bias.shape[0] == 1 else attn_bias.stride(0)
            sh = 0 if attn_bias.shape[1] == 1 else attn_bias.stride(1)
            sr = 0 if attn_bias.shape[3] == 1 else attn_bias.stride(3)
            _rows_call(lib.fdma_gather_rows, attn_bias, bias_c, key_pos, Bc, Hc, Sk, cap, 1, (sb, sr, sh),
                       (bias_c.stride(0), 1, bias_c.stride(1)), dev)
    return k_c, v_c, bias_c


def scatter_kept_rows(src_c: torch.Tensor, key_pos: torch.Tensor, rows_full: int, bias_layout: bool = False) -> torch.Tensor:
    """Inverse of the gather for gradients: src_c (B,Wp,Hk,d) -> (B,rows_full,Hk,d), or with bias_layout
    (Bc,Hc,1,Wp) -> (Bc,Hc,1,rows_full); rows that no slot points at are zero."""
    lib = _lib.load()
    dev = src_c.device
    cap = key_pos.shape[-1]
    with torch.cuda.device(dev):
        if bias_layout:
            Bc, Hc = src_c.shape[0], src_c.shape[1]
            full = torch.empty((Bc, Hc, 1, rows_full), dtype=src_c.dtype, device=dev)
            _rows_call(lib.fdma_scatter_rows, src_c, full, key_pos, Bc, Hc, rows_full, cap, 1,
                       (src_c.stride(0), 1, src_c.stride(1)), (full.stride(0), 1, full.stride(1)), dev)
            return full
        B, _, Hk, d = src_c.shape
        full = torch.empty((B, rows_full, Hk, d), dtype=src_c.dtype, device=dev)
        _rows_call(lib.fdma_scatter_rows, src_c, full, key_pos, B, Hk, rows_full, cap, d, _bsh(src_c), _bsh(full), dev)
        return full


def _set_positions(p, ck: CompactKeys, seqlen_q: int, causal_shift: Optional[int] = None):
    p.key_pos = ck.key_pos.data_ptr()
    p.key_pos_batch_stride = 0 if ck.key_pos.shape[0] == 1 else ck.key_pos.stride(0)
    p.key_pos_head_stride = ck.key_pos.stride(1)
    p.h_pos = ck.key_pos.shape[1]
    p.causal_shift = ck.seqlen_k - seqlen_q if causal_shift is None else causal_shift


def compact_forward(q: torch.Tensor, ck: CompactKeys, softmax_scale: float, is_causal: bool,
                    causal_shift: Optional[int] = None):
    """Forward over gathered keys: returns (out (B,Sq,H,d), lse (B,H,Sq) fp32). Key slot k is visible to query row
    i iff key_pos[k] <= i + causal_shift (default: the bottom-right alignment, seqlen_k - seqlen_q)."""
    lib = _lib.load()
    _check_inputs(q, ck.key, ck.value, ck.mask, ck.bias)
    B, Sq, H, d = q.shape
    dev = q.device
    with torch.cuda.device(dev):
        _raise_if_kernel_timed_out(lib)
        out = torch.empty_like(q)
        lse = torch.empty((B, H, Sq), dtype=torch.float32, device=dev)
        p = _lib.FwdParams()
        _fill_fwd(p, q, ck.key, ck.value, ck.mask, ck.bias, out, lse, softmax_scale, is_causal)
        _set_positions(p, ck, Sq, causal_shift)
        ws_bytes = lib.fdma_fwd_workspace_bytes(ctypes.byref(p))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws_bytes
        _lib.check(lib.fdma_fwd(ctypes.byref(p), _stream_ptr(dev)), "fdma_fwd")
    return out, lse


def compact_backward(dout, q, ck: CompactKeys, out, lse, softmax_scale: float, is_causal: bool, k_shape,
                     bias_shape=None, causal_shift: Optional[int] = None, scatter: bool = True,
                     deterministic: bool = False):
    """Backward over gathered keys, gradients scattered back to full shapes: returns dq, dk, dv (shape k_shape) and
    dbias (shape bias_shape, or None). Dimensions the bias broadcast over are summed. scatter=False returns the
    gradients of the gathered tensors themselves (dq, dk_c, dv_c, dbias_c)."""
    lib = _lib.load()
    k_c, v_c, mask_c, bias_c, key_pos, Sk = ck.key, ck.value, ck.mask, ck.bias, ck.key_pos, ck.seqlen_k
    B, Sq, H, d = q.shape
    Hk, cap = k_c.shape[2], k_c.shape[1]
    dev = q.device
    dout = dout if dout.stride(-1) == 1 else dout.contiguous()
    with torch.cuda.device(dev):
        _raise_if_kernel_timed_out(lib)
        dq = torch.empty_like(q)
        dk_c, dv_c = torch.empty_like(k_c), torch.empty_like(v_c)
        dbias_c = torch.empty_like(bias_c) if bias_c is not None else None
        bp = _lib.BwdParams()
        _fill_fwd(bp.f, q, k_c, v_c, mask_c, bias_c, out, lse, softmax_scale, is_causal)
        _set_positions(bp.f, ck, Sq, causal_shift)
        bp.dout = dout.data_ptr()
        bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride = _bsh(dout)
        bp.dq, bp.dk, bp.dv = dq.data_ptr(), dk_c.data_ptr(), dv_c.data_ptr()
        bp.dq_batch_stride, bp.dq_row_stride, bp.dq_head_stride = _bsh(dq)
        bp.dk_batch_stride, bp.dk_row_stride, bp.dk_head_stride = _bsh(dk_c)
        bp.dv_batch_stride, bp.dv_row_stride, bp.dv_head_stride = _bsh(dv_c)
        if dbias_c is not None:
            bp.dbias = dbias_c.data_ptr()
            bp.dbias_batch_stride, bp.dbias_head_stride, bp.dbias_row_stride = dbias_c.stride()[:3]
            bp.dbias_b, bp.dbias_h, bp.dbias_rows, bp.dbias_keys = dbias_c.shape
        bp.deterministic = 1 if deterministic else 0
        ws_bytes = lib.fdma_bwd_workspace_bytes(ctypes.byref(bp))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
        if ws is not None:
            bp.f.workspace, bp.f.workspace_bytes = ws.data_ptr(), ws_bytes
        _lib.check(lib.fdma_bwd(ctypes.byref(bp), _stream_ptr(dev)), "fdma_bwd")
        if not scatter:
            return dq, dk_c, dv_c, dbias_c
        dk = torch.empty(k_shape, dtype=q.dtype, device=dev)
        dv = torch.empty(k_shape, dtype=q.dtype, device=dev)
        for src, dst in ((dk_c, dk), (dv_c, dv)):
            _rows_call(lib.fdma_scatter_rows, src, dst, key_pos, B, Hk, Sk, cap, d, _bsh(src), _bsh(dst), dev)
        dbias = None
        if dbias_c is not None:
            Bc, Hc = dbias_c.shape[0], dbias_c.shape[1]
            full = torch.empty((Bc, Hc, 1, Sk), dtype=q.dtype, device=dev)
            _rows_call(lib.fdma_scatter_rows, dbias_c, full, key_pos, Bc, Hc, Sk, cap, 1,
                       (dbias_c.stride(0), 1, dbias_c.stride(1)), (full.stride(0), 1, full.stride(1)), dev)
            # dimensions the bias broadcast over (and the compaction widened) are summed back
            for dim in (0, 1, 3):
                if bias_shape[dim] == 1 and full.shape[dim] != 1:
                    full = full.sum(dim=dim, keepdim=True, dtype=torch.float32).to(q.dtype)
            if bias_shape[3] > Sk:
                full = torch.nn.functional.pad(full, [0, bias_shape[3] - Sk])
            dbias = full
    return dq, dk, dv, dbias


def kept_keys_to_mask(kept) -> torch.Tensor:
    """Bool mask (Bm, Hm, 1, Sk) of a `KeptKeys` position list (for calls the gathered route does not serve)."""
    Bm, Hm, cap = kept.key_pos.shape
    Sk = kept.seqlen_k
    mask = torch.zeros((Bm, Hm, 1, Sk + 1), dtype=torch.bool, device=kept.key_pos.device)
    idx = kept.key_pos.clamp(max=Sk).to(torch.int64).unsqueeze(2)          # unused slots land in the spare column
    mask.scatter_(-1, idx, torch.ones_like(idx, dtype=torch.bool))
    return mask[..., :Sk]


# ------------------------------------------------------------------------------------------------------------------
# The gathered route as custom ops (with fake kernels), so that torch.compile traces it like the dense operators.
# ------------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("flash_sparse_attn::_index_kept_keys", mutates_args=(), device_types="cuda")
def _index_kept_keys_op(mask_rows: torch.Tensor, capacity: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """mask_rows bool (Bm, Hm, Sk) -> key_pos (Bm, Hm, Wp) int32, count (Bm, Hm) int32, slot mask (Bm, Hm, 1, Wp)."""
    m = mask_rows if mask_rows.stride(-1) == 1 else mask_rows.contiguous()
    return index_kept_keys(m, capacity, check_capacity=False)


@torch.library.register_fake("flash_sparse_attn::_index_kept_keys")
def _index_kept_keys_fake(mask_rows, capacity):
    Bm, Hm, _ = mask_rows.shape
    cap = max(_TILE, round_multiple(int(capacity), _TILE))
    dev = mask_rows.device
    return (torch.empty((Bm, Hm, cap), dtype=torch.int32, device=dev),
            torch.empty((Bm, Hm), dtype=torch.int32, device=dev),
            torch.empty((Bm, Hm, 1, cap), dtype=torch.bool, device=dev))


def _bias_c_shape(bias, key_pos, B):
    Bc, Hc = _bias_layout(bias, key_pos, B)
    return (Bc, Hc, 1, key_pos.shape[-1])


@torch.library.custom_op("flash_sparse_attn::_compact_forward", mutates_args=(), device_types="cuda")
def _compact_forward_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: Optional[torch.Tensor],
                        key_pos: torch.Tensor, slot_mask: torch.Tensor, softmax_scale: float, is_causal: bool,
                        ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gather K, V, bias at key_pos and run the forward over the gathered keys. Returns out, lse and the gathered
    K, V, bias (an empty tensor without a bias), which the backward reuses."""
    q = q if q.stride(-1) == 1 else q.contiguous()
    k_c, v_c, bias_c = gather_kept_keys(k, v, bias, key_pos)
    ck = CompactKeys(k_c, v_c, slot_mask, bias_c, key_pos, None, k.shape[1])
    out, lse = compact_forward(q, ck, softmax_scale, is_causal)
    if bias_c is None:
        bias_c = torch.empty((0,), dtype=q.dtype, device=q.device)
    return out, lse, k_c, v_c, bias_c


@torch.library.register_fake("flash_sparse_attn::_compact_forward")
def _compact_forward_fake(q, k, v, bias, key_pos, slot_mask, softmax_scale, is_causal):
    B, Sq, H, d = q.shape
    Hk, cap = k.shape[2], key_pos.shape[-1]
    kc = torch.empty((B, cap, Hk, d), dtype=q.dtype, device=q.device)
    bias_c = (torch.empty(_bias_c_shape(bias, key_pos, B), dtype=q.dtype, device=q.device) if bias is not None
              else torch.empty((0,), dtype=q.dtype, device=q.device))
    return (torch.empty_like(q), torch.empty((B, H, Sq), dtype=torch.float32, device=q.device), kc,
            torch.empty_like(kc), bias_c)


@torch.library.custom_op("flash_sparse_attn::_compact_backward", mutates_args=(), device_types="cuda")
def _compact_backward_op(dout: torch.Tensor, q: torch.Tensor, k_c: torch.Tensor, v_c: torch.Tensor,
                         bias_c: Optional[torch.Tensor], key_pos: torch.Tensor, slot_mask: torch.Tensor,
                         out: torch.Tensor, lse: torch.Tensor, softmax_scale: float, is_causal: bool, seqlen_k: int,
                         bias_b: int, bias_h: int, bias_keys: int, deterministic: bool,
                         ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward over the gathered keys; dK, dV come back scattered to (B, seqlen_k, Hk, d) and dBias to
    (bias_b, bias_h, 1, bias_keys) (an empty tensor without a bias)."""
    B, cap, Hk, d = k_c.shape
    ck = CompactKeys(k_c, v_c, slot_mask, bias_c, key_pos, None, seqlen_k)
    dq, dk, dv, dbias = compact_backward(dout, q, ck, out, lse, softmax_scale, is_causal, (B, seqlen_k, Hk, d),
                                         (bias_b, bias_h, 1, bias_keys) if bias_c is not None else None,
                                         deterministic=deterministic)
    if dbias is None:
        dbias = torch.empty((0,), dtype=q.dtype, device=q.device)
    return dq, dk, dv, dbias


@torch.library.register_fake("flash_sparse_attn::_compact_backward")
def _compact_backward_fake(dout, q, k_c, v_c, bias_c, key_pos, slot_mask, out, lse, softmax_scale, is_causal, seqlen_k,
                           bias_b, bias_h, bias_keys, deterministic):
    B, cap, Hk, d = k_c.shape
    dk = torch.empty((B, seqlen_k, Hk, d), dtype=q.dtype, device=q.device)
    dbias = (torch.empty((bias_b, bias_h, 1, bias_keys), dtype=q.dtype, device=q.device) if bias_c is not None
             else torch.empty((0,), dtype=q.dtype, device=q.device))
    return torch.empty_like(q), dk, torch.empty_like(dk), dbias


class _CompactAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, key_pos, slot_mask, softmax_scale, is_causal, deterministic):
        out, lse, k_c, v_c, bias_c = torch.ops.flash_sparse_attn._compact_forward(
            q, k, v, bias, key_pos, slot_mask, softmax_scale, is_causal)
        ctx.save_for_backward(q, k_c, v_c, slot_mask, key_pos, out, lse, bias_c)
        ctx.has_bias = bias is not None
        ctx.deterministic = bool(deterministic)
        ctx.meta = (softmax_scale, is_causal, k.shape[1], tuple(bias.shape) if bias is not None else (0, 0, 0, 0))
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k_c, v_c, slot_mask, key_pos, out, lse, bias_c = ctx.saved_tensors
        softmax_scale, is_causal, Sk, bias_shape = ctx.meta
        dq, dk, dv, dbias = torch.ops.flash_sparse_attn._compact_backward(
            dout, q, k_c, v_c, bias_c if ctx.has_bias else None, key_pos, slot_mask, out, lse, softmax_scale,
            is_causal, Sk, bias_shape[0], bias_shape[1], bias_shape[3], ctx.deterministic)
        return dq, dk, dv, (dbias if ctx.has_bias else None), None, None, None, None, None


def flash_sparse_attn_compact_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask,
    attn_bias: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    is_causal: Optional[bool] = None,
    capacity: Optional[int] = None,
    _trusted_capacity: bool = False,
    deterministic: bool = False,
):
    """Same result as `flash_sparse_attn_func(query, key, value, attn_mask, attn_bias, softmax_scale, is_causal)`
    for a row-broadcast mask ({B|1}, {Hk|1}, 1, Sk) and bias ({B|1}, {H|Hk|1}, 1, Sk), computed over the kept keys
    only. attn_mask is a bool tensor or the `KeptKeys` position list of `utils.mask.create_kept_keys` (then no bool
    mask is read at all). `capacity` bounds the kept keys per row of a bool mask (e.g. the keep_window_size it was
    built with); when omitted it is read back from the device. head_dim must be a multiple of 8."""
    from .utils.mask import KeptKeys

    softmax_scale = query.shape[-1] ** (-0.5) if softmax_scale is None else softmax_scale
    is_causal = bool(is_causal) if is_causal is not None else False
    B, Sk, Hk, _ = key.shape
    if attn_bias is not None and attn_bias.shape[-1] not in (1, Sk) and attn_bias.shape[-1] < Sk:
        raise RuntimeError("attn_bias has fewer keys than key")
    if isinstance(attn_mask, KeptKeys):
        if attn_mask.seqlen_k != Sk:
            raise RuntimeError("the position list was built for a different number of keys")
        key_pos, slot_mask = attn_mask.key_pos, attn_mask.slot_mask
    else:
        m = _row_mask(attn_mask, B, Hk, Sk)
        trusted = _trusted_capacity and capacity is not None
        if capacity is None:
            capacity = int(m.sum(dim=-1, dtype=torch.int32).max().item())
        key_pos, count, slot_mask = torch.ops.flash_sparse_attn._index_kept_keys(m, int(capacity))
        if not trusted and int(count.max().item()) > key_pos.shape[-1]:
            raise RuntimeError(f"a mask row keeps more than capacity={key_pos.shape[-1]} keys")
    return _CompactAttnFunc.apply(query, key, value, attn_bias, key_pos, slot_mask, softmax_scale, is_causal,
                                  bool(deterministic))
