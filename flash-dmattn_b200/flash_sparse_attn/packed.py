"""Bit-packed per-query masks: one bit per (query, key) instead of one byte, plus one byte per 128 x 128 tile that
says whether the tile holds a kept element. `utils.mask.create_packed_mask` writes both straight from the bias (no
bool tensor in between); `flash_sparse_attn_func` takes the result in place of `attn_mask`. The tensor-core kernels
read an eighth of the mask bytes on every pass and skip the kernel that derives the tile activity from a bool mask
(the reference always materialises the bool tensor: flash_sparse_attn/utils/mask.py:102-110,
csrc/flash_sparse_attn/flash_api.cpp:388-391).

Served natively: head dim 128 (forward and backward), masks with one row per query, batch extent of the mask equal to
the batch size. Anything else is expanded to the bool mask and takes the ordinary route."""
import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

_KEY_PAD = 128


@dataclass
class PackedMask:
    """bits (B, Hm, Sq, round_up(Sk,128)/32) int32: bit (k & 31) of word k >> 5 = key k kept (keys >= Sk: 0);
    activity (B, Hm, ceil(Sq/128), ceil(Sk/128)) uint8: non-zero iff the tile holds a kept element."""
    bits: torch.Tensor
    activity: torch.Tensor
    seqlen_k: int

    @property
    def shape(self):
        return (*self.bits.shape[:3], self.seqlen_k)

    def to_bool(self) -> torch.Tensor:
        """The (B, Hm, Sq, Sk) bool mask these bits stand for."""
        shifts = torch.arange(32, device=self.bits.device, dtype=torch.int32)
        m = ((self.bits.unsqueeze(-1) >> shifts) & 1).to(torch.bool)
        return m.reshape(*self.bits.shape[:3], -1)[..., : self.seqlen_k]


def pack_mask(mask: torch.Tensor) -> PackedMask:
    """Packs a bool mask (B, Hm, Sq, Sk) with torch operations (any device)."""
    B, Hm, Sq, Sk = mask.shape
    Sk_r = (Sk + _KEY_PAD - 1) // _KEY_PAD * _KEY_PAD
    m = torch.nn.functional.pad(mask, [0, Sk_r - Sk]) if Sk_r != Sk else mask
    shifts = torch.arange(32, device=mask.device, dtype=torch.int64)
    words = (m.reshape(B, Hm, Sq, Sk_r // 32, 32).to(torch.int64) << shifts).sum(dim=-1)
    bits = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    Sq_r = (Sq + 127) // 128 * 128
    mq = torch.nn.functional.pad(m, [0, 0, 0, Sq_r - Sq]) if Sq_r != Sq else m
    act = mq.reshape(B, Hm, Sq_r // 128, 128, Sk_r // 128, 128).any(dim=5).any(dim=3).to(torch.uint8)
    return PackedMask(bits.contiguous(), act.contiguous(), Sk)


def _native(q, k, packed: PackedMask, bias, needs_grad: bool) -> bool:
    B, Sq, H, d = q.shape
    if d != 128 or Sq == 1 or packed.bits.shape[0] != B or packed.bits.shape[2] != Sq:
        return False
    if packed.bits.shape[1] not in (1, k.shape[2], H) or packed.seqlen_k != k.shape[1]:
        return False
    return q.dtype in (torch.float16, torch.bfloat16) and packed.bits.is_cuda


class _PackedAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, bits, activity, softmax_scale, is_causal, deterministic):
        from . import flash_sparse_attn_interface as iface

        q, k, v, bias = (iface.maybe_contiguous(x) for x in (q, k, v, bias))
        keys_padded = iface.round_multiple(k.shape[1], _KEY_PAD)
        bias_keys_given = bias.shape[-1] if bias is not None else 0
        if bias is not None and bias.shape[-1] != keys_padded:
            bias = (bias.expand(*bias.shape[:-1], keys_padded) if bias.shape[-1] == 1
                    else torch.nn.functional.pad(bias, [0, keys_padded - bias.shape[-1]]))
        iface._check_inputs(q, k, v, None, bias)
        lib = _lib.load()
        B, Sq, H, d = q.shape
        with torch.cuda.device(q.device):
            iface._raise_if_kernel_timed_out(lib)
            out = torch.empty_like(q)
            lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
            p = _lib.FwdParams()
            _fill(p, q, k, v, bias, bits, activity, out, lse, softmax_scale, is_causal)
            ws_bytes = lib.fdma_fwd_workspace_bytes(ctypes.byref(p))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
            if ws is not None:
                p.workspace, p.workspace_bytes = ws.data_ptr(), ws_bytes
            _lib.check(lib.fdma_fwd(ctypes.byref(p), iface._stream_ptr(q.device)), "fdma_fwd")
        ctx.save_for_backward(q, k, v, bias, bits, activity, out, lse)
        ctx.scale, ctx.causal, ctx.det, ctx.bias_keys_given = softmax_scale, is_causal, deterministic, bias_keys_given
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import flash_sparse_attn_interface as iface

        q, k, v, bias, bits, activity, out, lse = ctx.saved_tensors
        dout = iface.maybe_contiguous(dout)
        lib = _lib.load()
        B, Sq, H, d = q.shape
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dbias = torch.empty(bias.shape, dtype=bias.dtype, device=bias.device) if bias is not None else None
        with torch.cuda.device(q.device):
            iface._raise_if_kernel_timed_out(lib)
            bp = _lib.BwdParams()
            _fill(bp.f, q, k, v, bias, bits, activity, out, lse, ctx.scale, ctx.causal)
            bp.dout = dout.data_ptr()
            bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride = iface._bsh(dout)
            bp.dq, bp.dk, bp.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
            bp.dq_batch_stride, bp.dq_row_stride, bp.dq_head_stride = iface._bsh(dq)
            bp.dk_batch_stride, bp.dk_row_stride, bp.dk_head_stride = iface._bsh(dk)
            bp.dv_batch_stride, bp.dv_row_stride, bp.dv_head_stride = iface._bsh(dv)
            if dbias is not None:
                bp.dbias = dbias.data_ptr()
                bp.dbias_batch_stride, bp.dbias_head_stride, bp.dbias_row_stride = dbias.stride()[:3]
                bp.dbias_b, bp.dbias_h, bp.dbias_rows, bp.dbias_keys = dbias.shape
            else:
                bp.dbias = None
            bp.deterministic = 1 if ctx.det else 0
            bp.softmax_d = None
            ws_bytes = lib.fdma_bwd_workspace_bytes(ctypes.byref(bp))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
            if ws is not None:
                bp.f.workspace, bp.f.workspace_bytes = ws.data_ptr(), ws_bytes
            _lib.check(lib.fdma_bwd(ctypes.byref(bp), iface._stream_ptr(q.device)), "fdma_bwd")
        if dbias is not None:
            dbias = dbias[..., : k.shape[1]]
            if ctx.bias_keys_given == 1:
                dbias = dbias.sum(dim=-1, keepdim=True)
        return dq, dk, dv, dbias, None, None, None, None, None


def _fill(p, q, k, v, bias, bits, activity, out, lse, softmax_scale, is_causal):
    from . import flash_sparse_attn_interface as iface

    iface._fill_fwd(p, q, k, v, None, bias, out, lse, softmax_scale, is_causal)
    p.mask = bits.data_ptr()
    p.mask_bits = 1
    p.h_mask = bits.shape[1]
    p.mask_batch_stride, p.mask_head_stride, p.mask_row_stride = bits.stride()[:3]
    if bits.shape[1] == 1:
        p.mask_head_stride = 0
    p.tile_activity = activity.data_ptr()


def flash_sparse_attn_packed_func(query, key, value, packed: PackedMask, attn_bias: Optional[torch.Tensor] = None,
                                  softmax_scale: Optional[float] = None, is_causal: Optional[bool] = None,
                                  deterministic: Optional[bool] = None) -> torch.Tensor:
    """`flash_sparse_attn_func` with the mask given as a `PackedMask`. Falls back to the bool mask where the kernels
    do not read bits (see the module docstring)."""
    from .flash_sparse_attn_interface import flash_sparse_attn_func

    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value))
    if not _native(query, key, packed, attn_bias, needs_grad):
        return flash_sparse_attn_func(query, key, value, packed.to_bool(), attn_bias, softmax_scale, is_causal,
                                      None, deterministic)
    scale = query.shape[-1] ** (-0.5) if softmax_scale is None else softmax_scale
    return _PackedAttnFunc.apply(query, key, value, attn_bias, packed.bits, packed.activity, float(scale),
                                 bool(is_causal), bool(deterministic))
