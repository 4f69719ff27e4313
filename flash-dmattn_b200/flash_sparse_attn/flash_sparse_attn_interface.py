"""Python operator layer of the B200 dynamic-mask attention library.

Mirrors the public surface of the reference's CUDA backend
(flash_sparse_attn/flash_sparse_attn_interface.py:610-684 `flash_sparse_attn_func`, :382-498
`FlashDMAttnFunc`, custom ops :73-99 and :206-251): same names, argument order, defaults, saved tensors and
gradient slicing. Underneath, tensors are handed as raw pointers + element strides to the C ABI declared in
include/fdma.h; PyTorch only owns memory and the stream.
"""
from typing import Any, Optional, Tuple

import ctypes
import torch

from . import _lib

__all__ = ["flash_sparse_attn_func", "flash_sparse_attn_varlen_func", "FlashDMAttnFunc", "set_kernel_path",
           "set_compaction"]

_KEY_PAD = 128  # mask / bias key dimension is padded to a multiple of this (interface.py:420-430 of the reference)
_kernel_path = _lib.PATH_AUTO


def set_kernel_path(path: str) -> None:
    """Selects the kernel family: "auto" (default), "simt" (CUDA-core kernels), "tcgen05" or "decode". Used by tests."""
    global _kernel_path
    _kernel_path = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tcgen05": _lib.PATH_TCGEN05,
                    "decode": _lib.PATH_DECODE}[path]


_compaction = "auto"


def set_compaction(mode: str) -> None:
    """"auto" (default): a row-broadcast mask is handled by gathering its kept keys first (see compaction.py);
    "off": always run over the full key range with tile skipping."""
    global _compaction
    if mode not in ("auto", "off"):
        raise ValueError("compaction mode must be 'auto' or 'off'")
    _compaction = mode


def _compaction_capacity(query, key, attn_mask, attn_bias, softcap, return_attn_probs) -> Optional[int]:
    """Slots per mask row if this call is to run over gathered keys, else None. Eligible: Sq > 1, head dim a
    multiple of 8, mask ({B|1}, {Hk|1}, 1, >=Sk) -- a bool tensor or the `KeptKeys` positions that
    `utils.mask.create_kept_keys` returns --, bias absent or row-broadcast, no softcap / returned probabilities.
    The slot count comes from the position list itself when there is one: passed in, or cached on the bool mask by
    `create_mask` and still valid. Any other bool mask has its counts read back from the device, which
    synchronises the stream. A mask that keeps more than three quarters of the keys is left to the tile-skipping
    path."""
    from .utils.mask import KeptKeys

    if _compaction != "auto" or attn_mask is None or softcap or return_attn_probs:
        return None
    if query.dim() != 4 or key.dim() != 4:
        return None
    B, Sq, H, d = query.shape
    Sk, Hk = key.shape[1], key.shape[2]
    if Sq <= 1 or d % 8 or not query.is_cuda:
        return None
    if attn_bias is not None:
        if attn_bias.dim() != 4 or attn_bias.shape[2] != 1 or attn_bias.shape[3] < Sk:
            return None
        if attn_bias.shape[0] not in (1, B) or attn_bias.shape[1] not in (1, Hk, H):
            return None
    if isinstance(attn_mask, KeptKeys):
        kp = attn_mask.key_pos
        if attn_mask.seqlen_k != Sk or kp.shape[0] not in (1, B) or kp.shape[1] not in (1, Hk):
            return None
        cap = kp.shape[-1]
    else:
        if attn_mask.dim() != 4 or attn_mask.dtype != torch.bool:
            return None
        if attn_mask.shape[2] != 1 or attn_mask.shape[1] not in (1, Hk) or attn_mask.shape[0] not in (1, B):
            return None
        if attn_mask.shape[3] < Sk:
            return None
        kept = _cached_kept_keys(attn_mask, Sk)
        if kept is not None:
            cap = kept.key_pos.shape[-1]
        else:
            bound = int(attn_mask[..., :Sk].sum(dim=-1, dtype=torch.int32).max().item())
            cap = max(_KEY_PAD, round_multiple(bound, _KEY_PAD))
    return cap if 4 * cap <= 3 * round_multiple(Sk, _KEY_PAD) else None


def _cached_kept_keys(attn_mask, seqlen_k):
    """The position list `create_mask` computed together with this bool mask, if the mask is unchanged since."""
    if torch.compiler.is_compiling():  # Python attributes of tensors are not part of a traced graph
        return None
    tag = getattr(attn_mask, "_fdma_kept", None)
    if tag is not None and tag[1] == attn_mask._version and tag[0].seqlen_k == seqlen_k:
        return tag[0]
    return None


def _cached_packed_mask(attn_mask):
    """The bit-packed form `create_mask` wrote together with this per-query bool mask, if the mask is unchanged."""
    if torch.compiler.is_compiling() or not isinstance(attn_mask, torch.Tensor):
        return None
    tag = getattr(attn_mask, "_fdma_packed", None)
    if tag is not None and tag[1] == attn_mask._version and tuple(tag[0].shape) == tuple(attn_mask.shape):
        return tag[0]
    return None


def _raise_if_kernel_timed_out(lib) -> None:
    """A tcgen05 kernel whose bounded wait gave up leaves partly written results behind and a code in page-locked
    host memory. Checked (one host load, no GPU work) at the entry of every operator call, so that the failure
    surfaces at the next call at the latest instead of passing as valid data."""
    if lib.fdma_poll_kernel_status(None) != 0:
        detail = ctypes.c_int32(0)
        lib.fdma_last_kernel_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(detail))
        raise RuntimeError(
            f"an earlier attention kernel on this device gave up a bounded wait (code {detail.value}): "
            f"{lib.fdma_strerror(-6).decode()}; results of calls since then are not valid")


def _kernel_head_dim(d: int, needs_grad: bool) -> int:
    """Head dim the tensor-core kernels run this call at: the forward kernels exist for 64, 128 and 256, the backward
    kernels for 128 and 256. Other head dims are zero-padded up to the next of these (zero columns change neither the
    scores nor the kept columns of the results; the reference likewise runs every head dim on the next larger kernel,
    csrc/flash_sparse_attn/src/static_switch.h:60-82)."""
    if _kernel_path != _lib.PATH_AUTO:
        return d
    if needs_grad:
        return 128 if d <= 128 else (256 if d <= 256 else d)
    for target in (64, 128, 256):
        if d <= target:
            return target
    return d


def round_multiple(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def maybe_contiguous(x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.FDMA_BF16
    if t.dtype == torch.float16:
        return _lib.FDMA_FP16
    raise RuntimeError("FlashSparseAttention only supports fp16 and bf16 data type")


def _bsh(t: torch.Tensor) -> Tuple[int, int, int]:
    """(batch, row, head) element strides of a (B, S, H, d) tensor; size-1 dims get a dense stride."""
    sb, sr, sh, _ = t.stride()
    B, S, H, d = t.shape
    if H == 1:
        sh = d
    if S == 1:
        sr = H * d if sh == d else sr
    if B == 1:
        sb = max(sb, 1)
    return sb, sr, sh


def _mb_strides(t: Optional[torch.Tensor]) -> Tuple[int, int, int]:
    """(batch, head, row) strides of a 4-D mask/bias; broadcast (size-1 or expanded) dims give 0."""
    if t is None:
        return 0, 0, 0
    return tuple(0 if t.shape[i] == 1 else t.stride(i) for i in range(3))


def _check_inputs(q, k, v, mask, bias):
    if not q.is_cuda:
        raise RuntimeError("Input tensor must be on CUDA device")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("FlashSparseAttention only supports fp16 and bf16 data type")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError("query, key and value must have the same dtype")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("query, key and value must be (batch, seqlen, nheads, headdim)")
    B, Sq, H, d = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    if B <= 0:
        raise RuntimeError("batch size must be positive")
    if d > 256:
        raise RuntimeError("FlashSparseAttention forward only supports head dimension at most 256")
    if d % 8 != 0:
        raise RuntimeError("query, key, value, and out_ must have a head_size that is a multiple of 8")
    if H % Hk != 0:
        raise RuntimeError("Number of heads in key/value must divide number of heads in query")
    if k.shape != (B, Sk, Hk, d) or v.shape != (B, Sk, Hk, d):
        raise RuntimeError("key/value shape mismatch")
    Sk_r = round_multiple(Sk, _KEY_PAD)
    for name, t in (("mask", mask), ("bias", bias)):
        if t is None:
            continue
        if t.dim() != 4:
            raise RuntimeError(f"{name} must have 4 dimensions")
        if t.device != q.device:
            raise RuntimeError(f"{name} must be on the same device as query")
        if t.shape[0] not in (1, B):
            raise RuntimeError(f"{name} batch dimension must be 1 or batch_size")
        if t.shape[1] not in (1, Hk, H):
            raise RuntimeError(f"{name} head dimension must be 1, num_heads_k or num_heads")
        if t.shape[2] not in (1, Sq):
            raise RuntimeError(f"{name} query-length dimension must be 1 or seqlen_q")
        if t.shape[3] != Sk_r:
            raise RuntimeError(f"{name} key dimension must be seqlen_k rounded up to a multiple of {_KEY_PAD}")
    if mask is not None and mask.dtype != torch.bool:
        raise RuntimeError("mask must have dtype bool")
    if bias is not None and bias.dtype != q.dtype:
        raise RuntimeError("bias must have the same dtype as inputs")


def _fill_fwd(p: "_lib.FwdParams", q, k, v, mask, bias, out, lse, softmax_scale, is_causal):
    B, Sq, H, d = q.shape
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.mask = mask.data_ptr() if mask is not None else None
    p.bias = bias.data_ptr() if bias is not None else None
    p.out, p.lse = out.data_ptr(), lse.data_ptr()
    p.q_batch_stride, p.q_row_stride, p.q_head_stride = _bsh(q)
    p.k_batch_stride, p.k_row_stride, p.k_head_stride = _bsh(k)
    p.v_batch_stride, p.v_row_stride, p.v_head_stride = _bsh(v)
    p.o_batch_stride, p.o_row_stride, p.o_head_stride = _bsh(out)
    p.mask_batch_stride, p.mask_head_stride, p.mask_row_stride = _mb_strides(mask)
    p.bias_batch_stride, p.bias_head_stride, p.bias_row_stride = _mb_strides(bias)
    p.b, p.seqlen_q, p.seqlen_k, p.h, p.h_k, p.d = B, Sq, k.shape[1], H, k.shape[2], d
    p.h_mask = mask.shape[1] if mask is not None else 1
    p.h_bias = bias.shape[1] if bias is not None else 1
    p.dtype = _dtype_code(q)
    p.is_causal = 1 if is_causal else 0
    p.softmax_scale = float(softmax_scale)
    p.path = _kernel_path
    p.workspace, p.workspace_bytes = None, 0


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


@torch.library.custom_op("flash_sparse_attn::_flash_sparse_attn_forward", mutates_args=(), device_types="cuda")
def _flash_sparse_attn_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: Optional[torch.Tensor],
    bias: Optional[torch.Tensor],
    softmax_scale: float,
    is_causal: bool,
    softcap: float,
    return_softmax: bool,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    if softcap != 0.0:
        raise NotImplementedError("softcap > 0 is not built into the B200 kernels")
    # return_softmax: the caller gets softmax_lse; the probability matrix itself is never materialised (third result
    # stays empty), which the reference only offers for testing (interface.py:672-676)
    q, k, v, mask, bias = [maybe_contiguous(x) for x in (q, k, v, mask, bias)]
    _check_inputs(q, k, v, mask, bias)
    lib = _lib.load()
    B, Sq, H, d = q.shape
    with torch.cuda.device(q.device):
        _raise_if_kernel_timed_out(lib)
        out = torch.empty_like(q)
        lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
        p = _lib.FwdParams()
        _fill_fwd(p, q, k, v, mask, bias, out, lse, softmax_scale, is_causal)
        ws_bytes = lib.fdma_fwd_workspace_bytes(ctypes.byref(p))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws_bytes
        _lib.check(lib.fdma_fwd(ctypes.byref(p), _stream_ptr(q.device)), "fdma_fwd")
    return out, lse, torch.empty((0,), dtype=q.dtype, device=q.device)


@torch.library.register_fake("flash_sparse_attn::_flash_sparse_attn_forward")
def _flash_sparse_attn_forward_fake(q, k, v, mask, bias, softmax_scale, is_causal, softcap, return_softmax):
    B, Sq, H, _ = q.shape
    out = torch.empty_like(q)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    return out, lse, torch.empty((0,), dtype=q.dtype, device=q.device)


@torch.library.custom_op(
    "flash_sparse_attn::_flash_sparse_attn_backward", mutates_args=("dq", "dk", "dv", "dbias"), device_types="cuda"
)
def _flash_sparse_attn_backward(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: Optional[torch.Tensor],
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    dq: Optional[torch.Tensor],
    dk: Optional[torch.Tensor],
    dv: Optional[torch.Tensor],
    dbias: Optional[torch.Tensor],
    softmax_scale: float,
    is_causal: bool,
    softcap: float,
    deterministic: bool,
) -> torch.Tensor:
    if softcap != 0.0:
        raise NotImplementedError("softcap > 0 is not built into the B200 kernels")
    if dq is None or dk is None or dv is None:
        raise RuntimeError("dq, dk and dv must be pre-allocated by the caller")
    dout, q, k, v, mask, bias, out = [maybe_contiguous(x) for x in (dout, q, k, v, mask, bias, out)]
    _check_inputs(q, k, v, mask, bias)
    if dout.shape != q.shape or out.shape != q.shape:
        raise RuntimeError("dout / out shape mismatch")
    if dbias is not None and bias is None:
        raise RuntimeError("dbias given without bias")
    lib = _lib.load()
    B, Sq, H, d = q.shape
    lse = softmax_lse.contiguous()
    with torch.cuda.device(q.device):
        _raise_if_kernel_timed_out(lib)
        bp = _lib.BwdParams()
        _fill_fwd(bp.f, q, k, v, mask, bias, out, lse, softmax_scale, is_causal)
        bp.dout = dout.data_ptr()
        bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride = _bsh(dout)
        bp.dq, bp.dk, bp.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        bp.dq_batch_stride, bp.dq_row_stride, bp.dq_head_stride = _bsh(dq)
        bp.dk_batch_stride, bp.dk_row_stride, bp.dk_head_stride = _bsh(dk)
        bp.dv_batch_stride, bp.dv_row_stride, bp.dv_head_stride = _bsh(dv)
        if dbias is not None:
            if dbias.stride(-1) != 1:
                raise RuntimeError("dbias must be contiguous in its key dimension")
            bp.dbias = dbias.data_ptr()
            bp.dbias_batch_stride, bp.dbias_head_stride, bp.dbias_row_stride = dbias.stride()[:3]
            bp.dbias_b, bp.dbias_h, bp.dbias_rows, bp.dbias_keys = dbias.shape
        else:
            bp.dbias = None
        bp.deterministic = 1 if deterministic else 0
        # D = rowsum(dOut o Out), the `softmax_d` the reference's mha_bwd returns (flash_api.cpp:952, :1049)
        softmax_d = torch.empty((B, H, round_multiple(Sq, 128)), dtype=torch.float32, device=q.device)
        bp.softmax_d = softmax_d.data_ptr()
        ws_bytes = lib.fdma_bwd_workspace_bytes(ctypes.byref(bp))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
        if ws is not None:
            bp.f.workspace, bp.f.workspace_bytes = ws.data_ptr(), ws_bytes
        _lib.check(lib.fdma_bwd(ctypes.byref(bp), _stream_ptr(q.device)), "fdma_bwd")
    return softmax_d


@torch.library.register_fake("flash_sparse_attn::_flash_sparse_attn_backward")
def _flash_sparse_attn_backward_fake(
    dout, q, k, v, mask, bias, out, softmax_lse, dq, dk, dv, dbias, softmax_scale, is_causal, softcap, deterministic
):
    B, Sq, H, _ = q.shape
    return torch.empty((B, H, round_multiple(Sq, 128)), dtype=torch.float32, device=q.device)


class FlashDMAttnFunc(torch.autograd.Function):
    """Autograd boundary; argument list and saved state follow the reference's FlashDMAttnFunc
    (flash_sparse_attn_interface.py:382-498)."""

    @staticmethod
    def forward(ctx, q, k, v, mask, bias, softmax_scale, is_causal, softcap, deterministic, return_softmax,
                is_grad_enabled=True):
        is_grad = is_grad_enabled and any(x.requires_grad for x in (q, k, v))
        softmax_scale = q.shape[-1] ** (-0.5) if softmax_scale is None else softmax_scale
        is_causal = False if is_causal is None else is_causal
        softcap = 0.0 if softcap is None else softcap
        deterministic = False if deterministic is None else deterministic
        return_softmax = False if return_softmax is None else return_softmax
        bias_keys_given = bias.shape[-1] if bias is not None else 0

        head_size_og = q.size(3)
        if head_size_og % 8 != 0:  # 16-bit rows are kept 16-byte aligned
            pad = 8 - head_size_og % 8
            q, k, v = (torch.nn.functional.pad(x, [0, pad]) for x in (q, k, v))
        keys_padded = round_multiple(k.shape[1], _KEY_PAD)

        def fit_keys(t):
            if t is None or t.shape[-1] == keys_padded:
                return t
            if t.shape[-1] == 1:
                return t.expand(*t.shape[:-1], keys_padded)
            return torch.nn.functional.pad(t, [0, keys_padded - t.shape[-1]])

        mask, bias = fit_keys(mask), fit_keys(bias)
        out_padded, softmax_lse, s_dmask = torch.ops.flash_sparse_attn._flash_sparse_attn_forward(
            q, k, v, mask, bias, softmax_scale, is_causal, softcap, return_softmax
        )
        if is_grad:
            ctx.save_for_backward(q, k, v, mask, bias, out_padded, softmax_lse)
            ctx.softmax_scale = softmax_scale
            ctx.is_causal = is_causal
            ctx.softcap = softcap
            ctx.deterministic = deterministic
            ctx.bias_keys_given = bias_keys_given
        out = out_padded[..., :head_size_og]
        return out if not return_softmax else (out, softmax_lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args: Any):
        q, k, v, mask, bias, out, softmax_lse = ctx.saved_tensors
        # the kernels overwrite every gradient element, so no zero fill is needed
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dbias = None
        if bias is not None:
            dbias = torch.empty(bias.shape, dtype=bias.dtype, device=bias.device)
        head_size_og = dout.size(3)
        dout_padded = dout
        if head_size_og % 8 != 0:
            dout_padded = torch.nn.functional.pad(dout, [0, 8 - head_size_og % 8])
        torch.ops.flash_sparse_attn._flash_sparse_attn_backward(
            dout_padded, q, k, v, mask, bias, out, softmax_lse, dq, dk, dv, dbias,
            ctx.softmax_scale, ctx.is_causal, ctx.softcap, ctx.deterministic,
        )
        dq, dk, dv = dq[..., :head_size_og], dk[..., :head_size_og], dv[..., :head_size_og]
        if dbias is not None:
            dbias = dbias[..., : k.shape[1]]
            if ctx.bias_keys_given == 1:
                dbias = dbias.sum(dim=-1, keepdim=True)
        return dq, dk, dv, None, dbias, None, None, None, None, None, None


def flash_sparse_attn_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask: Optional[torch.Tensor] = None,
    attn_bias: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    is_causal: Optional[bool] = None,
    softcap: Optional[float] = None,
    deterministic: Optional[bool] = None,
    return_attn_probs: Optional[bool] = None,
):
    """Dynamic-mask attention, drop-in for the reference function of the same name
    (flash_sparse_attn/flash_sparse_attn_interface.py:610-684).

    query (B, Sq, H, d); key, value (B, Sk, Hk, d) with H % Hk == 0 (MQA/GQA); fp16 or bf16 on a B200.
    attn_mask: bool ({B|1}, {H|Hk|1}, {Sq|1}, {Sk|1}), False = masked out (or the `KeptKeys` position list of
    `utils.mask.create_kept_keys`, for a row-broadcast selection); attn_bias: same broadcast rules as the mask,
    dtype of query, added to the scaled scores before the softmax. is_causal aligns the causal mask to the
    bottom-right corner (key k visible to query q iff k <= q + Sk - Sq). Rows with no visible key return 0.
    softmax_scale defaults to d ** -0.5. softcap > 0 raises NotImplementedError. return_attn_probs=True returns
    (out, softmax_lse (B, H, Sq) fp32, empty tensor): the probability matrix is not materialised.
    Returns out (B, Sq, H, d); gradients flow to query, key, value and attn_bias.

    A row-broadcast mask (one keep-set per batch and kv head) is run over its gathered kept keys, which gives the
    same result in far fewer key tiles when the kept keys are scattered; `set_compaction("off")` disables that.
    """
    from .packed import PackedMask
    from .utils.mask import KeptKeys

    if isinstance(attn_mask, PackedMask):  # one bit per (query, key): utils.mask.create_packed_mask
        from .packed import flash_sparse_attn_packed_func

        if softcap or return_attn_probs:
            attn_mask = attn_mask.to_bool()
        else:
            return flash_sparse_attn_packed_func(query, key, value, attn_mask, attn_bias, softmax_scale, is_causal,
                                                 deterministic)
    cached = _cached_packed_mask(attn_mask)
    if cached is not None and not softcap and not return_attn_probs and query.dim() == 4:
        from .packed import _native, flash_sparse_attn_packed_func

        if _native(query, key, cached, attn_bias, True):
            return flash_sparse_attn_packed_func(query, key, value, cached, attn_bias, softmax_scale, is_causal,
                                                 deterministic)
    d = query.shape[-1]
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value))
    d_run = _kernel_head_dim(d, needs_grad) if query.dim() == 4 and not return_attn_probs else d
    if d_run != d:
        softmax_scale = d ** (-0.5) if softmax_scale is None else softmax_scale
        query, key, value = (torch.nn.functional.pad(t, [0, d_run - d]) for t in (query, key, value))
        out = flash_sparse_attn_func(query, key, value, attn_mask, attn_bias, softmax_scale, is_causal, softcap,
                                     deterministic, return_attn_probs)
        return out[..., :d]
    cap = _compaction_capacity(query, key, attn_mask, attn_bias, softcap, return_attn_probs)
    if cap is not None:
        from .compaction import flash_sparse_attn_compact_func

        kept = attn_mask if isinstance(attn_mask, KeptKeys) else _cached_kept_keys(attn_mask, key.shape[1])
        return flash_sparse_attn_compact_func(query, key, value, kept if kept is not None else attn_mask, attn_bias,
                                              softmax_scale, is_causal, cap, _trusted_capacity=True,
                                              deterministic=bool(deterministic))
    if isinstance(attn_mask, KeptKeys):  # a call the gathered route does not serve: back to a bool mask
        from .compaction import kept_keys_to_mask

        attn_mask = kept_keys_to_mask(attn_mask)
    return FlashDMAttnFunc.apply(
        query, key, value, attn_mask, attn_bias, softmax_scale, is_causal, softcap, deterministic,
        return_attn_probs, torch.is_grad_enabled(),
    )


def flash_sparse_attn_varlen_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    softmax_scale: Optional[float] = None,
    is_causal: Optional[bool] = None,
    softcap: Optional[float] = None,
    deterministic: Optional[bool] = None,
    return_attn_probs: Optional[bool] = None,
    block_table: Optional[torch.Tensor] = None,
):
    """Attention over packed variable-length sequences; same signature and result as the reference function of the
    same name (flash_sparse_attn/flash_sparse_attn_interface.py:687-790), which, like this one, takes no dynamic
    mask or bias.

    query (total_q, H, d); key, value (total_k, Hk, d); cu_seqlens_q / cu_seqlens_k (n + 1,) int32 cumulative lengths.
    Sequence i is rows cu_seqlens_q[i] : cu_seqlens_q[i+1] of query against rows cu_seqlens_k[i] : cu_seqlens_k[i+1]
    of key / value; is_causal aligns each sequence's causal mask to ITS bottom-right corner. Returns out
    (total_q, H, d), or with return_attn_probs=True (out, softmax_lse (H, total_q) fp32, empty tensor).

    Each sequence is a contiguous slice of the packed tensors, so it is handed to the dense kernels as a zero-copy
    (1, L, H, d) view: one forward (and backward) launch sequence per packed sequence, no padding, no mask. The
    boundaries are read on the host (one device synchronisation per call). A paged KV cache (`block_table`) is not
    built and raises NotImplementedError."""
    if block_table is not None:
        raise NotImplementedError("paged KV (block_table) is not built into the B200 kernels")
    if query.dim() != 3 or key.dim() != 3 or value.dim() != 3:
        raise RuntimeError("query, key and value must be (total_tokens, nheads, headdim)")
    if cu_seqlens_q.numel() != cu_seqlens_k.numel() or cu_seqlens_q.numel() < 2:
        raise RuntimeError("cu_seqlens_q and cu_seqlens_k must both have batch_size + 1 entries")
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    if cq[-1] > query.shape[0] or ck[-1] > key.shape[0]:
        raise RuntimeError("cu_seqlens exceed the number of packed tokens")
    H, d = query.shape[1], query.shape[2]
    outs, lses = [], []
    if cq[0] > 0:  # tokens before the first boundary belong to no sequence
        outs.append(query.new_zeros((cq[0], H, d)))
        lses.append(torch.full((H, cq[0]), float("inf"), dtype=torch.float32, device=query.device))
    for i in range(len(cq) - 1):
        lq, lk = cq[i + 1] - cq[i], ck[i + 1] - ck[i]
        if lq <= 0:
            continue
        if lq > max_seqlen_q or lk > max_seqlen_k:
            raise RuntimeError("a sequence is longer than max_seqlen_q / max_seqlen_k")
        q_i = query[cq[i]:cq[i + 1]].unsqueeze(0)
        if lk <= 0:  # no key at all: zero output, LSE = +inf (flash_api.cpp:532-539)
            outs.append((q_i * 0)[0])
            lses.append(torch.full((H, lq), float("inf"), dtype=torch.float32, device=query.device))
            continue
        res = flash_sparse_attn_func(q_i, key[ck[i]:ck[i + 1]].unsqueeze(0), value[ck[i]:ck[i + 1]].unsqueeze(0),
                                     None, None, softmax_scale, is_causal, softcap, deterministic, return_attn_probs)
        if return_attn_probs:
            outs.append(res[0][0])
            lses.append(res[1][0])
        else:
            outs.append(res[0])
    tail = query.shape[0] - cq[-1]
    if tail > 0:
        outs.append(query.new_zeros((tail, H, d)))
        lses.append(torch.full((H, tail), float("inf"), dtype=torch.float32, device=query.device))
    out = torch.cat(outs, dim=0) if outs else query.new_zeros(query.shape)
    if not return_attn_probs:
        return out
    return out, torch.cat(lses, dim=1), torch.empty((0,), dtype=query.dtype, device=query.device)
