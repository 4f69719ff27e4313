"""CPU oracle for dynamic-mask attention -- TEST INFRASTRUCTURE, not a product path.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this file;
the library under flash-dmattn_b200/ never does.

It restates, in fp32 eager PyTorch, the reference's own eager implementation:
  * attention forward/backward: benchmarks/backward_equivalence.py:118-133 (`dynamic_mask_attention_python`)
    and benchmarks/forward_equivalence.py:70-126 -- repeat_kv, QK^T*scale + bias, masked_fill(-inf), softmax, PV;
  * mask construction: flash_sparse_attn/utils/mask.py:76-120 (`topk_mask`), :123-159 (`relu_mask`),
    :47-73 (`block_smooth`), :163-240 (`create_mask`).
Two deliberate differences from the eager reference, both matching the reference's CUDA kernel contract:
  * rows with no visible key give probability 0 / output 0 / LSE +inf (csrc/flash_sparse_attn/src/softmax.h:211-214)
    where eager softmax gives NaN;
  * causal masking is bottom-right aligned, key k visible to query q iff k <= q + Sk - Sq (src/mask.h:39).

Pinning: tests/test_oracle_golden.py checks this file against tests/golden/*.npz, which
tests/golden/make_golden.py produced by importing and running the reference's Python code itself.
torch.topk leaves the choice among equal values at the selection threshold unspecified and the reference has no
test for it, so mask parity is "unpinned at ties": `create_mask` below breaks ties by ascending key index and
`masks_tie_equivalent` states what is compared when ties exist.
"""
import math
from typing import Optional, Tuple

import torch


# --------------------------------------------------------------------------------------------------------------
# create_mask
# --------------------------------------------------------------------------------------------------------------
def block_smooth(mask: torch.Tensor, key_len: int, block_size: int) -> torch.Tensor:
    """Majority vote per block of keys, tail block included (utils/mask.py:47-73)."""
    if block_size <= 0:
        raise ValueError(f"block_size must be a positive integer, got {block_size}.")
    if block_size == 1:
        return mask
    out = mask.clone()
    for start in range(0, key_len, block_size):
        blk = mask[..., start : start + block_size]
        keep = blk.sum(dim=-1, keepdim=True).to(torch.int64) * 2 > blk.shape[-1]
        out[..., start : start + block_size] = keep
    return out


def _reshape_2d_mask(attention_mask, batch_size, query_len, key_len):
    """2-D padding mask -> (B,1,1,Sk), left-padded with True (utils/mask.py:198-218)."""
    if attention_mask is None or attention_mask.dim() != 2:
        return attention_mask
    if attention_mask.shape[-1] == key_len:
        return attention_mask.view(batch_size, 1, 1, key_len)
    if attention_mask.shape[-1] == query_len:
        m = attention_mask.view(batch_size, 1, 1, query_len)
        pad = key_len - query_len
        if pad > 0:
            m = torch.cat([torch.ones((batch_size, 1, 1, pad), dtype=torch.bool, device=m.device), m], dim=-1)
        return m
    raise ValueError(
        f"attention_mask shape {attention_mask.shape} is not compatible with key_len {key_len} or query_len {query_len}."
    )


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
    """Restatement of utils/mask.py:163-240 with a DEFINED tie rule: among equal values at the selection
    threshold the lowest key indices win (stable descending sort instead of torch.topk(sorted=False))."""
    attention_mask = _reshape_2d_mask(attention_mask, batch_size, query_len, key_len)
    bias = attention_bias.detach()
    if attention_mask is not None:
        bias = bias.masked_fill(~attention_mask, min_dtype)
    if type == "topk":
        if window_size > bias.shape[-1]:
            raise RuntimeError("selected index k out of range")
        # stable sort, descending: equal values keep ascending index order
        values, order = torch.sort(bias.float(), dim=-1, descending=True, stable=True)
        top_idx = order[..., :window_size]
        top_val = values[..., :window_size]
        min_as_stored = torch.tensor(min_dtype, dtype=attention_bias.dtype).float()
        mask = torch.zeros_like(bias, dtype=torch.bool).scatter_(-1, top_idx, top_val != min_as_stored)
    elif type == "relu":
        mask = bias > 0
    else:
        raise ValueError(f"Unsupported mask type: {type}. Supported types are 'topk' and 'relu'.")
    if block_size is not None and block_size > 1:
        mask = block_smooth(mask, mask.shape[-1], block_size)
    return mask


def masks_tie_equivalent(mask_a: torch.Tensor, mask_b: torch.Tensor, values: torch.Tensor) -> bool:
    """True iff two top-k masks differ at most in WHICH of the equal threshold values they picked:
    per row the same number of keys is selected, and every key where they differ carries the row's smallest
    selected value (the threshold). `values` are the (pre-masked) bias values broadcast to the mask shape."""
    if mask_a.shape != mask_b.shape:
        return False
    if (mask_a.sum(-1) != mask_b.sum(-1)).any():
        return False
    v = values.float().expand(mask_a.shape)
    inf = torch.full_like(v, float("inf"))
    thr_a = torch.where(mask_a, v, inf).amin(-1, keepdim=True)
    thr_b = torch.where(mask_b, v, inf).amin(-1, keepdim=True)
    diff = mask_a ^ mask_b
    ok = (~diff) | ((v == thr_a) & (v == thr_b))
    return bool(ok.all())


# --------------------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------------------
def _expand_heads(t: torch.Tensor, n_heads: int) -> torch.Tensor:
    """(B|1, h, Sq|1, Sk) -> head dim n_heads, heads repeated block-wise like repeat_kv
    (benchmarks/backward_equivalence.py:55-67)."""
    h = t.shape[1]
    if h == n_heads:
        return t
    return t.repeat_interleave(n_heads // h, dim=1)


def visible_mask(
    mask: Optional[torch.Tensor], B: int, H: int, Sq: int, Sk: int, is_causal: bool, device
) -> torch.Tensor:
    """bool (B,H,Sq,Sk): attn_mask AND bottom-right causal."""
    full = torch.ones((B, H, Sq, Sk), dtype=torch.bool, device=device)
    if mask is not None:
        m = _expand_heads(mask[..., :Sk], H)
        full = full & m
    if is_causal and Sq > 1:
        q_idx = torch.arange(Sq, device=device).view(Sq, 1)
        k_idx = torch.arange(Sk, device=device).view(1, Sk)
        full = full & (k_idx <= q_idx + (Sk - Sq))
    return full


def attention_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: Optional[torch.Tensor],
    bias: Optional[torch.Tensor],
    softmax_scale: Optional[float] = None,
    is_causal: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """q (B,Sq,H,d), k/v (B,Sk,Hk,d), mask bool / bias float ({B|1},{H|Hk|1},{Sq|1},>=Sk). fp32 math.
    Returns out (B,Sq,H,d) fp32 and lse (B,H,Sq) fp32 (+inf for rows without a visible key)."""
    B, Sq, H, d = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    qf = q.float().transpose(1, 2)                                  # (B,H,Sq,d)
    kf = _expand_heads(k.float().transpose(1, 2), H)                # repeat_kv
    vf = _expand_heads(v.float().transpose(1, 2), H)
    s = torch.matmul(qf, kf.transpose(-2, -1)) * scale
    if bias is not None:
        s = s + _expand_heads(bias[..., :Sk].float(), H)
    vis = visible_mask(mask, B, H, Sq, Sk, is_causal, q.device)
    s = s.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).unsqueeze(-1))
    p = torch.where(vis, p, torch.zeros_like(p))                   # safe softmax: empty rows -> 0
    out = torch.matmul(p, vf).transpose(1, 2).contiguous()
    lse = torch.where(torch.isneginf(lse), torch.full_like(lse, float("inf")), lse)
    return out, lse


def attention_forward_backward(q, k, v, mask, bias, dout, softmax_scale=None, is_causal=False):
    """Forward + autograd backward of `attention_forward` for loss = sum(out * dout).
    Returns out, lse, dq, dk, dv, dbias (dbias None when bias is None), all fp32, gradients shaped like the
    inputs (so broadcast dims of bias are summed, like flash_api.cpp:1027-1047 + interface.py:495-496)."""
    qf = q.detach().float().requires_grad_(True)
    kf = k.detach().float().requires_grad_(True)
    vf = v.detach().float().requires_grad_(True)
    bf = bias.detach().float().requires_grad_(True) if bias is not None else None
    out, lse = attention_forward(qf, kf, vf, mask, bf, softmax_scale, is_causal)
    (out * dout.float()).sum().backward()
    return (out.detach(), lse.detach(), qf.grad, kf.grad, vf.grad, bf.grad if bf is not None else None)


# --------------------------------------------------------------------------------------------------------------
# seeded inputs shared by tests, smoke() and bench.py
# --------------------------------------------------------------------------------------------------------------
def make_inputs(B, Sq, Sk, H, Hk, d, bias_shape, seed=0, dtype=torch.float32, device="cpu", with_dout=True):
    """Q, K, V, bias, dOut ~ N(0,1), drawn in that order from one CPU generator (device independent), in fp32,
    then cast to `dtype`."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn((B, Sq, H, d), generator=g)
    k = torch.randn((B, Sk, Hk, d), generator=g)
    v = torch.randn((B, Sk, Hk, d), generator=g)
    bias = torch.randn(bias_shape, generator=g) if bias_shape is not None else None
    dout = torch.randn((B, Sq, H, d), generator=g) if with_dout else None
    cast = lambda t: None if t is None else t.to(dtype).to(device)
    return cast(q), cast(k), cast(v), cast(bias), cast(dout)


def error_report(name: str, got: torch.Tensor, ref: torch.Tensor, dtype=torch.bfloat16) -> dict:
    """max-abs / mean-abs error next to the floor that rounding the exact result to `dtype` alone produces (the
    measured floor over the tensor's elements, and `floor_bound` = half an ulp at the tensor's largest magnitude, the
    value the measured maximum approaches on large tensors), and the largest error in units of the last place,
    max |got - ref| / ulp_dtype(max(|ref|, 1)) (the ulp is taken at magnitude 1 for smaller references, where the
    absolute bounds are the binding ones)."""
    got, ref = got.float(), ref.float()
    err = (got - ref).abs()
    floor = (ref.to(dtype).float() - ref).abs()
    mant = {torch.bfloat16: 7, torch.float16: 10}.get(dtype, 23)
    ulp1 = torch.exp2(torch.floor(torch.log2(ref.abs().clamp(min=1.0))) - mant)
    ref_max = ref.abs().max().item() if ref.numel() else 0.0
    half_ulp_at_max = 0.5 * 2.0 ** (math.floor(math.log2(ref_max)) - mant) if ref_max > 0 and math.isfinite(ref_max) else 0.0
    return {
        "name": name,
        "max_abs": err.max().item() if err.numel() else 0.0,
        "mean_abs": err.mean().item() if err.numel() else 0.0,
        "floor_max_abs": floor.max().item() if floor.numel() else 0.0,
        "floor_mean_abs": floor.mean().item() if floor.numel() else 0.0,
        "floor_bound": half_ulp_at_max,
        "ulp_norm": (err / ulp1).max().item() if err.numel() else 0.0,
        "ref_max": ref_max,
    }


# Bounds of the parity tests: max-abs <= 2e-2 and mean-abs <= 2e-3 against the fp32 result. dK, dV and dBias are sums
# over many queries whose exact value, rounded once to 16 bits, already misses those bounds; for them the allowance
# grows by 2 x the rounding floor of the exact result: max-abs <= 2e-2 + ONE ulp at the tensor's largest magnitude
# (2 x half an ulp), mean-abs <= 2e-3 + 2 x (mean rounding error of the exact values). The max bound uses the floor's
# supremum rather than the largest rounding error that happens to occur, which on small tensors is noise. Measured on
# a B200 over every case of the suite, max-abs / (half an ulp at the maximum) lies between 1.0 and 1.5 (1.48 for dK
# at S = 32768, |dK| up to 97), with two small tensors above: a (1,1,1,256) dBias of magnitude 40 at 1.37 and the
# (1,2,1,512) dBias of the smoke case at 2.2 (0.138 against a half-ulp of 0.0625: the kernel's fp32 sum sits 0.076
# from the oracle's -- D = rowsum(dO o O) is formed from the 16-bit O, as in the reference -- and then rounds away
# from it). Errors of the reduced gradients do not scale with the element (a small dK element is the cancelled sum of
# the same large terms), so a per-element ulp bound would be the wrong model.
MAX_ABS, MEAN_ABS, FLOOR_FACTOR = 2e-2, 2e-3, 2.0


def within_tolerance(report: dict, reduced: bool) -> Tuple[bool, str]:
    """Applies the bounds above to an `error_report`; returns (ok, message with every figure of the report)."""
    lim = MAX_ABS + (FLOOR_FACTOR * report["floor_bound"] if reduced else 0.0)
    mlim = MEAN_ABS + (FLOOR_FACTOR * report["floor_mean_abs"] if reduced else 0.0)
    ok = report["max_abs"] <= lim and report["mean_abs"] <= mlim
    msg = (f"{report['name']}: max-abs {report['max_abs']:.4g} (limit {lim:.4g}; measured floor "
           f"{report['floor_max_abs']:.3g}, half-ulp at max {report['floor_bound']:.3g}), "
           f"mean-abs {report['mean_abs']:.4g} (limit {mlim:.4g}, floor {report['floor_mean_abs']:.3g}), "
           f"max |err|/ulp {report['ulp_norm']:.2f}, max |ref| {report['ref_max']:.3g}")
    return ok, msg
