"""The HuggingFace-side caller (flash_sparse_attn.integrations) against the fp32 oracle: (B,H,S,d) layout in,
(B,S,H,d) out, mask built from the bias only when the key length exceeds the window, fp32 activations recast to the
module's half dtype. Tolerances: max-abs <= 2e-2, mean-abs <= 2e-3 (bf16 inputs, fp32 oracle)."""
import pytest
import torch

from oracle import oracle

from test_gpu_attention import check

pytestmark = pytest.mark.gpu


class _Attn(torch.nn.Module):
    is_causal = True
    layer_idx = 0

    def __init__(self, dtype):
        super().__init__()
        self.proj = torch.nn.Linear(8, 8).to(dtype)


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.mark.parametrize("window,fp32_in", [(128, False), (4096, False), (128, True)])
def test_forward_matches_oracle(dev, window, fp32_in):
    from flash_sparse_attn.integrations import flash_sparse_attention_forward

    B, S, H, Hk, d = 2, 512, 4, 2, 128
    dtype = torch.bfloat16
    q, k, v, bias, _ = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, 1, S), seed=9, dtype=dtype)
    want_mask = None
    if S > window:
        want_mask = oracle.create_mask(bias, None, B, S, S, window, torch.finfo(dtype).min)
    ref = oracle.attention_forward(q, k, v, want_mask, bias, d ** -0.5, True)[0]
    cast = (lambda t: t.float()) if fp32_in else (lambda t: t)
    module = _Attn(dtype).to(dev)
    out, none = flash_sparse_attention_forward(
        module, cast(q).to(dev).transpose(1, 2), cast(k).to(dev).transpose(1, 2), cast(v).to(dev).transpose(1, 2),
        None, cast(bias).to(dev), scaling=d ** -0.5, window_size=window)
    assert none is None and out.shape == (B, S, H, d) and out.dtype == dtype
    check("out", out.cpu(), ref, dtype)


def test_per_query_bias_through_the_caller(dev):
    """A bias with one row per query: the caller's `create_mask` leaves the bit-packed mask beside the bool tensor
    and the attention call reads it; result and the gradient of the bias against the oracle."""
    from flash_sparse_attn.integrations import flash_sparse_attention_forward

    B, S, H, Hk, d, window = 1, 384, 4, 2, 128, 96
    dtype = torch.bfloat16
    q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, S, S), seed=13, dtype=dtype)
    # values distinct within a row: the selection then has no ties and equals the oracle's
    g = torch.Generator().manual_seed(14)
    bias = (torch.argsort(torch.rand((B, Hk, S, S), generator=g), dim=-1).float() / S - 0.5).to(dtype)
    want_mask = oracle.create_mask(bias, None, B, S, S, window, torch.finfo(dtype).min)
    ref = oracle.attention_forward_backward(q, k, v, want_mask, bias, dout, d ** -0.5, True)
    module = _Attn(dtype).to(dev)
    ql = q.to(dev).transpose(1, 2).requires_grad_(True)
    bl = bias.to(dev).requires_grad_(True)
    out, _ = flash_sparse_attention_forward(module, ql, k.to(dev).transpose(1, 2), v.to(dev).transpose(1, 2), None, bl,
                                            scaling=d ** -0.5, window_size=window)
    out.backward(dout.to(dev))
    torch.cuda.synchronize()
    check("out", out.detach().cpu(), ref[0], dtype)
    check("dq", ql.grad.transpose(1, 2).cpu(), ref[2], dtype)
    check("dbias", bl.grad.cpu(), ref[5], dtype, reduced=True)


@pytest.mark.parametrize("side", ["right", "left"])
@pytest.mark.parametrize("lengths", [(256, 100, 37), (256, 256, 200)])
def test_padding_mask_matches_unpadded_attention(dev, side, lengths):
    """2-D padding mask: every example must equal plain causal attention over its own valid tokens (what the
    reference computes by un-padding, flash_sparse_attn/integrations/modeling_flash_sparse_attention_utils.py:511-536),
    padded rows zero; gradients of valid tokens likewise, of padded tokens zero."""
    from flash_sparse_attn.integrations import flash_sparse_attention_forward

    B, S, H, Hk, d = len(lengths), 256, 4, 2, 64
    dtype = torch.bfloat16
    q, k, v, _, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, 1, S), seed=21, dtype=dtype)
    pad = torch.zeros(B, S, dtype=torch.bool)
    for b, n in enumerate(lengths):
        if side == "right":
            pad[b, :n] = True
        else:
            pad[b, S - n:] = True
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    module = _Attn(dtype).to(dev)
    out, _ = flash_sparse_attention_forward(module, qd.transpose(1, 2), kd.transpose(1, 2), vd.transpose(1, 2),
                                            pad.to(dev), None, scaling=d ** -0.5)
    assert out.shape == (B, S, H, d)
    out.backward(dout.to(dev))
    for b, n in enumerate(lengths):
        sel = pad[b]
        r_out, _, r_dq, r_dk, r_dv, _ = oracle.attention_forward_backward(
            q[b:b + 1, sel], k[b:b + 1, sel], v[b:b + 1, sel], None, None, dout[b:b + 1, sel], d ** -0.5, True)
        check(f"out[{b}]", out[b:b + 1, sel.to(dev)].detach().cpu(), r_out, dtype)
        check(f"dq[{b}]", qd.grad[b:b + 1, sel.to(dev)].cpu(), r_dq, dtype)
        check(f"dk[{b}]", kd.grad[b:b + 1, sel.to(dev)].cpu(), r_dk, dtype)
        check(f"dv[{b}]", vd.grad[b:b + 1, sel.to(dev)].cpu(), r_dv, dtype)
        if n < S:
            assert out[b, ~sel.to(dev)].abs().max().item() == 0.0
            for g in (qd.grad, kd.grad, vd.grad):
                assert g[b, ~sel.to(dev)].abs().max().item() == 0.0


def test_padding_mask_single_query(dev):
    """Decode step with a padded cache: one query per example, keys limited to the example's valid ones."""
    from flash_sparse_attn.integrations import flash_sparse_attention_forward

    B, S, H, Hk, d = 2, 384, 4, 2, 128
    dtype = torch.bfloat16
    q, k, v, _, _ = oracle.make_inputs(B, 1, S, H, Hk, d, (B, Hk, 1, S), seed=22, dtype=dtype)
    pad = torch.ones(B, S, dtype=torch.bool)
    pad[1, :150] = False
    module = _Attn(dtype).to(dev)
    out, _ = flash_sparse_attention_forward(module, q.to(dev).transpose(1, 2), k.to(dev).transpose(1, 2),
                                            v.to(dev).transpose(1, 2), pad.to(dev), None, scaling=d ** -0.5)
    for b in range(B):
        sel = pad[b]
        ref = oracle.attention_forward(q[b:b + 1], k[b:b + 1, sel], v[b:b + 1, sel], None, None, d ** -0.5, False)[0]
        check(f"out[{b}]", out[b:b + 1].cpu(), ref, dtype)


@pytest.mark.parametrize("route", ["visibility-mask", "per-example"])
@pytest.mark.parametrize("how", ["position_ids", "cu_seqlens"])
def test_packed_sequences_match_per_example_attention(dev, how, route):
    """Packed examples in one row (reference: flash_sparse_attn/integrations/modeling_flash_sparse_attention_utils.py
    :538-565): each example must equal causal attention over its own tokens, values and gradients -- both through
    the one-launch visibility-mask route (small packs) and through flash_sparse_attn_varlen_func (large packs)."""
    from flash_sparse_attn.integrations import flash_sparse_attention_forward
    from flash_sparse_attn.integrations import modeling_flash_sparse_attention_utils as glue

    lens = (200, 180, 132)
    S, H, Hk, d = sum(lens), 4, 2, 64
    dtype = torch.bfloat16
    q, k, v, _, dout = oracle.make_inputs(1, S, S, H, Hk, d, (1, Hk, 1, S), seed=23, dtype=dtype)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    module = _Attn(dtype).to(dev)
    kw = {}
    if how == "position_ids":
        kw["position_ids"] = torch.cat([torch.arange(n) for n in lens])[None].to(dev)
    else:
        cu = torch.tensor([0, 200, 380, 512], dtype=torch.int32, device=dev)
        kw.update(cu_seq_lens_q=cu, cu_seq_lens_k=cu, max_length_q=200, max_length_k=200)
    limit = glue._PACKED_MASK_LIMIT
    if route == "per-example":
        glue._PACKED_MASK_LIMIT = 100
    try:
        out, _ = flash_sparse_attention_forward(module, qd.transpose(1, 2), kd.transpose(1, 2), vd.transpose(1, 2),
                                                None, None, scaling=d ** -0.5, **kw)
    finally:
        glue._PACKED_MASK_LIMIT = limit
    assert out.shape == (1, S, H, d)
    out.backward(dout.to(dev))
    lo = 0
    for n in lens:
        sl = slice(lo, lo + n)
        r_out, _, r_dq, r_dk, r_dv, _ = oracle.attention_forward_backward(
            q[:, sl], k[:, sl], v[:, sl], None, None, dout[:, sl], d ** -0.5, True)
        check(f"out[{lo}]", out[:, sl].detach().cpu(), r_out, dtype)
        check(f"dq[{lo}]", qd.grad[:, sl].cpu(), r_dq, dtype)
        check(f"dk[{lo}]", kd.grad[:, sl].cpu(), r_dk, dtype)
        check(f"dv[{lo}]", vd.grad[:, sl].cpu(), r_dv, dtype)
        lo += n


def test_unsupported_branches_raise(dev):
    from flash_sparse_attn.integrations import flash_sparse_attention_forward
    from flash_sparse_attn.integrations import modeling_flash_sparse_attention_utils as glue

    module = _Attn(torch.bfloat16).to(dev)
    q = torch.zeros(1, 2, 16, 64, device=dev, dtype=torch.bfloat16)
    pad = torch.ones(1, 16, dtype=torch.bool, device=dev)
    with pytest.raises(ValueError):
        flash_sparse_attention_forward(module, q, q, q, pad, torch.zeros(1, 2, 1, 16, device=dev, dtype=torch.bfloat16))
    from flash_sparse_attn import flash_sparse_attn_varlen_func

    cu = torch.tensor([0, 8, 16], dtype=torch.int32, device=dev)
    with pytest.raises(NotImplementedError):  # paged KV is not built
        flash_sparse_attn_varlen_func(q[0].transpose(0, 1), q[0].transpose(0, 1), q[0].transpose(0, 1), cu, cu, 8, 8,
                                      block_table=torch.zeros(2, 1, dtype=torch.int32, device=dev))


def test_varlen_func_ragged_lengths_vs_oracle(dev):
    """flash_sparse_attn_varlen_func (reference: flash_sparse_attn_interface.py:687-790): ragged query / key lengths
    per sequence (bottom-right causal alignment of each sequence's own lengths, a sequence without keys, one
    without queries), output, LSE and gradients against the oracle run per sequence."""
    from flash_sparse_attn import flash_sparse_attn_varlen_func

    lq = (130, 0, 64, 200)
    lk = (300, 50, 0, 200)
    H, Hk, d = 4, 2, 128
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(41)
    q = torch.randn(sum(lq), H, d, generator=g).to(dtype)
    k = torch.randn(sum(lk), Hk, d, generator=g).to(dtype)
    v = torch.randn(sum(lk), Hk, d, generator=g).to(dtype)
    dout = torch.randn(sum(lq), H, d, generator=g).to(dtype)
    cu_q = torch.tensor([0] + list(torch.tensor(lq).cumsum(0)), dtype=torch.int32, device=dev)
    cu_k = torch.tensor([0] + list(torch.tensor(lk).cumsum(0)), dtype=torch.int32, device=dev)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    out, lse, _ = flash_sparse_attn_varlen_func(qd, kd, vd, cu_q, cu_k, max(lq), max(lk), is_causal=True,
                                                return_attn_probs=True)
    assert out.shape == q.shape and lse.shape == (H, sum(lq))
    out.backward(dout.to(dev))
    oq = ok_ = 0
    for a, b in zip(lq, lk):
        sq, sk = slice(oq, oq + a), slice(ok_, ok_ + b)
        if a > 0 and b > 0:
            r = oracle.attention_forward_backward(q[None, sq], k[None, sk], v[None, sk], None, None, dout[None, sq],
                                                  None, True)
            check("out", out[sq].detach().cpu()[None], r[0], dtype)
            fin = torch.isfinite(r[1][0])
            assert (lse[:, sq].cpu()[fin] - r[1][0][fin]).abs().max() < 2e-3
            check("dq", qd.grad[sq].cpu()[None], r[2], dtype)
            check("dk", kd.grad[sk].cpu()[None], r[3], dtype, reduced=True)
            check("dv", vd.grad[sk].cpu()[None], r[4], dtype, reduced=True)
        elif a > 0:
            assert bool((out[sq] == 0).all()) and bool(torch.isposinf(lse[:, sq]).all())
            assert bool((qd.grad[sq] == 0).all())
        oq, ok_ = oq + a, ok_ + b
