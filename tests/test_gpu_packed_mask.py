"""Bit-packed per-query masks: `create_packed_mask` against the oracle's bool mask (bit for bit, and the tile
activity), and attention forward + backward with a `PackedMask` in place of the bool mask against the fp32 oracle."""
import pytest
import torch

from oracle import oracle

from test_gpu_attention import check, _kernel_status_ok

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.mark.parametrize("shape,window,dtype,premask", [
    ((1, 2, 300, 1024), 128, torch.bfloat16, False),
    ((2, 1, 130, 2048), 300, torch.float16, True),
    ((1, 2, 64, 8192), 1024, torch.bfloat16, False),     # four chunks per thread
    ((1, 1, 257, 200), 50, torch.bfloat16, False),       # ragged key count (multiple of 8)
    ((1, 1, 33, 40000), 2048, torch.bfloat16, False),    # longer than the register kernel takes: packed from the bool mask
    ((1, 2, 40, 512), 100, torch.float32, False),        # fp32 bias: packed from the bool mask
])
def test_packed_mask_equals_the_bool_mask(dev, shape, window, dtype, premask):
    from flash_sparse_attn.packed import pack_mask
    from flash_sparse_attn.utils.mask import create_packed_mask

    B, H, Sq, Sk = shape
    g = torch.Generator().manual_seed(3)
    # distinct values per row: ties at the threshold are not pinned by the reference
    bias = (torch.argsort(torch.rand(shape, generator=g), dim=-1).float() / Sk - 0.5).to(dtype)
    if dtype != torch.float32 and Sk > 2000:   # 16-bit types cannot hold that many distinct values: accept ties, compare counts below
        bias = torch.randn(shape, generator=g).to(dtype)
    pm = (torch.rand(shape, generator=g) < 0.8) if premask else None
    md = torch.finfo(dtype).min
    want = oracle.create_mask(bias, pm, B, Sq, Sk, window, md)
    got = create_packed_mask(bias.to(dev), None if pm is None else pm.to(dev), B, Sq, Sk, window, md)
    torch.cuda.synchronize()
    assert got.bits.shape == (B, H, Sq, (Sk + 127) // 128 * 4) and got.bits.dtype == torch.int32
    back = got.to_bool().cpu()
    if dtype != torch.float32 and Sk > 2000:
        from flash_sparse_attn.utils.mask import create_mask

        want = create_mask(bias.to(dev), None if pm is None else pm.to(dev), B, Sq, Sk, window, md).cpu()
    assert torch.equal(back, want)
    ref = pack_mask(want)
    assert torch.equal(got.bits.cpu(), ref.bits)
    assert torch.equal(got.activity.cpu() != 0, ref.activity != 0)


@pytest.mark.parametrize("geom,bias_shape,causal,dtype", [
    ((1, 256, 384, 4, 2, 128), "kv", True, torch.bfloat16),
    ((1, 300, 420, 4, 4, 128), "q", True, torch.bfloat16),       # one mask row per query head, ragged
    ((2, 384, 512, 2, 1, 128), "kv", False, torch.float16),
    ((1, 256, 256, 4, 2, 128), None, True, torch.bfloat16),      # mask only
    ((1, 200, 264, 2, 1, 64), "kv", True, torch.bfloat16),       # head dim 64: expanded to the bool mask
])
def test_attention_with_a_packed_mask(dev, geom, bias_shape, causal, dtype):
    from flash_sparse_attn import flash_sparse_attn_func
    from flash_sparse_attn.packed import pack_mask
    from flash_sparse_attn.utils.mask import create_packed_mask

    B, Sq, Sk, H, Hk, d = geom
    hm = {"kv": Hk, "q": H, None: Hk}[bias_shape]
    q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, None if bias_shape is None else (B, hm, Sq, Sk),
                                             seed=21, dtype=dtype)
    g = torch.Generator().manual_seed(22)
    if bias is not None:
        mask = oracle.create_mask(bias, None, B, Sq, Sk, max(8, Sk // 4), torch.finfo(dtype).min)
    else:
        mask = torch.rand((B, hm, Sq, Sk), generator=g) < 0.3
    ref = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, causal)
    ql, kl, vl = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    bl = bias.to(dev).requires_grad_(True) if bias is not None else None
    if bias is not None and Sk % 8 == 0:
        packed = create_packed_mask(bl.detach(), None, B, Sq, Sk, max(8, Sk // 4), torch.finfo(dtype).min)
        assert torch.equal(packed.to_bool().cpu(), mask)
    else:
        packed = pack_mask(mask.to(dev))
    out = flash_sparse_attn_func(ql, kl, vl, attn_mask=packed, attn_bias=bl, is_causal=causal)
    out.backward(dout.to(dev))
    torch.cuda.synchronize()
    _kernel_status_ok()
    check("out", out.detach().cpu(), ref[0], dtype)
    check("dq", ql.grad.cpu(), ref[2], dtype)
    check("dk", kl.grad.cpu(), ref[3], dtype, reduced=True)
    check("dv", vl.grad.cpu(), ref[4], dtype, reduced=True)
    if bl is not None:
        check("dbias", bl.grad.cpu(), ref[5], dtype, reduced=True)


def test_create_mask_leaves_the_packed_form_on_a_per_query_mask(dev):
    """`create_mask` on a per-query bias returns the reference's bool tensor and caches the bit-packed form on it;
    `flash_sparse_attn_func` then reads the bits (checked through the result against the oracle), an in-place edit of
    the mask voids the cache, and a row-broadcast mask gets the position list instead."""
    from flash_sparse_attn import flash_sparse_attn_func
    from flash_sparse_attn import flash_sparse_attn_interface as iface
    from flash_sparse_attn.utils.mask import create_mask

    B, Sq, Sk, H, Hk, d = 1, 256, 384, 4, 2, 128
    q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, (B, Hk, Sq, Sk), seed=31, dtype=torch.bfloat16)
    md = torch.finfo(torch.bfloat16).min
    want_mask = oracle.create_mask(bias, None, B, Sq, Sk, 96, md)
    mask = create_mask(bias.to(dev), None, B, Sq, Sk, 96, md)
    assert mask.dtype == torch.bool and torch.equal(mask.cpu(), want_mask)
    cached = iface._cached_packed_mask(mask)
    assert cached is not None and torch.equal(cached.to_bool(), mask)
    ref = oracle.attention_forward_backward(q, k, v, want_mask, bias, dout, None, True)
    ql, kl, vl, bl = (t.to(dev).requires_grad_(True) for t in (q, k, v, bias))
    out = flash_sparse_attn_func(ql, kl, vl, attn_mask=mask, attn_bias=bl, is_causal=True)
    out.backward(dout.to(dev))
    torch.cuda.synchronize()
    _kernel_status_ok()
    check("out", out.detach().cpu(), ref[0], torch.bfloat16)
    check("dq", ql.grad.cpu(), ref[2], torch.bfloat16)
    check("dbias", bl.grad.cpu(), ref[5], torch.bfloat16, reduced=True)
    # an edited mask must be read as it is now
    mask[0, 0, 10, :] = False
    assert iface._cached_packed_mask(mask) is None
    want_mask[0, 0, 10, :] = False
    ref2 = oracle.attention_forward_backward(q, k, v, want_mask, bias, dout, None, True)
    out2 = flash_sparse_attn_func(ql.detach(), kl.detach(), vl.detach(), attn_mask=mask, attn_bias=bl.detach(), is_causal=True)
    check("out", out2.cpu(), ref2[0], torch.bfloat16)
    # row-broadcast: position list, no packed form
    rb = create_mask(bias[:, :, :1].to(dev), None, B, Sq, Sk, 96, md)
    assert iface._cached_packed_mask(rb) is None and iface._cached_kept_keys(rb, Sk) is not None
