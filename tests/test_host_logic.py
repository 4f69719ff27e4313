"""Host-side logic of the operator layer that needs no GPU: argument checks, stride handling, padding rules,
shape inference for torch.compile, and the 2-D padding-mask reshape of create_mask."""
import pytest
import torch

import flash_sparse_attn
from flash_sparse_attn import flash_sparse_attn_interface as iface
from flash_sparse_attn.utils import mask as mask_mod


def test_public_names_and_signature():
    import inspect

    sig = inspect.signature(flash_sparse_attn.flash_sparse_attn_func)
    assert list(sig.parameters) == [
        "query", "key", "value", "attn_mask", "attn_bias", "softmax_scale", "is_causal", "softcap",
        "deterministic", "return_attn_probs",
    ]
    assert all(p.default is None for n, p in sig.parameters.items() if n not in ("query", "key", "value"))
    sig = inspect.signature(mask_mod.create_mask)
    assert list(sig.parameters) == [
        "attention_bias", "attention_mask", "batch_size", "query_len", "key_len", "window_size", "min_dtype",
        "block_size", "type",
    ]
    assert sig.parameters["type"].default == "topk"
    assert hasattr(torch.ops.flash_sparse_attn, "_flash_sparse_attn_forward")
    assert hasattr(torch.ops.flash_sparse_attn, "_flash_sparse_attn_backward")


def test_cpu_tensors_are_rejected_loudly():
    q = torch.randn(1, 8, 2, 64, dtype=torch.bfloat16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        flash_sparse_attn.flash_sparse_attn_func(q, q, q)
    with pytest.raises(RuntimeError):
        mask_mod.create_mask(torch.randn(1, 1, 1, 16), None, 1, 1, 16, 4, -1e30)


def test_input_checks():
    dev_q = torch.empty(2, 16, 4, 64, dtype=torch.bfloat16, device="meta")

    class FakeCuda:  # _check_inputs only looks at metadata; emulate is_cuda on meta tensors
        pass

    def chk(q, k, v, mask=None, bias=None):
        orig = torch.Tensor.is_cuda
        try:
            torch.Tensor.is_cuda = property(lambda self: True)
            iface._check_inputs(q, k, v, mask, bias)
        finally:
            torch.Tensor.is_cuda = orig

    k = torch.empty(2, 32, 2, 64, dtype=torch.bfloat16, device="meta")
    chk(dev_q, k, k)
    with pytest.raises(RuntimeError, match="divide"):
        chk(dev_q, torch.empty(2, 32, 3, 64, dtype=torch.bfloat16, device="meta"),
            torch.empty(2, 32, 3, 64, dtype=torch.bfloat16, device="meta"))
    with pytest.raises(RuntimeError, match="multiple of 8"):
        q2 = torch.empty(2, 16, 4, 60, dtype=torch.bfloat16, device="meta")
        k2 = torch.empty(2, 32, 2, 60, dtype=torch.bfloat16, device="meta")
        chk(q2, k2, k2)
    with pytest.raises(RuntimeError, match="fp16 and bf16"):
        chk(dev_q.float(), k.float(), k.float())
    with pytest.raises(RuntimeError, match="bool"):
        chk(dev_q, k, k, mask=torch.empty(2, 2, 16, 128, dtype=torch.uint8, device="meta"))
    with pytest.raises(RuntimeError, match="key dimension"):
        chk(dev_q, k, k, mask=torch.empty(2, 2, 16, 32, dtype=torch.bool, device="meta"))
    with pytest.raises(RuntimeError, match="head dimension"):
        chk(dev_q, k, k, bias=torch.empty(2, 3, 16, 128, dtype=torch.bfloat16, device="meta"))
    with pytest.raises(RuntimeError, match="same dtype"):
        chk(dev_q, k, k, bias=torch.empty(2, 2, 16, 128, dtype=torch.float16, device="meta"))
    chk(dev_q, k, k, mask=torch.empty(1, 1, 1, 128, dtype=torch.bool, device="meta"),
        bias=torch.empty(2, 4, 16, 128, dtype=torch.bfloat16, device="meta"))


def test_stride_helpers():
    t = torch.empty(2, 16, 4, 64)
    assert iface._bsh(t) == (16 * 4 * 64, 4 * 64, 64)
    tt = torch.empty(2, 4, 16, 64).transpose(1, 2)  # (B,S,H,d) view of a (B,H,S,d) buffer
    assert iface._bsh(tt) == (4 * 16 * 64, 64, 16 * 64)
    m = torch.empty(2, 1, 1, 128, dtype=torch.bool)
    assert iface._mb_strides(m) == (128, 0, 0)
    e = torch.empty(1, 2, 1, 128).expand(3, 2, 16, 128)
    assert iface._mb_strides(e) == (0, 128, 0)
    assert iface._mb_strides(None) == (0, 0, 0)
    assert iface.round_multiple(129, 128) == 256 and iface.round_multiple(128, 128) == 128


def test_fake_kernels_infer_shapes():
    q = torch.empty(2, 16, 4, 64, dtype=torch.bfloat16, device="meta")
    k = torch.empty(2, 32, 2, 64, dtype=torch.bfloat16, device="meta")
    out, lse, p = torch.ops.flash_sparse_attn._flash_sparse_attn_forward(q, k, k, None, None, 0.125, True, 0.0, False)
    assert out.shape == q.shape and lse.shape == (2, 4, 16) and lse.dtype == torch.float32 and p.numel() == 0
    sd = torch.ops.flash_sparse_attn._flash_sparse_attn_backward(
        q, q, k, k, None, None, out, lse, torch.empty_like(q), torch.empty_like(k), torch.empty_like(k), None,
        0.125, True, 0.0, False)
    assert sd.shape == (2, 4, 128)


def test_create_mask_argument_errors():
    bias = torch.randn(2, 1, 1, 16)
    with pytest.raises(ValueError, match="not compatible"):
        mask_mod.create_mask(bias, torch.ones(2, 7, dtype=torch.bool), 2, 4, 16, 4, -1e30)
    with pytest.raises(ValueError, match="Unsupported mask type"):
        mask_mod.create_mask(bias, None, 2, 4, 16, 4, -1e30, type="sigmoid")
    with pytest.raises(ValueError, match="block_size"):
        mask_mod.create_mask(bias, None, 2, 4, 16, 4, -1e30, block_size=0)


def test_head_dim_routing_and_compaction_eligibility():
    """Which head dim a call runs at, and which mask shapes take the gathered-keys route (metadata only: the
    capacity comes from the position list create_mask leaves on its result, never from the device here)."""
    for d, fwd, bwd in ((32, 64, 128), (64, 64, 128), (72, 128, 128), (128, 128, 128), (136, 256, 256),
                        (256, 256, 256), (320, 320, 320)):
        assert iface._kernel_head_dim(d, False) == fwd and iface._kernel_head_dim(d, True) == bwd
    iface.set_kernel_path("simt")
    try:
        assert iface._kernel_head_dim(40, True) == 40  # a forced kernel family keeps the head dim
    finally:
        iface.set_kernel_path("auto")

    B, Sq, Sk, H, Hk, d = 2, 256, 4096, 8, 2, 128
    orig = torch.Tensor.is_cuda
    torch.Tensor.is_cuda = property(lambda self: True)
    try:
        q = torch.empty(B, Sq, H, d, dtype=torch.bfloat16, device="meta")
        k = torch.empty(B, Sk, Hk, d, dtype=torch.bfloat16, device="meta")
        bias = torch.empty(B, Hk, 1, Sk, dtype=torch.bfloat16, device="meta")

        from flash_sparse_attn.utils.mask import KeptKeys

        def tagged(shape, bound):
            """A bool mask carrying the position list create_mask computes with it (metadata only here)."""
            m = torch.empty(shape, dtype=torch.bool, device="meta")
            cap = max(128, (bound + 127) // 128 * 128)
            kept = KeptKeys(torch.empty(shape[:2] + (cap,), dtype=torch.int32, device="meta"),
                            torch.empty(shape[:2], dtype=torch.int32, device="meta"),
                            torch.empty(shape[:2] + (1, cap), dtype=torch.bool, device="meta"), shape[-1])
            m._fdma_kept = (kept, m._version)
            return m

        cap = lambda m, b=bias, **kw: iface._compaction_capacity(q, k, m, b, kw.get("softcap"), kw.get("probs"))
        assert cap(tagged((B, Hk, 1, Sk), 300)) == 384          # rounded up to whole 128-key tiles
        assert cap(tagged((1, 1, 1, Sk), 1)) == 128
        assert cap(tagged((B, Hk, 1, Sk), 3500)) is None        # more than 3/4 of the keys kept: tile skipping
        assert cap(tagged((B, Hk, Sq, Sk), 300)) is None        # per-query mask
        assert cap(tagged((B, H, 1, Sk), 300)) is None          # one row per QUERY head: K/V cannot be shared
        assert cap(tagged((B, Hk, 1, Sk), 300), torch.empty(B, Hk, Sq, Sk, dtype=torch.bfloat16, device="meta")) is None
        assert cap(tagged((B, Hk, 1, Sk), 300), None) == 384
        assert cap(tagged((B, Hk, 1, Sk), 300), probs=True) is None
        assert cap(None) is None
        # the position list itself in place of the mask
        assert cap(tagged((B, Hk, 1, Sk), 300)._fdma_kept[0]) == 384
        assert cap(tagged((B, Hk, 1, Sk), 3500)._fdma_kept[0]) is None
        assert cap(tagged((B, Hk, 1, Sk // 2), 300)._fdma_kept[0]) is None   # built for another key count
        q1 = torch.empty(B, 1, H, d, dtype=torch.bfloat16, device="meta")
        assert iface._compaction_capacity(q1, k, tagged((B, Hk, 1, Sk), 300), bias, None, None) is None  # decode
        iface.set_compaction("off")
        try:
            assert cap(tagged((B, Hk, 1, Sk), 300)) is None
        finally:
            iface.set_compaction("auto")
        with pytest.raises(ValueError):
            iface.set_compaction("sometimes")
    finally:
        torch.Tensor.is_cuda = orig


def test_packed_visibility_matches_brute_force():
    """Visibility of packed examples (HF glue): same example, and causal with each example's own bottom-right
    alignment (reference: the varlen call of modeling_flash_sparse_attention_utils.py:538-565)."""
    import torch
    from flash_sparse_attn.integrations.modeling_flash_sparse_attention_utils import _packed_visibility

    cu_q = torch.tensor([0, 3, 5, 9])
    cu_k = torch.tensor([0, 4, 9, 12])
    for causal in (False, True):
        got = _packed_visibility(cu_q, cu_k, 10, 13, causal, "cpu")   # one token past the last boundary on each side
        want = torch.zeros(10, 13, dtype=torch.bool)
        for s in range(3):
            lq, lk = int(cu_q[s + 1] - cu_q[s]), int(cu_k[s + 1] - cu_k[s])
            for i in range(lq):
                for j in range(lk):
                    if not causal or j <= i + lk - lq:
                        want[cu_q[s] + i, cu_k[s] + j] = True
        assert torch.equal(got, want)


def test_pack_mask_round_trip_and_tile_activity():
    """`pack_mask` / `PackedMask.to_bool` on CPU tensors: bit k & 31 of word k >> 5 is key k, rows hold
    round_up(Sk,128)/32 words with zero padding bits, one activity byte per 128 x 128 tile."""
    from flash_sparse_attn.packed import PackedMask, pack_mask

    g = torch.Generator().manual_seed(5)
    mask = torch.rand((2, 3, 200, 333), generator=g) < 0.2
    mask[:, :, :128, 128:256] = False          # an empty tile
    mask[0, 0, 5, 31] = True                   # the sign bit of a word
    packed = pack_mask(mask)
    assert isinstance(packed, PackedMask) and packed.shape == (2, 3, 200, 333)
    assert packed.bits.shape == (2, 3, 200, 12) and packed.bits.dtype == torch.int32
    assert packed.activity.shape == (2, 3, 2, 3) and packed.activity.dtype == torch.uint8
    assert torch.equal(packed.to_bool(), mask)
    assert (packed.bits[0, 0, 5, 0].item() >> 31) & 1 == 1
    assert packed.bits[..., 10].bitwise_and(~((1 << 13) - 1)).eq(0).all()   # keys 333..351 of word 10 stay zero
    assert packed.bits[..., 11].eq(0).all()
    assert packed.activity[:, :, 0, 1].eq(0).all() and packed.activity[:, :, 0, 0].ne(0).all()
    want = torch.nn.functional.pad(mask, [0, 51, 0, 56]).reshape(2, 3, 2, 128, 3, 128).any(dim=5).any(dim=3)
    assert torch.equal(packed.activity != 0, want)
