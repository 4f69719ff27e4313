"""GPU parity of the key-compaction path (fdma_compact_index / fdma_gather_rows / fdma_scatter_rows and the
key-position causal test of fdma_fwd / fdma_bwd) against the fp32 oracle run on the FULL, uncompacted tensors,
and bit-exact checks of the index / gather / scatter kernels against torch indexing.

Tolerances as in test_gpu_attention.py (oracle.within_tolerance): max-abs <= 2e-2, mean-abs <= 2e-3; for dK / dV /
dBias the max bound grows by one ulp at the tensor's largest magnitude, the mean bound by 2 x the mean bf16
rounding floor."""
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


@pytest.fixture
def kernel_path():
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    yield iface.set_kernel_path
    iface.set_kernel_path("auto")


def scattered_mask(Bm, Hm, Sk, keep, seed):
    """Row-broadcast mask with `keep` kept keys per row at random positions (different per row)."""
    g = torch.Generator().manual_seed(seed)
    mask = torch.zeros(Bm, Hm, 1, Sk, dtype=torch.bool)
    for b in range(Bm):
        for h in range(Hm):
            idx = torch.randperm(Sk, generator=g)[: keep - (b + h) % 3]  # rows differ in their counts too
            mask[b, h, 0, idx] = True
    return mask


def test_index_gather_scatter_exact(dev):
    """Positions, gathered rows and scattered rows equal torch.nonzero / index_select / index_copy_ bit for bit."""
    from flash_sparse_attn.compaction import compact_keys
    from flash_sparse_attn import _lib
    import ctypes

    B, Sk, Hk, d, keep = 2, 5000, 2, 64, 300
    g = torch.Generator().manual_seed(5)
    k = torch.randn(B, Sk, Hk, d, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(B, Sk, Hk, d, generator=g).to(torch.bfloat16).to(dev)
    bias = torch.randn(B, 2 * Hk, 1, Sk, generator=g).to(torch.bfloat16).to(dev)
    mask = scattered_mask(B, Hk, Sk, keep, 7).to(dev)
    ck = compact_keys(k, v, mask, bias)
    cap = ck.key_pos.shape[-1]
    assert cap % 128 == 0 and cap >= keep
    for b in range(B):
        for h in range(Hk):
            idx = torch.nonzero(mask[b, h, 0]).flatten()
            n = idx.numel()
            assert int(ck.count[b, h]) == n
            assert torch.equal(ck.key_pos[b, h, :n].long(), idx)
            assert bool((ck.key_pos[b, h, n:] == 2**31 - 1).all())
            assert bool(ck.mask[b, h, 0, :n].all()) and not bool(ck.mask[b, h, 0, n:].any())
            assert torch.equal(ck.key[b, :n, h], k[b, idx, h]) and bool((ck.key[b, n:, h] == 0).all())
            assert torch.equal(ck.value[b, :n, h], v[b, idx, h])
            for hb in (2 * h, 2 * h + 1):  # bias heads map onto mask heads in groups
                assert torch.equal(ck.bias[b, hb, 0, :n], bias[b, hb, 0, idx])
    # scatter: the inverse, with zeros elsewhere
    lib = _lib.load()
    from flash_sparse_attn.compaction import _rows_call
    from flash_sparse_attn.flash_sparse_attn_interface import _bsh

    back = torch.full_like(k, 7.0)
    _rows_call(lib.fdma_scatter_rows, ck.key, back, ck.key_pos, B, Hk, Sk, cap, d, _bsh(ck.key), _bsh(back), dev)
    torch.cuda.synchronize()
    want = torch.where(mask[:, :, 0].permute(0, 2, 1)[..., None], k, torch.zeros_like(k))
    assert torch.equal(back, want)
    # a capacity smaller than the fullest row is refused
    with pytest.raises(RuntimeError):
        compact_keys(k, v, mask, None, capacity=128)


# (B, Sq, Sk, H, Hk, d), mask (Bm is B or 1, Hm is Hk or 1), bias heads (0 none, else 1 | Hk | H), keep, causal, path
CASES = [
    ((1, 256, 256, 2, 1, 64), (1, 1), 1, 100, True, "auto"),
    ((2, 384, 1024, 4, 2, 128), (2, 2), 2, 200, True, "auto"),
    ((2, 384, 1024, 4, 2, 128), (1, 2), 4, 200, True, "auto"),     # batch-broadcast mask, per-query-head bias
    ((1, 512, 1536, 4, 2, 128), (1, 1), 1, 300, True, "auto"),     # one mask row for all heads, Sq < Sk
    ((1, 640, 640, 8, 2, 128), (1, 2), 0, 150, True, "auto"),      # no bias
    ((1, 640, 640, 8, 2, 128), (1, 2), 2, 150, False, "auto"),     # non-causal: positions are ignored
    ((2, 200, 333, 4, 2, 32), (2, 2), 2, 77, True, "auto"),        # ragged sizes on the CUDA-core kernels
    ((1, 384, 1024, 4, 2, 128), (1, 2), 2, 200, True, "simt"),
    ((1, 700, 300, 2, 2, 128), (1, 2), 2, 120, True, "auto"),      # Sq > Sk: leading rows see nothing
    ((1, 1, 900, 8, 2, 128), (1, 2), 2, 100, True, "auto"),        # single query (decode)
]


@pytest.mark.parametrize("geom,mshape,hb,keep,causal,path", CASES)
def test_compact_vs_oracle(dev, kernel_path, geom, mshape, hb, keep, causal, path):
    from flash_sparse_attn import flash_sparse_attn_compact_func

    B, Sq, Sk, H, Hk, d = geom
    dtype = torch.bfloat16
    Bm = B if mshape[0] > 1 else 1
    Hm = mshape[1] if mshape[1] <= Hk else Hk
    bshape = None if hb == 0 else (B, {1: 1, 2: Hk, 4: H}[hb], 1, Sk)
    q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, bshape, seed=11, dtype=dtype)
    mask = scattered_mask(Bm, Hm, Sk, keep, 3)
    ref = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, causal)
    kernel_path(path)
    ql, kl, vl = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    bl = bias.to(dev).requires_grad_(True) if bias is not None else None
    out = flash_sparse_attn_compact_func(ql, kl, vl, mask.to(dev), bl, is_causal=causal)
    out.backward(dout.to(dev))
    torch.cuda.synchronize()
    _kernel_status_ok()
    check("out", out.detach().cpu(), ref[0], dtype)
    check("dq", ql.grad.cpu(), ref[2], dtype)
    check("dk", kl.grad.cpu(), ref[3], dtype, reduced=True)
    check("dv", vl.grad.cpu(), ref[4], dtype, reduced=True)
    if bias is not None:
        assert bl.grad.shape == bias.shape
        check("dbias", bl.grad.cpu(), ref[5], dtype, reduced=True)
    # dK / dV of dropped keys are exactly zero
    dropped = ~mask[:, :, 0].expand(B, Hm, Sk)
    if Hm == Hk:
        assert bool((kl.grad.cpu().permute(0, 2, 1, 3)[dropped] == 0).all())


def test_compact_matches_tile_path_full_window(dev):
    """With the configuration-3 mask shape (top-k of a bias row) at S = 4096, the compacted result agrees with the
    tile-skipping result of flash_sparse_attn_func within the same tolerances (both against the oracle's value)."""
    from flash_sparse_attn import flash_sparse_attn_compact_func, flash_sparse_attn_func
    from flash_sparse_attn.utils.mask import create_mask

    B, S, H, Hk, d, W = 1, 4096, 8, 2, 128, 512
    dtype = torch.bfloat16
    q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, 1, S), seed=2, dtype=dtype)
    q, k, v, bias, dout = (t.to(dev) for t in (q, k, v, bias, dout))
    mask = create_mask(bias, None, B, S, S, W, torch.finfo(dtype).min)
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    iface.set_compaction("off")
    try:
        a = flash_sparse_attn_func(q, k, v, mask, bias, is_causal=True)
    finally:
        iface.set_compaction("auto")
    b = flash_sparse_attn_compact_func(q, k, v, mask, bias, is_causal=True, capacity=W)
    torch.cuda.synchronize()
    _kernel_status_ok()
    assert (a.float() - b.float()).abs().max().item() <= 2e-2


def test_default_route_selection(dev):
    """flash_sparse_attn_func picks the gathered-keys route from the mask's shape: the position list left by
    create_mask sizes and feeds the gather without a read-back, an in-place edit of the mask voids it (counts are read back
    instead), a mostly-kept mask and a per-query mask stay on the full-range route."""
    from flash_sparse_attn import flash_sparse_attn_func
    from flash_sparse_attn import flash_sparse_attn_interface as iface
    from flash_sparse_attn.utils.mask import create_mask

    B, S, H, Hk, d, W = 1, 1024, 4, 2, 128, 256
    dtype = torch.bfloat16
    q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, 1, S), seed=4, dtype=dtype)
    qd, kd, vd, bd = (t.to(dev) for t in (q, k, v, bias))
    mask = create_mask(bd, None, B, S, S, W, torch.finfo(dtype).min)
    kept, version = mask._fdma_kept
    assert version == mask._version and kept.seqlen_k == S and kept.key_pos.shape == (B, Hk, 256)
    for h in range(Hk):  # the cached positions are the mask's kept keys
        assert torch.equal(kept.key_pos[0, h, :W].long(), torch.nonzero(mask[0, h, 0]).flatten())
    assert iface._compaction_capacity(qd, kd, mask, bd, None, None) == 256
    ref = oracle.attention_forward(q, k, v, mask.cpu(), bias, None, True)[0]
    check("out", flash_sparse_attn_func(qd, kd, vd, mask, bd, is_causal=True).cpu(), ref, dtype)

    # in-place edit: 100 more keys kept than the stale bound says
    extra = torch.zeros_like(mask)
    extra[..., :400] = True
    mask.logical_or_(extra)
    kept = int(mask.sum(-1).max())
    assert kept > W
    assert iface._compaction_capacity(qd, kd, mask, bd, None, None) == (kept + 127) // 128 * 128
    ref = oracle.attention_forward(q, k, v, mask.cpu(), bias, None, True)[0]
    check("out", flash_sparse_attn_func(qd, kd, vd, mask, bd, is_causal=True).cpu(), ref, dtype)

    dense = torch.ones(B, Hk, 1, S, dtype=torch.bool, device=dev)
    assert iface._compaction_capacity(qd, kd, dense, bd, None, None) is None
    perq = torch.ones(B, Hk, S, S, dtype=torch.bool, device=dev)
    assert iface._compaction_capacity(qd, kd, perq, bd, None, None) is None
    iface.set_compaction("off")
    try:
        assert iface._compaction_capacity(qd, kd, create_mask(bd, None, B, S, S, W, torch.finfo(dtype).min), bd,
                                          None, None) is None
    finally:
        iface.set_compaction("auto")
    torch.cuda.synchronize()
    _kernel_status_ok()
