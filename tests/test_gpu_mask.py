"""GPU parity of create_mask (through fdma_create_mask) against the CPU oracle and the golden fixtures.
Integer/selection work: bit-exact is the bar. With equal values at the threshold the kernel's rule (lowest key
index first) is the oracle's rule, so even tie-heavy bf16 rows compare bit-exactly with the oracle; against
torch.topk, whose tie choice is unspecified, the comparison is tie-equivalence."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _cm(*a, **kw):
    from flash_sparse_attn.utils.mask import create_mask

    return create_mask(*a, **kw)


@pytest.mark.parametrize("name", ["mask_rowbcast", "mask_causal_premask", "mask_padding2d", "mask_block_smooth",
                                  "mask_relu"])
def test_golden_masks(dev, golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    window, _, block_size, is_relu = [int(x) for x in z["meta"]]
    bias = torch.from_numpy(z["bias"]).to(dev)
    pm = torch.from_numpy(z["premask"]).to(dev) if z["premask"].size else None
    B, _, Sq, Sk = bias.shape
    m = _cm(bias, pm, B, Sq, Sk, window, torch.finfo(torch.float32).min, block_size=block_size or None,
            type="relu" if is_relu else "topk")
    assert m.dtype == torch.bool and m.shape == z["mask"].shape
    assert torch.equal(m.cpu(), torch.from_numpy(z["mask"]))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,window", [((2, 3, 1, 1000), 100), ((1, 2, 37, 640), 64), ((1, 1, 1, 4096), 4096),
                                          ((1, 1, 2, 70000), 1024), ((1, 1, 1, 8), 3)])
def test_topk_bit_exact_vs_oracle(dev, dtype, shape, window):
    g = torch.Generator().manual_seed(hash((shape, window)) % 1000)
    bias = torch.randn(shape, generator=g).to(dtype)
    want = oracle.create_mask(bias, None, shape[0], shape[2], shape[3], window, torch.finfo(dtype).min)
    got = _cm(bias.to(dev), None, shape[0], shape[2], shape[3], window, torch.finfo(dtype).min)
    assert torch.equal(got.cpu(), want)
    assert int(got.sum()) == window * shape[0] * shape[1] * shape[2]


def test_ties_vs_torch_topk_on_device(dev):
    # bf16 N(0,1) over 32768 keys, top-2048: ~30 equal values at the threshold
    g = torch.Generator().manual_seed(0)
    bias = torch.randn((2, 8, 1, 32768), generator=g).to(torch.bfloat16).to(dev)
    got = _cm(bias, None, 2, 1, 32768, 2048, torch.finfo(torch.bfloat16).min)
    idx = torch.topk(bias, 2048, dim=-1, largest=True, sorted=False).indices
    ref = torch.zeros_like(bias, dtype=torch.bool).scatter_(-1, idx, True)
    assert oracle.masks_tie_equivalent(got.cpu(), ref.cpu(), bias.cpu())
    want = oracle.create_mask(bias.cpu(), None, 2, 1, 32768, 2048, torch.finfo(torch.bfloat16).min)
    assert torch.equal(got.cpu(), want)


def test_premask_broadcast_min_dtype_and_degenerate_rows(dev):
    B, H, Sq, Sk, w = 2, 2, 48, 256, 32
    g = torch.Generator().manual_seed(3)
    bias = torch.randn((B, H, 1, Sk), generator=g).to(torch.bfloat16)
    causal = torch.tril(torch.ones(Sq, Sk, dtype=torch.bool), diagonal=Sk - Sq)[None, None]
    mn = torch.finfo(torch.bfloat16).min
    want = oracle.create_mask(bias, causal, B, Sq, Sk, w, mn)
    got = _cm(bias.to(dev), causal.to(dev), B, Sq, Sk, w, mn)
    assert got.shape == (B, H, Sq, Sk) and torch.equal(got.cpu(), want)
    # fewer visible keys than the window: only the visible ones may be set (values == min_dtype never are)
    pm = torch.zeros(B, 1, 1, Sk, dtype=torch.bool)
    pm[..., :5] = True
    got = _cm(bias.to(dev), pm.to(dev), B, 1, Sk, w, mn)
    assert torch.equal(got.cpu(), pm.expand(B, H, 1, Sk))
    # all-equal row: ties everywhere, lowest indices win
    flat = torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16)
    got = _cm(flat.to(dev), None, 1, 1, 64, 10, mn)
    assert got.cpu().view(-1).tolist() == [True] * 10 + [False] * 54
    with pytest.raises(RuntimeError, match="out of range"):
        _cm(flat.to(dev), None, 1, 1, 64, 65, mn)


def test_2d_padding_mask_and_block_smooth(dev):
    B, Sq, Sk, w = 2, 64, 200, 40
    g = torch.Generator().manual_seed(5)
    bias = torch.randn((B, 2, 1, Sk), generator=g)
    pad_k = torch.ones(B, Sk, dtype=torch.bool)
    pad_k[0, :50] = False
    pad_q = torch.ones(B, Sq, dtype=torch.bool)
    pad_q[1, :7] = False
    mn = torch.finfo(torch.float32).min
    for pm in (pad_k, pad_q):
        for bs in (None, 16, 64):
            want = oracle.create_mask(bias, pm, B, Sq, Sk, w, mn, block_size=bs)
            got = _cm(bias.to(dev), pm.to(dev), B, Sq, Sk, w, mn, block_size=bs)
            assert torch.equal(got.cpu(), want), (pm.shape, bs)


def test_full_size_rows_properties(dev):
    # rows of 8192 keys, top-1024, many rows: exact count per row and every selected
    # value >= every unselected value -- properties that need no CPU-side oracle at this size
    bias = torch.randn((1, 8, 2048, 8192), device=dev, dtype=torch.bfloat16)
    got = _cm(bias, None, 1, 2048, 8192, 1024, torch.finfo(torch.bfloat16).min)
    assert (got.sum(-1) == 1024).all()
    big = torch.finfo(torch.float32).max
    lo_sel = torch.where(got, bias.float(), torch.full_like(bias, big, dtype=torch.float32)).amin(-1)
    hi_unsel = torch.where(got, torch.full_like(bias, -big, dtype=torch.float32), bias.float()).amax(-1)
    assert (lo_sel >= hi_unsel).all()


def test_topk_indices_vs_torch(dev):
    """`topk_indices` (reference: utils/mask.py:20-44 = torch.topk(...).indices sorted) on tie-free fp32 rows, where
    the selection is unique: int64, ascending, equal to torch's."""
    from flash_sparse_attn.utils.mask import topk_indices

    g = torch.Generator().manual_seed(12)
    for shape, w in (((2, 3, 5000), 257), ((1, 2, 128), 128), ((1, 1, 40000), 1000)):
        n = shape[0] * shape[1] * shape[2]
        bias = ((torch.randperm(n, generator=g).float() - n / 2) * 1e-3).view(shape).to(dev)  # all values distinct
        assert bias.unique().numel() == bias.numel()
        got = topk_indices(bias, w)
        want = torch.topk(bias, w, dim=-1, largest=True, sorted=False).indices.sort(dim=-1).values
        assert got.dtype == torch.int64 and got.shape == shape[:2] + (w,)
        assert torch.equal(got, want)
    with pytest.raises(RuntimeError, match="out of range"):
        topk_indices(bias, 40001)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,window", [((2, 3, 1, 1000), 100), ((1, 8, 1, 32768), 2048), ((1, 1, 1, 70000), 1024),
                                          ((2, 2, 1, 4096), 4096), ((1, 2, 1, 8), 3)])
def test_positions_bit_exact_vs_oracle(dev, dtype, shape, window):
    """The position output of the selection kernel (fdma_mask_params::key_pos / count / slot_mask) equals
    torch.nonzero of the oracle's mask, also on the tie-heavy 16-bit rows; the bool mask written by the same launch
    is unchanged; positions-only mode (no bool mask) gives the same list."""
    from flash_sparse_attn.utils.mask import create_kept_keys, create_mask

    B, H, _, Sk = shape
    g = torch.Generator().manual_seed(hash((shape, window)) % 1000 + 1)
    bias = torch.randn(shape, generator=g).to(dtype)
    pm = torch.rand((B, 1, 1, Sk), generator=g) < 0.9   # a pre-mask that removes a tenth of the keys
    mn = torch.finfo(dtype).min
    for premask in (None, pm):
        want = oracle.create_mask(bias, premask, B, 1, Sk, window, mn)
        pmd = premask.to(dev) if premask is not None else None
        mask = create_mask(bias.to(dev), pmd, B, 1, Sk, window, mn)
        assert torch.equal(mask.cpu(), want)
        only = create_kept_keys(bias.to(dev), pmd, B, 1, Sk, window, mn)
        for kept in (mask._fdma_kept[0], only):
            cap = kept.key_pos.shape[-1]
            assert cap % 128 == 0 and cap >= min(window, Sk) and kept.seqlen_k == Sk
            assert kept.key_pos.shape == (B, H, cap) and kept.count.shape == (B, H)
            assert kept.slot_mask.shape == (B, H, 1, cap)
            for b in range(B):
                for h in range(H):
                    idx = torch.nonzero(want[b, h, 0]).flatten()
                    n = idx.numel()
                    assert int(kept.count[b, h]) == n
                    assert torch.equal(kept.key_pos[b, h, :n].cpu().long(), idx)
                    assert bool((kept.key_pos[b, h, n:] == 2**31 - 1).all())
                    assert bool(kept.slot_mask[b, h, 0, :n].all()) and not bool(kept.slot_mask[b, h, 0, n:].any())
