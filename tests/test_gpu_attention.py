"""GPU parity of fdma_fwd / fdma_bwd (through the Python operator API, which calls the C ABI) against the fp32
oracle on identical seeded inputs.

Tolerances (bf16/fp16 inputs, fp32 oracle): max-abs <= 2e-2 and mean-abs <= 2e-3. dK, dV and dBias are sums over
many queries and reach magnitudes where ONE bf16 rounding of the exact result already exceeds the bound
(`floor` = |ref - bf16(ref)|, the error of a perfect kernel that returns bf16); for those three the bounds are
max-abs <= 2e-2 + one ulp at the tensor's largest magnitude and mean-abs <= 2e-3 + 2 * floor_mean
(oracle.within_tolerance, with the measured ratios that back the factor). A failure
message carries every figure: max-abs, mean-abs, both floors and the largest error in ulps of the reference."""
import itertools

import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS = oracle.MAX_ABS, oracle.MEAN_ABS


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True, params=["off", "auto"], ids=["tiles", "compaction"])
def compaction_mode(request):
    """Every case runs twice: over the full key range with tile skipping, and with the library's default, which
    gathers the kept keys first when the mask is row-broadcast (cases with other mask shapes run the same code in
    both modes)."""
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    iface.set_compaction(request.param)
    yield request.param
    iface.set_compaction("auto")


@pytest.fixture
def kernel_path():
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    yield iface.set_kernel_path
    iface.set_kernel_path("auto")


def _kernel_status_ok():
    import ctypes
    from flash_sparse_attn import _lib

    detail = ctypes.c_int32(0)
    st = _lib.load().fdma_last_kernel_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(detail))
    assert st == 0, f"kernel wait timed out, code {detail.value}"


def build_case(dev, B, Sq, Sk, H, Hk, d, bias_kind, mask_kind, window, dtype, seed=0):
    """bias_kind: none | bcast (B,Hk,1,Sk) | perq (B,Hk,Sq,Sk) | perhead (B,H,Sq,Sk) | b1h1 (1,1,1,Sk)
    mask_kind: none | topk (create_mask on the bias, oracle version) | block (contiguous kept blocks, row-bcast,
    per kv head) | randq (random per-query mask, one head)."""
    shapes = {"none": None, "bcast": (B, Hk, 1, Sk), "perq": (B, Hk, Sq, Sk), "perhead": (B, H, Sq, Sk),
              "b1h1": (1, 1, 1, Sk)}
    q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, shapes[bias_kind], seed=seed, dtype=dtype)
    g = torch.Generator().manual_seed(seed + 100)
    if mask_kind == "none":
        mask = None
    elif mask_kind == "topk":
        src = bias if bias is not None else torch.randn((B, Hk, 1, Sk), generator=g).to(dtype)
        mask = oracle.create_mask(src, None, B, Sq, Sk, min(window, Sk), torch.finfo(dtype).min)
    elif mask_kind == "block":
        mask = torch.zeros(B, Hk, 1, Sk, dtype=torch.bool)
        for b, h in itertools.product(range(B), range(Hk)):
            start = int(torch.randint(0, max(1, Sk - window), (1,), generator=g))
            mask[b, h, 0, start : start + window] = True
    elif mask_kind == "randq":
        mask = torch.rand((B, 1, Sq, Sk), generator=g) < 0.3
    elif mask_kind == "randqh":  # per query head, with whole 128x128 tiles emptied for some heads
        mask = torch.rand((B, H, Sq, Sk), generator=g) < 0.3
        mask[:, ::2, : Sq // 2, Sk // 2 :] = False
    else:
        raise ValueError(mask_kind)
    to = lambda t: None if t is None else t.to(dev)
    return tuple(to(t) for t in (q, k, v, mask, bias, dout))


def run_ours(q, k, v, mask, bias, dout, is_causal, scale=None, want_grad=True):
    from flash_sparse_attn import flash_sparse_attn_func

    ql, kl, vl = (t.detach().clone().requires_grad_(want_grad) for t in (q, k, v))
    bl = bias.detach().clone().requires_grad_(want_grad) if bias is not None else None
    out = flash_sparse_attn_func(ql, kl, vl, attn_mask=mask, attn_bias=bl, is_causal=is_causal, softmax_scale=scale)
    if not want_grad:
        return out, None, None, None, None
    out.backward(dout)
    return out, ql.grad, kl.grad, vl.grad, (bl.grad if bl is not None else None)


def check(name, got, ref, dtype, reduced=False):
    r = oracle.error_report(name, got, ref, dtype)
    assert torch.isfinite(got.float()).all(), f"{name}: non-finite values"
    ok, msg = oracle.within_tolerance(r, reduced)
    assert ok, msg


def compare_all(case, is_causal, dtype, scale=None, fwd_only=False):
    q, k, v, mask, bias, dout = case
    ref = oracle.attention_forward_backward(q, k, v, mask, bias, dout, scale, is_causal)
    got = run_ours(q, k, v, mask, bias, dout, is_causal, scale, want_grad=not fwd_only)
    torch.cuda.synchronize()
    _kernel_status_ok()
    check("out", got[0], ref[0], dtype)
    if fwd_only:
        return
    check("dq", got[1], ref[2], dtype)
    check("dk", got[2], ref[3], dtype, reduced=True)
    check("dv", got[3], ref[4], dtype, reduced=True)
    if bias is not None:
        assert got[4].shape == bias.shape
        check("dbias", got[4], ref[5], dtype, reduced=True)


# geometry: (B, Sq, Sk, H, Hk, d)
SIMT_CASES = [
    ((1, 256, 256, 2, 1, 64), "bcast", "topk", 128, True),      # the small CPU-reference geometry (MQA, d=64, W=128)
    ((2, 100, 229, 4, 2, 32), "perq", "randq", 0, True),        # ragged, Sq < Sk, per-query everything
    ((1, 130, 130, 3, 3, 96), "perhead", "none", 0, False),     # MHA, per-head bias, odd head dim
    ((1, 64, 320, 2, 1, 256), "b1h1", "block", 96, True),       # d=256, fully broadcast bias
    ((2, 192, 64, 2, 2, 128), "none", "none", 0, True),         # Sq > Sk causal: leading rows see nothing
    ((1, 1, 700, 8, 2, 128), "bcast", "topk", 100, False),      # decode
    ((1, 80, 80, 2, 2, 40), "bcast", "topk", 16, True),         # head dim multiple of 8 only
]


@pytest.mark.parametrize("geom,bias_kind,mask_kind,window,causal", SIMT_CASES)
def test_simt_path(dev, kernel_path, geom, bias_kind, mask_kind, window, causal):
    kernel_path("simt")
    case = build_case(dev, *geom, bias_kind, mask_kind, window, torch.bfloat16)
    compare_all(case, causal, torch.bfloat16)


def test_head_dim_not_multiple_of_8_is_padded(dev, kernel_path):
    kernel_path("simt")
    case = build_case(dev, 1, 64, 64, 2, 1, 36, "bcast", "topk", 32, torch.bfloat16)
    compare_all(case, True, torch.bfloat16, scale=36 ** -0.5)


TC_CASES = [
    # row-broadcast bias + mask (production shape of the bias), causal and not, d = 64 / 128
    ((1, 256, 256, 2, 1, 64), "bcast", "topk", 128, True),
    ((1, 256, 256, 2, 1, 128), "bcast", "topk", 128, False),
    ((2, 512, 512, 4, 2, 128), "bcast", "topk", 200, True),
    ((1, 384, 640, 2, 2, 128), "bcast", "block", 128, True),    # Sq < Sk, whole key tiles skipped
    ((1, 300, 300, 2, 1, 128), "bcast", "topk", 77, True),      # ragged: 300 = 2*128 + 44
    ((1, 128, 1024, 4, 1, 64), "b1h1", "block", 256, False),    # MQA, fully broadcast, skipped tiles
    ((2, 640, 128, 2, 2, 128), "none", "none", 0, True),        # Sq > Sk: query tiles with no key tile at all
    ((1, 200, 520, 2, 1, 128), "none", "topk", 130, False),     # mask only
    ((1, 256, 384, 2, 2, 64), "bcast", "none", 0, True),        # bias only
    # per-query bias / mask
    ((1, 256, 256, 4, 2, 128), "perq", "randq", 0, True),
    ((2, 384, 384, 2, 1, 64), "perq", "none", 0, False),
    ((1, 300, 420, 4, 4, 128), "perhead", "randq", 0, True),
    ((1, 256, 512, 2, 1, 128), "bcast", "randq", 0, True),      # broadcast bias with per-query mask
    # head dim 256: one query tile per CTA, two-slot K/V ring
    ((1, 384, 640, 4, 1, 256), "bcast", "topk", 200, True),     # MQA with wide heads, Sq < Sk
    ((2, 300, 300, 2, 2, 256), "bcast", "block", 100, True),    # ragged, whole key tiles skipped
    ((1, 256, 1280, 2, 1, 256), "perq", "randq", 0, False),     # per-query bias and mask, 10 key tiles
    ((1, 640, 128, 2, 2, 256), "none", "none", 0, True),        # Sq > Sk
]


@pytest.mark.parametrize("geom,bias_kind,mask_kind,window,causal", TC_CASES)
def test_tcgen05_forward(dev, kernel_path, geom, bias_kind, mask_kind, window, causal):
    kernel_path("tcgen05")
    case = build_case(dev, *geom, bias_kind, mask_kind, window, torch.bfloat16)
    compare_all(case, causal, torch.bfloat16, fwd_only=True)


TC_BWD_CASES = [
    ((1, 256, 256, 2, 1, 128), "bcast", "topk", 128, True),     # column-sum dBias over a head group
    ((2, 512, 512, 4, 2, 128), "bcast", "topk", 200, True),
    ((1, 384, 640, 2, 2, 128), "bcast", "block", 128, True),    # key tiles without any kept key
    ((1, 300, 300, 2, 1, 128), "bcast", "topk", 77, True),      # ragged
    ((2, 640, 128, 2, 2, 128), "none", "none", 0, True),        # Sq > Sk
    ((1, 200, 520, 2, 1, 128), "none", "topk", 130, False),     # mask only, no dBias
    ((1, 256, 256, 4, 2, 128), "perq", "randq", 0, True),       # per-query dBias summed over the head group
    ((1, 300, 420, 4, 4, 128), "perhead", "randq", 0, True),    # per-head per-query dBias
    ((1, 256, 512, 2, 1, 128), "bcast", "randq", 0, True),      # broadcast bias, per-query mask
    ((1, 256, 384, 4, 2, 128), "b1h1", "topk", 100, True),      # bias shared by all heads: fp32 atomics
    ((2, 256, 256, 2, 2, 128), "b1h1", "none", 0, False),       # bias shared by the batch
    ((1, 512, 512, 4, 2, 128), "perq", "randqh", 0, False),     # per-query-head mask, tiles empty for some heads
    ((1, 1, 700, 8, 2, 128), "bcast", "topk", 100, False),      # single query row
    ((1, 64, 256, 2, 2, 128), "bcast", "topk", 100, True),      # one step per CTA: only one softmax team ever works
    ((1, 128, 256, 2, 2, 128), "bcast", "topk", 100, False),    # two steps per CTA
    ((1, 192, 320, 2, 2, 128), "bcast", "topk", 90, False),     # three steps per CTA: odd count, teams uneven
]


@pytest.mark.parametrize("geom,bias_kind,mask_kind,window,causal", TC_BWD_CASES)
def test_tcgen05_forward_backward(dev, kernel_path, geom, bias_kind, mask_kind, window, causal):
    kernel_path("tcgen05")
    case = build_case(dev, *geom, bias_kind, mask_kind, window, torch.bfloat16)
    compare_all(case, causal, torch.bfloat16)


@pytest.mark.parametrize("geom,bias_kind,mask_kind,causal", [
    ((1, 256, 384, 4, 2, 128), "perq", "randq", True),      # per-query bias / mask / dBias shared by a head group
    ((1, 300, 420, 4, 4, 128), "perhead", "randq", True),   # one row per query head, ragged
    ((1, 256, 1280, 2, 1, 256), "perq", "randq", False),    # head dim 256 forward; CUDA-core backward
])
def test_per_query_tensors_in_fp16(dev, kernel_path, geom, bias_kind, mask_kind, causal):
    """The per-query kernels' 16- and 32-byte bias / mask / dBias accesses in the other 16-bit type."""
    kernel_path("auto")
    case = build_case(dev, *geom, bias_kind, mask_kind, 0, torch.float16)
    compare_all(case, causal, torch.float16)


def test_tcgen05_backward_fp16_and_run_to_run_spread(dev, kernel_path):
    kernel_path("tcgen05")
    case = build_case(dev, 1, 384, 384, 4, 2, 128, "bcast", "topk", 100, torch.float16)
    compare_all(case, True, torch.float16)
    # dQ goes through fp32 atomics: two runs may differ by accumulation order, but only at fp32 round-off
    q, k, v, mask, bias, dout = case
    a = run_ours(q, k, v, mask, bias, dout, True)
    b = run_ours(q, k, v, mask, bias, dout, True)
    for x, y in zip(a, b):
        assert (x.float() - y.float()).abs().max() <= 1e-2 * max(1.0, x.float().abs().max().item())
    assert torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])  # dK, dV have a fixed accumulation order


@pytest.mark.parametrize("d,bias_kind,mask_kind", [(128, "bcast", "topk"), (128, "perq", "randq"), (256, "bcast", "topk")])
def test_tcgen05_backward_deterministic(dev, kernel_path, d, bias_kind, mask_kind):
    """deterministic=True (reference: per-split dQ buffers, csrc/flash_sparse_attn/flash_api.cpp:960-965): the
    tensor-core backward kernels accumulate dQ in 64-bit fixed point, so repeated runs give bit-identical gradients,
    and the values still meet the oracle tolerance. 16 key tiles x 4 kv heads of CTAs add into every dQ tile."""
    from flash_sparse_attn import flash_sparse_attn_func

    kernel_path("tcgen05")
    dtype = torch.bfloat16
    q, k, v, mask, bias, dout = build_case(dev, 1, 2048, 2048, 8, 4, d, bias_kind, mask_kind, 600, dtype, seed=5)
    ref = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, True)

    def run():
        ql, kl, vl, bl = (t.detach().clone().requires_grad_(True) for t in (q, k, v, bias))
        out = flash_sparse_attn_func(ql, kl, vl, attn_mask=mask, attn_bias=bl, is_causal=True, deterministic=True)
        out.backward(dout)
        return out.detach(), ql.grad, kl.grad, vl.grad, bl.grad

    first = run()
    torch.cuda.synchronize()
    _kernel_status_ok()
    check("out", first[0], ref[0], dtype)
    check("dq", first[1], ref[2], dtype)
    check("dk", first[2], ref[3], dtype, reduced=True)
    check("dv", first[3], ref[4], dtype, reduced=True)
    check("dbias", first[4], ref[5], dtype, reduced=True)
    for _ in range(3):
        again = run()
        for name, a, b in zip(("out", "dq", "dk", "dv", "dbias"), first, again):
            assert torch.equal(a, b), f"{name} differs between runs"


TC_BWD256_CASES = [
    ((1, 384, 640, 4, 1, 256), "bcast", "topk", 200, True),     # MQA with wide heads, Sq < Sk
    ((2, 300, 300, 4, 2, 256), "bcast", "block", 100, True),    # ragged, GQA, whole key tiles without a kept key
    ((1, 256, 256, 2, 2, 256), "bcast", "topk", 64, False),     # MHA, non-causal
    ((1, 640, 128, 2, 1, 256), "none", "none", 0, True),        # Sq > Sk, neither mask nor bias
    ((1, 1024, 1024, 8, 1, 256), "bcast", "topk", 300, True),   # 8 key tiles x 16 query tiles x 8 heads: split grid
    ((1, 200, 520, 2, 1, 256), "none", "topk", 130, False),     # mask only, no dBias
    ((2, 130, 130, 16, 2, 256), "bcast", "topk", 40, True),     # batch of 2, groups of 8, ragged query tile
    ((1, 1, 700, 8, 2, 256), "bcast", "topk", 100, False),      # single query row
    ((1, 2048, 256, 2, 1, 256), "b1h1", "none", 0, True),       # 2 key tiles x 32 query tiles: 64 splits; Sq > Sk
]


def test_tcgen05_backward_head_dim_256_fp16(dev, kernel_path):
    kernel_path("tcgen05")
    case = build_case(dev, 1, 256, 384, 4, 2, 256, "bcast", "topk", 100, torch.float16)
    compare_all(case, True, torch.float16)


@pytest.mark.parametrize("geom,bias_kind,mask_kind,window,causal", TC_BWD256_CASES)
def test_tcgen05_backward_head_dim_256(dev, kernel_path, geom, bias_kind, mask_kind, window, causal):
    """Head dim 256: two-pass backward kernel (dV + dQ + dBias, then dK) for row-broadcast masks and biases."""
    kernel_path("tcgen05")
    case = build_case(dev, *geom, bias_kind, mask_kind, window, torch.bfloat16)
    compare_all(case, causal, torch.bfloat16)


PADDED_DIM_CASES = [
    ((1, 256, 256, 2, 1, 64), "bcast", "topk", 128, True),      # the small CPU-reference geometry: d=64 trains at 128
    ((2, 200, 333, 4, 2, 32), "perq", "randq", 0, True),
    ((1, 300, 300, 3, 3, 96), "perhead", "none", 0, False),
    ((1, 160, 160, 2, 2, 40), "bcast", "topk", 50, True),
    ((1, 256, 384, 2, 1, 192), "bcast", "topk", 100, True),     # forward and backward at 256
]


@pytest.mark.parametrize("geom,bias_kind,mask_kind,window,causal", PADDED_DIM_CASES)
def test_default_path_pads_small_head_dims(dev, geom, bias_kind, mask_kind, window, causal):
    """With the default kernel choice, head dims without a tensor-core kernel of their own are zero-padded to the
    next one (64 / 128 / 256 forward, 128 when gradients are needed); results and gradients keep their shape."""
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    d = geom[-1]
    assert iface._kernel_head_dim(d, True) == (128 if d <= 128 else 256)
    assert iface._kernel_head_dim(d, False) == (64 if d <= 64 else 128 if d <= 128 else 256)
    case = build_case(dev, *geom, bias_kind, mask_kind, window, torch.bfloat16)
    compare_all(case, causal, torch.bfloat16)


DECODE_CASES = [
    ((1, 1, 700, 8, 2, 128), "bcast", "topk", 100, "decode"),     # GQA group of 4 shares K/V rows
    ((2, 1, 5000, 4, 4, 64), "b1h1", "block", 300, "decode"),     # MHA, fully broadcast bias, long runs of skipped keys
    ((3, 1, 4096, 6, 2, 128), "perhead", "randqh", 0, "decode"),  # per-head mask/bias: one head per CTA
    ((1, 1, 333, 16, 2, 256), "bcast", "none", 0, "auto"),        # group of 8 at d=256: falls back to other kernels
    ((2, 1, 9000, 8, 1, 256), "bcast", "topk", 64, "auto"),       # MQA, d=256, group of 8 -> fallback, very sparse
    ((2, 1, 2048, 8, 4, 256), "bcast", "topk", 700, "decode"),    # d=256, group of 2
    ((1, 1, 40, 2, 2, 128), "none", "none", 0, "decode"),         # shorter than one chunk per warp
    ((2, 1, 20000, 8, 2, 128), "bcast", "topk", 1501, "decode"),  # group of 4: many ring drains, short tail batch
    ((1, 1, 3000, 8, 1, 64), "bcast", "topk", 333, "decode"),     # group of 8 at d=64
    ((1, 1, 1000, 4, 1, 64), "b1h1", "none", 0, "decode"),        # group of 4 at d=64, every key kept
    ((2, 1, 6000, 8, 1, 128), "bcast", "topk", 777, "decode"),    # group of 8 at d=128: all eight rows of the quad layout
    ((2, 1, 3000, 4, 2, 128), "bcast", "topk", 250, "decode"),    # group of 2 at d=128
    ((1, 1, 2500, 3, 3, 128), "bcast", "topk", 90, "decode"),     # no grouping (MHA) at d=128, short tail batches
]


@pytest.mark.parametrize("geom,bias_kind,mask_kind,window,path", DECODE_CASES)
def test_decode_forward_backward(dev, kernel_path, geom, bias_kind, mask_kind, window, path):
    kernel_path(path)
    case = build_case(dev, *geom, bias_kind, mask_kind, window, torch.bfloat16)
    compare_all(case, False, torch.bfloat16)


def test_decode_all_keys_masked_and_fp16(dev, kernel_path):
    from flash_sparse_attn import flash_sparse_attn_func

    kernel_path("decode")
    q, k, v, mask, bias, dout = build_case(dev, 2, 1, 512, 4, 2, 128, "bcast", "topk", 50, torch.float16)
    mask = mask.clone()
    mask[1] = False  # batch element 1 sees nothing: output 0
    out = flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias)
    ref, _ = oracle.attention_forward(q, k, v, mask, bias, None, False)
    check("out", out, ref, torch.float16)
    assert (out[1] == 0).all()


def test_tcgen05_forward_fp16(dev, kernel_path):
    kernel_path("tcgen05")
    case = build_case(dev, 1, 256, 256, 2, 1, 128, "bcast", "topk", 100, torch.float16)
    compare_all(case, True, torch.float16, fwd_only=True)


def test_tcgen05_matches_simt_lse(dev):
    """LSE is not visible through the autograd API; compare the two kernel families through the custom op."""
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    q, k, v, mask, bias, _ = build_case(dev, 1, 384, 384, 2, 1, 128, "bcast", "block", 64, torch.bfloat16)
    res = {}
    for path in ("simt", "tcgen05"):
        iface.set_kernel_path(path)
        res[path] = torch.ops.flash_sparse_attn._flash_sparse_attn_forward(q, k, v, mask, bias, 128 ** -0.5, True, 0.0,
                                                                          False)
    iface.set_kernel_path("auto")
    ref_out, ref_lse = oracle.attention_forward(q, k, v, mask, bias, None, True)
    for path in res:
        lse = res[path][1]
        inf_ref = torch.isinf(ref_lse)
        assert torch.equal(torch.isinf(lse), inf_ref), path
        assert (lse[inf_ref] > 0).all()
        torch.testing.assert_close(lse[~inf_ref], ref_lse[~inf_ref], atol=2e-3, rtol=1e-3)
        assert (res[path][0][inf_ref.transpose(1, 2)] == 0).all()


def test_golden_config1_through_the_operator(dev, golden_dir):
    """The reference's own eager outputs for config-1 geometry (fp32) vs. our kernels fed the bf16-rounded
    inputs: the error budget is the bf16 input rounding, so the thresholds are the north-star ones."""
    import numpy as np, os

    z = np.load(os.path.join(golden_dir, "eager_c1_causal.npz"))
    q, k, v = (torch.from_numpy(z[n]).transpose(1, 2).contiguous().to(torch.bfloat16).to(dev) for n in "qkv")
    bias = torch.from_numpy(z["bias"]).to(torch.bfloat16).to(dev)
    mask = torch.from_numpy(z["mask"]).to(dev)
    dout = torch.ones_like(q)
    ref = oracle.attention_forward_backward(q, k, v, mask, bias, dout, 64 ** -0.5, False)
    got = run_ours(q, k, v, mask, bias, dout, False, 64 ** -0.5)
    check("out", got[0], ref[0], torch.bfloat16)
    check("dq", got[1], ref[2], torch.bfloat16)
    check("dk", got[2], ref[3], torch.bfloat16, reduced=True)
    check("dv", got[3], ref[4], torch.bfloat16, reduced=True)
    check("dbias", got[4], ref[5], torch.bfloat16, reduced=True)
    # and the oracle on bf16-rounded inputs stays close to the reference's fp32 result
    gold = torch.from_numpy(z["out"]).to(dev)
    assert (ref[0] - gold).abs().max() < 0.1


def test_return_attn_probs_gives_lse(dev):
    """return_attn_probs=True returns (out, softmax_lse, empty): LSE (natural log, (B,H,Sq) fp32) matches the oracle,
    rows without a visible key report +inf."""
    from flash_sparse_attn import flash_sparse_attn_func

    q, k, v, mask, bias, _ = build_case(dev, 1, 300, 420, 4, 2, 128, "bcast", "topk", 90, torch.bfloat16)
    mask = mask.clone()
    mask[:, 1] = False  # the query heads of kv head 1 see nothing
    out, lse, probs = flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias, is_causal=True,
                                             return_attn_probs=True)
    ref_out, ref_lse = oracle.attention_forward(q, k, v, mask, bias, None, True)
    check("out", out, ref_out, torch.bfloat16)
    assert probs.numel() == 0 and lse.shape == (1, 4, 300) and lse.dtype == torch.float32
    finite = torch.isfinite(ref_lse)
    assert torch.equal(torch.isposinf(lse.cpu()), torch.isposinf(ref_lse.cpu()))
    assert (lse.cpu()[finite.cpu()] - ref_lse.cpu()[finite.cpu()]).abs().max() <= 2e-2


def test_error_paths_on_device(dev):
    from flash_sparse_attn import flash_sparse_attn_func

    q = torch.randn(1, 16, 2, 64, device=dev, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        flash_sparse_attn_func(q, q, q, softcap=1.0)
    with pytest.raises(RuntimeError):
        flash_sparse_attn_func(q, q[:, :, :1].expand(1, 16, 3, 64), q)
    with pytest.raises(RuntimeError):
        flash_sparse_attn_func(q.float(), q.float(), q.float())
