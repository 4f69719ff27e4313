"""Runtime behaviour of the library around its kernels: the bounded wait's give-up path, use of two devices from one
process, non-finite gradients in the deterministic backward, the returned softmax_d, and the position-list route
(`create_kept_keys` -> `flash_sparse_attn_func`) eagerly and under torch.compile."""
import ctypes

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


def test_bounded_wait_gives_up_and_the_device_stays_usable(dev):
    """fdma_selftest_wait_timeout: a CTA waits, with a 20 ms limit, on a barrier nothing arrives on. The wait must
    run out, the code must reach the status word and its host mirror, the CTA must free its tensor memory and
    return; the operator layer must refuse the next call, and after the status is read everything works again."""
    from flash_sparse_attn import _lib, flash_sparse_attn_func

    lib = _lib.load()
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.fdma_last_kernel_status(stream, None) == 0
    assert lib.fdma_poll_kernel_status(None) == 0
    result = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.fdma_selftest_wait_timeout(20000, result.data_ptr(), stream) == 0
    torch.cuda.synchronize()                      # returns: the kernel did not hang
    assert int(result.item()) == 1                # every thread saw its wait fail
    detail = ctypes.c_int32(0)
    assert lib.fdma_poll_kernel_status(ctypes.byref(detail)) == -6 and detail.value == 901
    q, k, v, bias, _ = oracle.make_inputs(1, 256, 256, 2, 1, 128, (1, 1, 1, 256), seed=3, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="bounded wait"):
        flash_sparse_attn_func(q, k, v, attn_bias=bias, is_causal=True)   # refused: an earlier kernel timed out
    assert lib.fdma_poll_kernel_status(None) == 0                          # the refusal read and cleared the status
    assert lib.fdma_last_kernel_status(stream, None) == 0
    # tensor memory was released (a full 512-column allocation succeeds) and results are right
    out = flash_sparse_attn_func(q, k, v, attn_bias=bias, is_causal=True)
    ref = oracle.attention_forward(q.cpu(), k.cpu(), v.cpu(), None, bias.cpu(), None, True)[0]
    torch.cuda.synchronize()
    _kernel_status_ok()
    check("out", out.cpu(), ref, torch.bfloat16)
    assert lib.fdma_selftest_wait_timeout(0, result.data_ptr(), stream) == -1          # limit out of range
    assert lib.fdma_selftest_wait_timeout(2000000, result.data_ptr(), stream) == -1


def test_forward_on_two_devices_in_one_process():
    """The dynamic shared-memory opt-in of the tcgen05 kernels belongs to the (function, device) pair: a process that
    uses cuda:0 and then cuda:1 must get correct results on both."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from flash_sparse_attn import flash_sparse_attn_func

    q, k, v, bias, dout = oracle.make_inputs(1, 384, 384, 4, 2, 128, (1, 2, 1, 384), seed=9, dtype=torch.bfloat16)
    ref = oracle.attention_forward_backward(q, k, v, None, bias, dout, None, True)
    for index in (0, 1, 0):
        d = torch.device(f"cuda:{index}")
        ql, kl, vl, bl = (t.to(d).requires_grad_(True) for t in (q, k, v, bias))
        out = flash_sparse_attn_func(ql, kl, vl, attn_bias=bl, is_causal=True)
        out.backward(dout.to(d))
        torch.cuda.synchronize(d)
        check("out", out.detach().cpu(), ref[0], torch.bfloat16)
        check("dq", ql.grad.cpu(), ref[2], torch.bfloat16)
        check("dk", kl.grad.cpu(), ref[3], torch.bfloat16, reduced=True)


def test_first_backward_of_a_fresh_process(dev):
    """The backward runs on an autograd worker thread. When everything that thread needs comes out of the allocator's
    cache, its first CUDA call of any kind is the library's tensor-map encode, a driver-API call that wants a context
    current on the calling thread: the library has to bind one itself. Needs a process of its own -- in this one
    earlier tests have long since made the worker thread allocate."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import torch\n"
        "from flash_sparse_attn import flash_sparse_attn_func\n"
        "g = torch.Generator(device='cuda').manual_seed(0)\n"
        "r = lambda *s: torch.randn(s, generator=g, device='cuda', dtype=torch.float32).to(torch.bfloat16)\n"
        "for d in (128, 256):\n"
        "    q, k, v, bias, dout = r(1, 256, 2, d), r(1, 256, 1, d), r(1, 256, 1, d), r(1, 1, 1, 256), r(1, 256, 2, d)\n"
        "    q.requires_grad_(True)\n"
        "    out = flash_sparse_attn_func(q, k, v, attn_bias=bias, is_causal=True)\n"
        "    out.backward(dout)\n"
        "    torch.cuda.synchronize()\n"
        "    assert torch.isfinite(q.grad.float()).all()\n"
        "print('backward ok')\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([root, os.path.join(root, "flash-dmattn_b200"),
                                                        os.environ.get("PYTHONPATH", "")]))
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "backward ok" in res.stdout, res.stderr[-2000:]


@pytest.mark.parametrize("d", [128, 256])
def test_deterministic_backward_propagates_non_finite(dev, d):
    """deterministic=True sums dQ in 64-bit fixed point, which cannot hold Inf or NaN; a row whose dOut carries an
    Inf (what a loss-scale overflow produces) must still come out non-finite, as it does on the fp32 path."""
    from flash_sparse_attn import flash_sparse_attn_func
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    B, S, H, Hk = 1, 256, 2, 1
    q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, 1, S), seed=2, dtype=torch.bfloat16, device=dev)
    dout[0, 100, 1, 5] = float("inf")
    iface.set_compaction("off")
    try:
        for det in (False, True):
            ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
            out = flash_sparse_attn_func(ql, kl, vl, attn_bias=bias, is_causal=True, deterministic=det)
            out.backward(dout)
            torch.cuda.synchronize()
            assert not torch.isfinite(ql.grad[0, 100, 1].float()).any(), f"deterministic={det}"
            assert torch.isfinite(ql.grad[0, 99].float()).all() and torch.isfinite(ql.grad[0, 100, 0].float()).all()
    finally:
        iface.set_compaction("auto")
    _kernel_status_ok()


@pytest.mark.parametrize("heads", ["kv", "query"])
def test_per_query_dbias_with_an_unpadded_key_extent(dev, heads):
    """The backward operator with a per-(query, key) dBias whose key extent is Sk itself (420, not a multiple of 32),
    a view into a wider buffer: the warps that lie wholly inside write 16-byte row pieces, the one that straddles Sk
    writes element by element, and nothing lands beyond key Sk - 1 or query Sq - 1."""
    B, Sq, Sk, H, Hk, d = 1, 300, 420, 4, 2, 128
    hb = Hk if heads == "kv" else H
    q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, (B, hb, Sq, Sk), seed=11, dtype=torch.bfloat16, device=dev)
    g = torch.Generator(device="cpu").manual_seed(12)
    mask = (torch.rand(B, hb, Sq, Sk, generator=g) < 0.3).to(dev)
    Sk_r = (Sk + 127) // 128 * 128
    pad = lambda t: torch.nn.functional.pad(t, (0, Sk_r - Sk))
    bias_p, mask_p = pad(bias), pad(mask)
    out, lse, _ = torch.ops.flash_sparse_attn._flash_sparse_attn_forward(q, k, v, mask_p, bias_p, d ** -0.5, True, 0.0, False)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    sentinel = 12345.0
    buf = torch.full((B, hb, Sq + 4, Sk_r), sentinel, dtype=torch.bfloat16, device=dev)
    db = buf[:, :, :Sq, :Sk]
    torch.ops.flash_sparse_attn._flash_sparse_attn_backward(dout, q, k, v, mask_p, bias_p, out, lse, dq, dk, dv, db,
                                                            d ** -0.5, True, 0.0, False)
    torch.cuda.synchronize()
    assert (buf[:, :, :, Sk:] == sentinel).all() and (buf[:, :, Sq:, :] == sentinel).all(), "write outside dBias"
    ref = oracle.attention_forward_backward(q.cpu(), k.cpu(), v.cpu(), mask.cpu(), bias.cpu(), dout.cpu(), None, True)
    check("dbias", db.cpu(), ref[5], torch.bfloat16, reduced=True)
    check("dq", dq.cpu(), ref[2], torch.bfloat16)
    _kernel_status_ok()


@pytest.mark.parametrize("geom,path", [((2, 200, 264, 4, 2, 128), "auto"), ((1, 130, 130, 2, 2, 64), "simt"),
                                       ((1, 256, 256, 2, 1, 256), "auto")])
def test_backward_operator_returns_softmax_d(dev, geom, path):
    """The backward operator returns D = rowsum(dOut o Out) as (B, H, round_up(Sq, 128)) fp32 with zero padding, like
    the reference's mha_bwd (csrc/flash_sparse_attn/flash_api.cpp:952, :1049)."""
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    B, Sq, Sk, H, Hk, d = geom
    q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, (B, Hk, 1, Sk), seed=7, dtype=torch.bfloat16, device=dev)
    pad = (128 - Sk % 128) % 128
    bias_p = torch.nn.functional.pad(bias, (0, pad))
    iface.set_kernel_path(path)
    try:
        out, lse, _ = torch.ops.flash_sparse_attn._flash_sparse_attn_forward(q, k, v, None, bias_p, d ** -0.5, True, 0.0, False)
        dq, dk, dv, db = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(bias_p)
        sd = torch.ops.flash_sparse_attn._flash_sparse_attn_backward(dout, q, k, v, None, bias_p, out, lse, dq, dk, dv, db,
                                                                      d ** -0.5, True, 0.0, False)
    finally:
        iface.set_kernel_path("auto")
    torch.cuda.synchronize()
    want = (dout.float() * out.float()).sum(-1).permute(0, 2, 1)       # (B, H, Sq)
    r128 = (Sq + 127) // 128 * 128
    assert sd.shape == (B, H, r128) and sd.dtype == torch.float32
    assert (sd[..., :Sq] - want).abs().max() < 1e-3 * max(1.0, want.abs().max().item())
    assert bool((sd[..., Sq:] == 0).all())


@pytest.mark.parametrize("geom,hb", [((2, 384, 1024, 4, 2, 128), 2), ((1, 512, 1536, 4, 2, 128), 4),
                                     ((1, 640, 640, 8, 2, 64), 0), ((1, 1, 900, 8, 2, 128), 2)])
def test_position_list_route_vs_oracle(dev, geom, hb):
    """`create_kept_keys` (no bool mask anywhere) -> `flash_sparse_attn_func`: O and gradients against the oracle run
    with the oracle's own bool mask. The single-query case falls back to a bool mask internally."""
    from flash_sparse_attn import flash_sparse_attn_func
    from flash_sparse_attn.utils.mask import create_kept_keys

    B, Sq, Sk, H, Hk, d = geom
    W = 200
    dtype = torch.bfloat16
    bshape = (B, {0: Hk, 2: Hk, 4: H}[hb], 1, Sk)
    q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, bshape, seed=21, dtype=dtype)
    sel = bias if bias.shape[1] == Hk else bias[:, ::H // Hk]            # the selection is made per kv head
    sel = sel.contiguous()
    mask = oracle.create_mask(sel, None, B, Sq, Sk, W, torch.finfo(dtype).min)
    use_bias = hb != 0
    ref = oracle.attention_forward_backward(q, k, v, mask, bias if use_bias else None, dout, None, True)
    ql, kl, vl = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    bl = bias.to(dev).requires_grad_(True) if use_bias else None
    kept = create_kept_keys(sel.to(dev), None, B, Sq, Sk, W, torch.finfo(dtype).min)
    out = flash_sparse_attn_func(ql, kl, vl, attn_mask=kept, attn_bias=bl, is_causal=True)
    out.backward(dout.to(dev))
    torch.cuda.synchronize()
    _kernel_status_ok()
    check("out", out.detach().cpu(), ref[0], dtype)
    check("dq", ql.grad.cpu(), ref[2], dtype)
    check("dk", kl.grad.cpu(), ref[3], dtype, reduced=True)
    check("dv", vl.grad.cpu(), ref[4], dtype, reduced=True)
    if use_bias:
        check("dbias", bl.grad.cpu(), ref[5], dtype, reduced=True)


def test_position_list_route_under_torch_compile(dev):
    """The gathered route is made of custom ops with fake kernels: with the position list as an input, Dynamo and AOT
    autograd trace flash_sparse_attn_func in one graph, and the compiled function returns what eager returns."""
    from flash_sparse_attn import flash_sparse_attn_func
    from flash_sparse_attn.utils.mask import create_kept_keys

    B, S, H, Hk, d, W = 2, 512, 4, 2, 128, 128
    dtype = torch.bfloat16
    q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, 1, S), seed=33, dtype=dtype, device=dev)
    kept = create_kept_keys(bias, None, B, S, S, W, torch.finfo(dtype).min)

    def fn(q, k, v, kept, bias):
        return flash_sparse_attn_func(q, k, v, attn_mask=kept, attn_bias=bias, is_causal=True)

    def run(f):
        qq, kk, vv, bb = (t.detach().clone().requires_grad_(True) for t in (q, k, v, bias))
        out = f(qq, kk, vv, kept, bb)
        out.backward(dout)
        return out.detach(), qq.grad, kk.grad, vv.grad, bb.grad

    torch._dynamo.reset()
    want = run(fn)
    got = run(torch.compile(fn, backend="aot_eager", fullgraph=True))
    for n, a, b in zip(("out", "dq", "dk", "dv", "dbias"), got, want):
        assert a.shape == b.shape and a.dtype == b.dtype, n
        tol = 2e-2 if n == "dq" else 0.0   # same kernels; dq goes through fp32 reduce-adds whose order is not fixed
        assert (a.float() - b.float()).abs().max().item() <= tol, n
    torch.library.opcheck(torch.ops.flash_sparse_attn._compact_forward,
                          (q, k, v, bias, kept.key_pos, kept.slot_mask, d ** -0.5, True),
                          test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(torch.ops.flash_sparse_attn._index_kept_keys,
                          (torch.rand(B, Hk, S, device=dev) < 0.2, 256), test_utils=("test_schema", "test_faketensor"))
