"""The operator layer under torch.compile: the custom ops' schemas and fake (meta) kernels must let Dynamo / AOT
autograd trace flash_sparse_attn_func without graph breaks (reference: the custom_op + register_fake pairs of
flash_sparse_attn_interface.py:73-123 and :206-285), and the compiled function must return what eager returns.
`aot_eager` runs Dynamo, the fake-tensor propagation and AOT autograd's functionalisation without generating code."""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _inputs(dev, bias_rows):
    B, S, H, Hk, d = 2, 384, 4, 2, 128
    dtype = torch.bfloat16
    q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, Hk, bias_rows, S), seed=31, dtype=dtype)
    mask = oracle.create_mask(bias, None, B, S, S, 96, torch.finfo(dtype).min)
    return [t.to(dev) for t in (q, k, v, mask, bias, dout)]


@pytest.mark.parametrize("bias_rows", [1, 384])
def test_compiled_matches_eager(dev, bias_rows):
    from flash_sparse_attn import flash_sparse_attn_func

    q, k, v, mask, bias, dout = _inputs(dev, bias_rows)

    def fn(q, k, v, mask, bias):
        return flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias, is_causal=True)

    def run(f):
        qq, kk, vv, bb = (t.detach().clone().requires_grad_(True) for t in (q, k, v, bias))
        out = f(qq, kk, vv, mask, bb)
        out.backward(dout)
        return out.detach(), qq.grad, kk.grad, vv.grad, bb.grad

    from flash_sparse_attn.flash_sparse_attn_interface import set_compaction

    torch._dynamo.reset()
    compiled = torch.compile(fn, backend="aot_eager", fullgraph=True)
    set_compaction("off")  # the gathered-keys route is an eager-only choice; compare like with like
    try:
        want = run(fn)
        got = run(compiled)
    finally:
        set_compaction("auto")
    names = ("out", "dq", "dk", "dv", "dbias")
    for n, a, b in zip(names, got, want):
        assert a.shape == b.shape and a.dtype == b.dtype, n
        # same kernels on both sides; dq goes through fp32 reduce-adds whose order is not fixed
        tol = 2e-2 if n == "dq" else 0.0
        assert (a.float() - b.float()).abs().max().item() <= tol, n


def test_opcheck_forward_and_backward(dev):
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    q, k, v, mask, bias, dout = _inputs(dev, 1)
    scale = q.shape[-1] ** -0.5
    pad = (128 - mask.shape[-1] % 128) % 128
    mask_p = torch.nn.functional.pad(mask, (0, pad))
    bias_p = torch.nn.functional.pad(bias, (0, pad))
    fwd_args = (q, k, v, mask_p, bias_p, scale, True, 0.0, False)
    torch.library.opcheck(torch.ops.flash_sparse_attn._flash_sparse_attn_forward, fwd_args,
                          test_utils=("test_schema", "test_faketensor"))
    out, lse, _ = torch.ops.flash_sparse_attn._flash_sparse_attn_forward(*fwd_args)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    dbias = torch.zeros_like(bias_p)
    bwd_args = (dout, q, k, v, mask_p, bias_p, out, lse, dq, dk, dv, dbias, scale, True, 0.0, False)
    torch.library.opcheck(torch.ops.flash_sparse_attn._flash_sparse_attn_backward, bwd_args,
                          test_utils=("test_schema", "test_faketensor"))
