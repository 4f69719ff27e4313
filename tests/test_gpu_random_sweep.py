"""A seeded random sweep over shapes, head layouts, mask / bias layouts, dtypes, routes and the deterministic flag,
each case checked against the fp32 oracle. It looks for gross errors: a crash, a non-finite value, a kernel wait
that gave up, or an error beyond TWICE the bounds of `oracle.within_tolerance`. The bounds themselves are tuned to the
benchmark's value ranges; random head counts and lengths produce dQ and dBias of magnitude 4 to 200, where half an ulp
of the 16-bit result is 0.016 to 0.5, and about one case in 200 lands slightly above them (up to 1.9x in 28 881 cases
of this generator on a B200) -- the sweep allows 3 % of its cases to do so and none to reach 2x."""
import ctypes
import random

import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

CASES = 300


def _case(rng):
    d = rng.choice([32, 64, 64, 128, 128, 128, 96, 256, 40])
    Hk = rng.choice([1, 1, 2, 3])
    H = Hk * rng.choice([1, 2, 4, 8])
    B = rng.choice([1, 1, 2])
    Sq = rng.choice([1, 17, 64, 100, 128, 200, 256, 300, 384, 513])
    Sk = rng.choice([64, 100, 128, 200, 256, 333, 384, 512, 640, 1000])
    if rng.random() < 0.5:
        Sk = max(Sk, Sq)
    bshape = rng.choice([None, (B, Hk, 1, Sk), (B, Hk, Sq, Sk), (B, H, Sq, Sk), (1, 1, 1, Sk), (B, H, 1, Sk),
                         (1, Hk, 1, Sk), (B, 1, Sq, Sk)])
    return dict(B=B, Sq=Sq, Sk=Sk, H=H, Hk=Hk, d=d, causal=rng.random() < 0.6,
                dtype=rng.choice([torch.bfloat16, torch.bfloat16, torch.float16]), bshape=bshape,
                mkind=rng.choice(["none", "topk", "rowrand", "perq", "perqh", "perq1"]),
                window=rng.choice([16, 100, 300]), keep=rng.choice([0.05, 0.3, 0.9]),
                det=rng.random() < 0.2, route=rng.choice(["auto", "auto", "off"]), seed=rng.randrange(1 << 30))


def _mask(c, bias):
    B, Sq, Sk, H, Hk, dtype = c["B"], c["Sq"], c["Sk"], c["H"], c["Hk"], c["dtype"]
    g = torch.Generator().manual_seed(c["seed"] + 1)
    kind = c["mkind"]
    if kind == "none":
        return None
    if kind == "topk":
        src = bias if (bias is not None and bias.shape[2] == 1) else torch.randn((B, Hk, 1, Sk), generator=g).to(dtype)
        return oracle.create_mask(src, None, src.shape[0], Sq, Sk, max(1, min(c["window"], Sk)), torch.finfo(dtype).min)
    if kind == "rowrand":
        return torch.rand((B, Hk, 1, Sk), generator=g) < c["keep"]
    if kind == "perq":
        return torch.rand((B, Hk, Sq, Sk), generator=g) < 0.3
    if kind == "perqh":
        return torch.rand((B, H, Sq, Sk), generator=g) < 0.3
    return torch.rand((1, 1, Sq, Sk), generator=g) < 0.5


def test_random_configurations_against_the_oracle():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_sparse_attn import _lib, flash_sparse_attn_func
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    dev = torch.device("cuda:0")
    rng = random.Random(20240607)
    above, gross = [], []
    for _ in range(CASES):
        c = _case(rng)
        q, k, v, bias, dout = oracle.make_inputs(c["B"], c["Sq"], c["Sk"], c["H"], c["Hk"], c["d"], c["bshape"],
                                                 seed=c["seed"], dtype=c["dtype"])
        mask = _mask(c, bias)
        ref = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, c["causal"])
        ql, kl, vl = (t.to(dev).requires_grad_(True) for t in (q, k, v))
        bl = bias.to(dev).requires_grad_(True) if bias is not None else None
        iface.set_compaction(c["route"])
        try:
            out = flash_sparse_attn_func(ql, kl, vl, attn_mask=None if mask is None else mask.to(dev), attn_bias=bl,
                                         is_causal=c["causal"], deterministic=c["det"])
            out.backward(dout.to(dev))
            torch.cuda.synchronize()
        finally:
            iface.set_compaction("auto")
        detail = ctypes.c_int32(0)
        st = _lib.load().fdma_last_kernel_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(detail))
        assert st == 0, f"kernel wait timed out, code {detail.value}: {c}"
        got = (out, ql.grad, kl.grad, vl.grad, bl.grad if bl is not None else None)
        for name, gt, rf, red in (("out", got[0], ref[0], False), ("dq", got[1], ref[2], False),
                                  ("dk", got[2], ref[3], True), ("dv", got[3], ref[4], True),
                                  ("dbias", got[4], ref[5], True)):
            if gt is None:
                continue
            assert torch.isfinite(gt.float()).all(), f"{name} non-finite: {c}"
            r = oracle.error_report(name, gt.detach().cpu(), rf, c["dtype"])
            ok, msg = oracle.within_tolerance(r, red)
            if not ok:
                above.append((msg, c))
                lim = oracle.MAX_ABS + (oracle.FLOOR_FACTOR * r["floor_bound"] if red else 0.0)
                mlim = oracle.MEAN_ABS + (oracle.FLOOR_FACTOR * r["floor_mean_abs"] if red else 0.0)
                if r["max_abs"] > 2 * lim or r["mean_abs"] > 2 * mlim:
                    gross.append((msg, c))
    assert not gross, gross[:3]
    assert len(above) <= 0.03 * CASES, above[:5]
