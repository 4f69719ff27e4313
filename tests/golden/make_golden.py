"""Generates tests/golden/*.npz by RUNNING THE REFERENCE'S OWN PYTHON CODE (needs the reference checkout).

    python tests/golden/make_golden.py /path/to/flash-dmattn-checkout

Imported from the reference: `flash_sparse_attn.utils.mask.create_mask` and
`benchmarks/backward_equivalence.py::dynamic_mask_attention_python` (its eager forward+backward). Every case
stores its seeded inputs next to the reference's outputs, so the fixtures are self-contained; the test-suite
only reads the .npz files. fp32 on CPU, one torch seed per case.
"""
import io
import contextlib
import os
import sys

import numpy as np
import torch

if len(sys.argv) != 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/flash-dmattn-checkout")
REF = sys.argv[1]
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "benchmarks"))
with contextlib.redirect_stdout(io.StringIO()):
    import backward_equivalence as ref_bwd  # noqa: E402
    from flash_sparse_attn.utils.mask import create_mask as ref_create_mask  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def eager_case(name, B, Sq, Sk, H, Hk, d, window, is_causal, seed):
    """dynamic_mask_attention_python as shipped: bias (B,Hk,Sq,Sk), mask = top-w among causally visible keys
    (create_mask(bias, causal_mask)), loss = out.sum()."""
    torch.manual_seed(seed)
    q = torch.randn(B, H, Sq, d)
    k = torch.randn(B, Hk, Sk, d)
    v = torch.randn(B, Hk, Sk, d)
    bias = torch.randn(B, Hk, Sq, Sk)
    causal_mask = torch.tril(torch.ones(Sq, Sk, dtype=torch.bool), diagonal=Sk - Sq)[None, None].expand(B, 1, Sq, Sk)
    ql, kl, vl, bl = (t.clone().requires_grad_(True) for t in (q, k, v, bias))
    out, dq, dk, dv, dbias = ref_bwd.dynamic_mask_attention_python(
        ql, kl, vl, bl, causal_mask if is_causal else None, d ** -0.5, window, is_causal
    )
    mask = ref_create_mask(bias, causal_mask if is_causal else None, B, Sq, Sk, window, torch.finfo(torch.float32).min)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        q=q.numpy(), k=k.numpy(), v=v.numpy(), bias=bias.numpy(), mask=mask.numpy(),
        out=out.detach().numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(), dbias=dbias.numpy(),
        meta=np.array([B, Sq, Sk, H, Hk, d, window, int(is_causal), seed]),
    )
    print(name, "ok; any NaN:", bool(torch.isnan(out).any()))


def mask_case(name, shape, window, seed, premask=None, block_size=None, kind="topk"):
    """create_mask alone, fp32 bias (no ties), optional 4-D pre-mask / block smoothing / relu."""
    torch.manual_seed(seed)
    bias = torch.randn(*shape)
    pm = None
    if premask == "causal":
        Sq, Sk = shape[2], shape[3]
        pm = torch.tril(torch.ones(Sq, Sk, dtype=torch.bool), diagonal=Sk - Sq)[None, None]
    elif premask == "padding2d":
        pm = torch.ones(shape[0], shape[3], dtype=torch.bool)
        pm[:, : shape[3] // 4] = False
    mask = ref_create_mask(bias, pm, shape[0], shape[2], shape[3], window, torch.finfo(torch.float32).min,
                           block_size=block_size, type=kind)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        bias=bias.numpy(), premask=(pm.numpy() if pm is not None else np.zeros(0, dtype=bool)), mask=mask.numpy(),
        meta=np.array([window, seed, block_size or 0, int(kind == "relu")]),
    )
    print(name, "ok; kept fraction:", float(mask.float().mean()))


if __name__ == "__main__":
    # BASELINE config-1 geometry (B1 S256 Hq2 Hkv1 d64 W128), run through the reference's eager function
    eager_case("eager_c1_causal", 1, 256, 256, 2, 1, 64, 128, True, 0)
    eager_case("eager_c1_noncausal", 1, 256, 256, 2, 1, 64, 128, False, 1)
    eager_case("eager_gqa_sq_lt_sk", 2, 64, 192, 4, 2, 32, 48, True, 2)
    mask_case("mask_rowbcast", (2, 2, 1, 512), 128, 3)
    mask_case("mask_causal_premask", (1, 2, 96, 96), 32, 4, premask="causal")
    mask_case("mask_padding2d", (2, 1, 1, 256), 64, 5, premask="padding2d")
    mask_case("mask_block_smooth", (1, 2, 1, 300), 150, 6, block_size=64)
    mask_case("mask_relu", (1, 2, 4, 200), 0, 7, kind="relu")
