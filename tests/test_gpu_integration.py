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


def test_unsupported_branches_raise(dev):
    from flash_sparse_attn.integrations import flash_sparse_attention_forward

    module = _Attn(torch.bfloat16).to(dev)
    q = torch.zeros(1, 2, 16, 64, device=dev, dtype=torch.bfloat16)
    pad = torch.ones(1, 16, dtype=torch.bool, device=dev)
    with pytest.raises(NotImplementedError):
        flash_sparse_attention_forward(module, q, q, q, pad, None)
    with pytest.raises(ValueError):
        flash_sparse_attention_forward(module, q, q, q, pad, torch.zeros(1, 2, 1, 16, device=dev, dtype=torch.bfloat16))
    packed = torch.cat([torch.arange(8), torch.arange(8)])[None].to(dev)
    with pytest.raises(NotImplementedError):
        flash_sparse_attention_forward(module, q, q, q, None, None, position_ids=packed)
