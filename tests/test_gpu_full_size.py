"""Full BASELINE sizes, checked through properties that need no full-size oracle, plus a row-chunked fp32 oracle for
one kv-head group at S = 32768.

Properties (exact in real arithmetic, so the tolerances are bf16/fp32 round-off):
  * with V = 1 every non-empty row of O is 1 (softmax weights sum to one);
  * sum_k dV[k, :] over the keys of a kv head = sum over its query heads and non-empty rows of dO;
  * dS rows sum to zero, so a query-broadcast dBias sums to zero over keys (per batch and bias head);
  * O is linear in V: O(V1 + V2) = O(V1) + O(V2) (same mask, same probabilities).
"""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True, params=["off", "auto"], ids=["tiles", "compaction"])
def compaction_mode(request):
    """Both routes at full size: tile skipping over all keys, and the default (kept keys gathered first)."""
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    iface.set_compaction(request.param)
    yield request.param
    iface.set_compaction("auto")


def _run(q, k, v, mask, bias, dout, causal=True):
    from flash_sparse_attn import flash_sparse_attn_func

    ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
    bl = bias.detach().requires_grad_(True)
    out = flash_sparse_attn_func(ql, kl, vl, attn_mask=mask, attn_bias=bl, is_causal=causal)
    out.backward(dout)
    return out.detach(), ql.grad, kl.grad, vl.grad, bl.grad


def _gen(dev, B, S, H, Hk, d, bias_rows, window, seed):
    from flash_sparse_attn.utils.mask import create_mask

    g = torch.Generator(device=dev).manual_seed(seed)
    rnd = lambda *s: torch.randn(s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, dout = rnd(B, S, H, d), rnd(B, S, Hk, d), rnd(B, S, Hk, d), rnd(B, S, H, d)
    bias = rnd(B, Hk, bias_rows, S)
    mask = create_mask(bias, None, B, S, S, window, torch.finfo(torch.bfloat16).min)
    return q, k, v, mask, bias, dout


@pytest.mark.parametrize("name,B,S,H,Hk,d,bias_rows,window", [
    ("config3_one_batch_element", 1, 32768, 32, 8, 128, 1, 2048),
    ("config2", 1, 8192, 32, 8, 128, 8192, 1024),
    ("config5_on_one_gpu", 1, 131072, 16, 1, 256, 1, 1024),
])
def test_properties_at_full_size(dev, compaction_mode, name, B, S, H, Hk, d, bias_rows, window):
    if name.startswith("config5") and compaction_mode == "off":
        pytest.skip("317 TFLOP over the full key range: covered at small sizes, run here over the gathered keys only")
    q, k, v, mask, bias, dout = _gen(dev, B, S, H, Hk, d, bias_rows, window, seed=0)
    G = H // Hk
    # rows that see at least one key: causal AND mask
    if bias_rows == 1:
        first_kept = mask[:, :, 0].float().argmax(-1)                      # (B,Hk): first kept key
        alive = torch.arange(S, device=dev).view(1, 1, S) >= first_kept.unsqueeze(-1)   # (B,Hk,S)
    else:
        causal = torch.arange(S, device=dev).view(S, 1) >= torch.arange(S, device=dev).view(1, S)
        alive = (mask & causal).any(-1)                                    # (B,Hk,S)
    alive_q = alive.repeat_interleave(G, 1).transpose(1, 2)                # (B,S,H)

    ones = torch.ones_like(v)
    out1, _, _, dv1, dbias1 = _run(q, k, ones, mask, bias, dout)
    assert torch.isfinite(out1.float()).all()
    assert (out1[alive_q].float() - 1).abs().max() < 1e-2                  # weights sum to one
    assert (out1[~alive_q] == 0).all()                                     # empty rows give zero
    # sum_k dV = sum of dO over alive rows of the head group
    want = (dout.float() * alive_q.unsqueeze(-1)).view(B, S, Hk, G, d).sum(dim=(1, 3))
    got = dv1.float().sum(1)
    assert (got - want).abs().max() <= 2e-3 * want.abs().max() + 0.5, (got - want).abs().max()

    out, dq, dk, dv, dbias = _run(q, k, v, mask, bias, dout)
    for t in (out, dq, dk, dv, dbias):
        assert torch.isfinite(t.float()).all()
    # dS rows sum to zero
    if bias_rows == 1:
        tot = dbias.float().sum(-1)
        scale = dbias.float().abs().sum(-1)
        assert (tot.abs() <= 2e-3 * scale + 1.0).all(), (tot, scale)
    else:
        row = dbias.float().sum(-1)                                        # (B,Hk,S)
        assert row.abs().max() < 0.25, row.abs().max()                     # each row: sum of ~1000 bf16-rounded terms
    # linearity in V
    v2 = torch.randn_like(v)
    from flash_sparse_attn import flash_sparse_attn_func
    with torch.no_grad():
        o_a = flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias, is_causal=True).float()
        o_b = flash_sparse_attn_func(q, k, v2, attn_mask=mask, attn_bias=bias, is_causal=True).float()
        o_ab = flash_sparse_attn_func(q, k, (v.float() + v2.float()).to(v.dtype), attn_mask=mask, attn_bias=bias,
                                      is_causal=True).float()
    assert (o_ab - (o_a + o_b)).abs().max() < 6e-2   # three bf16 roundings of O(1) values


def test_one_kv_head_group_against_chunked_oracle_at_32k(dev):
    """fp32 oracle evaluated in chunks of 2048 query rows (scores of a whole head do not fit): O and all gradients
    of one kv head with its four query heads at S = 32768, W = 2048."""
    B, S, H, Hk, d, W = 1, 32768, 4, 1, 128, 2048
    q, k, v, mask, bias, dout = _gen(dev, B, S, H, Hk, d, 1, W, seed=1)
    out, dq, dk, dv, dbias = _run(q, k, v, mask, bias, dout)
    kf = k.float().requires_grad_(True)
    vf = v.float().requires_grad_(True)
    bf = bias.float().requires_grad_(True)
    R = 2048
    o_ref = torch.empty((B, S, H, d), dtype=torch.float32, device=dev)
    dq_ref = torch.empty_like(o_ref)
    for r0 in range(0, S, R):
        qc = q[:, r0:r0 + R].float().requires_grad_(True)
        kc, vc = kf[:, : r0 + R], vf[:, : r0 + R]                          # causal: later keys are invisible anyway
        oc, _ = oracle.attention_forward(qc, kc, vc, mask[..., : r0 + R], bf[..., : r0 + R], None, True)
        (oc * dout[:, r0:r0 + R].float()).sum().backward()
        o_ref[:, r0:r0 + R] = oc.detach()
        dq_ref[:, r0:r0 + R] = qc.grad
    for name, got, ref, reduced in (("out", out, o_ref, False), ("dq", dq, dq_ref, False), ("dk", dk, kf.grad, True),
                                    ("dv", dv, vf.grad, True), ("dbias", dbias, bf.grad, True)):
        r = oracle.error_report(name, got, ref)
        lim = 2e-2 + (3 * r["floor_max_abs"] if reduced else 0.0)
        mlim = 2e-3 + (2 * r["floor_mean_abs"] if reduced else 0.0)
        assert r["max_abs"] <= lim and r["mean_abs"] <= mlim, r


def test_config5_geometry_forward_properties(dev):
    """BASELINE config 5 on one GPU, forward only (its backward runs on the CUDA-core kernels and is covered at small
    sizes): B=1, S=131072, Hq=16, Hkv=1, d=256, top-1024 row-broadcast mask, causal. Softmax weights sum to one on
    rows that see a key, rows before the first kept key give zero, and the output is linear in V."""
    from flash_sparse_attn import flash_sparse_attn_func

    B, S, H, Hk, d, W = 1, 131072, 16, 1, 256, 1024
    q, k, v, mask, bias, _ = _gen(dev, B, S, H, Hk, d, 1, W, seed=3)
    first_kept = int(mask[0, 0, 0].float().argmax())
    with torch.no_grad():
        o1 = flash_sparse_attn_func(q, k, torch.ones_like(v), attn_mask=mask, attn_bias=bias, is_causal=True).float()
        assert torch.isfinite(o1).all()
        assert (o1[:, first_kept:] - 1).abs().max() < 1e-2
        assert (o1[:, :first_kept] == 0).all()
        del o1
        v2 = torch.randn_like(v)
        o_a = flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias, is_causal=True).float()
        o_b = flash_sparse_attn_func(q, k, v2, attn_mask=mask, attn_bias=bias, is_causal=True).float()
        o_ab = flash_sparse_attn_func(q, k, (v.float() + v2.float()).to(v.dtype), attn_mask=mask, attn_bias=bias,
                                      is_causal=True).float()
    assert (o_ab - (o_a + o_b)).abs().max() < 6e-2
