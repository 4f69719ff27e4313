"""KV-ring context parallelism on CPU: world_size 2 and 4 `gloo` groups, the CPU oracle standing in for the device
operator. The gathered ring output and all gradients must equal the unsharded oracle on the full sequence."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_sparse_attn import ring
from oracle import oracle


def _fwd(q, k, v, mask, bias, scale, causal):
    return oracle.attention_forward(q, k, v, mask, bias, scale, causal)


def _bwd(dout, q, k, v, mask, bias, out, lse, scale, causal):
    """Gradients of one (query chunk, key chunk) pair given the GLOBAL out and lse of the query chunk."""
    B, Sq, H, d = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    G = H // Hk
    qf, do = q.float().transpose(1, 2), dout.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(G, 1)
    vf = v.float().transpose(1, 2).repeat_interleave(G, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if bias is not None:
        s = s + oracle._expand_heads(bias[..., :Sk].float(), H)
    vis = oracle.visible_mask(mask, B, H, Sq, Sk, causal, q.device)
    l = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).unsqueeze(-1)
    p = torch.where(vis & ~torch.isinf(lse).unsqueeze(-1), torch.exp(s - l), torch.zeros_like(s))
    D = (dout.float() * out.float()).sum(-1).transpose(1, 2).unsqueeze(-1)
    ds = p * (do @ vf.transpose(-1, -2) - D)
    dq = (ds @ kf * scale).transpose(1, 2)
    dk = (ds.transpose(-1, -2) @ qf * scale).view(B, Hk, G, Sk, d).sum(2).transpose(1, 2)
    dv = (p.transpose(-1, -2) @ do).view(B, Hk, G, Sk, d).sum(2).transpose(1, 2)
    dbias = None
    if bias is not None:
        db = ds
        if bias.shape[1] != H:
            db = db.view(B, bias.shape[1], H // bias.shape[1], Sq, Sk).sum(2)
        if bias.shape[2] == 1:
            db = db.sum(2, keepdim=True)
        if bias.shape[0] == 1:
            db = db.sum(0, keepdim=True)
        dbias = torch.nn.functional.pad(db, [0, bias.shape[-1] - Sk])
    return dq, dk, dv, dbias


def _worker(rank, world, port, causal, bias_heads, with_mask):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, Hk, d = 1, 4, 2, 16
        S = 2 * world * 128
        q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, bias_heads, 1, S), seed=3)
        mask = oracle.create_mask(bias, None, B, S, S, S // 5, torch.finfo(torch.float32).min) if with_mask else None
        want = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, causal)
        loc = lambda t, dim: ring.zigzag_split(t, dim, rank, world).contiguous()
        ql, kl, vl = (loc(t, 1).requires_grad_(True) for t in (q, k, v))
        bl = loc(bias, 3).requires_grad_(True)
        ml = loc(mask, 3) if mask is not None else None
        out = ring.ring_flash_sparse_attn_func(ql, kl, vl, ml, bl, None, causal, fwd_fn=_fwd, bwd_fn=_bwd)
        out.backward(loc(dout, 1))

        def gather(t, dim):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            return ring.zigzag_merge(parts, dim)

        torch.testing.assert_close(gather(out, 1), want[0], atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(gather(ql.grad, 1), want[2], atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(gather(kl.grad, 1), want[3], atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(gather(vl.grad, 1), want[4], atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(gather(bl.grad, 3), want[5], atol=1e-4, rtol=1e-4)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,causal,bias_heads,with_mask", [(2, True, 2, True), (2, False, 1, True), (4, True, 4, False)])
def test_ring_equals_unsharded(world, causal, bias_heads, with_mask):
    mp.spawn(_worker, args=(world, _free_port(), causal, bias_heads, with_mask), nprocs=world, join=True)


def test_zigzag_roundtrip():
    t = torch.arange(2 * 4 * 3).view(1, 24, 1)
    parts = [ring.zigzag_split(t, 1, r, 4) for r in range(4)]
    assert torch.equal(ring.zigzag_merge(parts, 1), t)
    assert ring.zigzag_chunks(1, 4) == (1, 6)
    with pytest.raises(ValueError):
        ring.zigzag_split(torch.zeros(1, 10, 1), 1, 0, 4)
