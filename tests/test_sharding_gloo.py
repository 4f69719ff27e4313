"""Multi-rank host logic on CPU: world_size-2 (and 4) `gloo` process groups run the unit sharding + gather with the
CPU oracle standing in for the device operator, and must reproduce the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_sparse_attn import sharding
from oracle import oracle


def test_plan_covers_every_unit_exactly_once():
    for B, H, Hk, world in [(8, 32, 8, 1), (8, 32, 8, 2), (8, 32, 8, 8), (1, 32, 8, 8), (2, 8, 4, 8), (4, 4, 2, 2)]:
        seen = torch.zeros(B, Hk, dtype=torch.int32)
        for r in range(world):
            s = sharding.plan_shard(B, H, Hk, r, world)
            seen[s.batch[0]:s.batch[1], s.kv_heads[0]:s.kv_heads[1]] += 1
            assert s.q_heads == (s.kv_heads[0] * (H // Hk), s.kv_heads[1] * (H // Hk))
        assert (seen == 1).all(), (B, H, Hk, world)
    with pytest.raises(ValueError):
        sharding.plan_shard(3, 4, 2, 0, 4)
    with pytest.raises(ValueError):
        sharding.plan_shard(1, 16, 1, 0, 2)  # a single kv head cannot be split into units


def _oracle_fn(q, k, v, attn_mask=None, attn_bias=None, softmax_scale=None, is_causal=None):
    return oracle.attention_forward(q, k, v, attn_mask, attn_bias, softmax_scale, bool(is_causal))[0]


def _worker(rank, world, port, B, H, Hk, bias_heads):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        Sq = Sk = 96
        d = 16
        q, k, v, bias, dout = oracle.make_inputs(B, Sq, Sk, H, Hk, d, (B, bias_heads, 1, Sk), seed=7)
        mask = oracle.create_mask(bias, None, B, Sq, Sk, 24, torch.finfo(torch.float32).min)
        want, _, dq_w, dk_w, dv_w, db_w = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, True)
        ql, kl, vl, bl = (t.clone().requires_grad_(True) for t in (q, k, v, bias))
        full = sharding.attention_sharded(ql, kl, vl, mask, bl, rank=rank, world=world, is_causal=True, gather=True,
                                          attn_fn=_oracle_fn)
        torch.testing.assert_close(full, want, atol=1e-5, rtol=1e-5)
        # gradients: each rank back-propagates only its own units; summed over ranks they give the full gradient
        local = sharding.attention_sharded(ql, kl, vl, mask, bl, rank=rank, world=world, is_causal=True,
                                           attn_fn=_oracle_fn)
        s = sharding.plan_shard(B, H, Hk, rank, world)
        local.backward(dout[s.batch[0]:s.batch[1], :, s.q_heads[0]:s.q_heads[1]])
        for got, ref in ((ql.grad, dq_w), (kl.grad, dk_w), (vl.grad, dv_w), (bl.grad, db_w)):
            g = got.clone()
            dist.all_reduce(g)
            torch.testing.assert_close(g, ref, atol=1e-4, rtol=1e-4)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,B,H,Hk,bias_heads", [(2, 2, 4, 2, 2), (2, 1, 4, 2, 4), (4, 2, 8, 4, 1)])
def test_sharded_equals_unsharded_gloo(world, B, H, Hk, bias_heads):
    mp.spawn(_worker, args=(world, _free_port(), B, H, Hk, bias_heads), nprocs=world, join=True)
