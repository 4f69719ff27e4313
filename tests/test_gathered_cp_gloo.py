"""Gathered-keys context parallelism on CPU: world_size 2 and 4 `gloo` groups, with a plain-torch implementation of
the five device operations (index / gather / scatter / forward / backward over gathered keys; the attention itself is
the CPU oracle with an explicit visibility mask built from the key positions). The gathered output and all
gradients must equal the unsharded oracle on the full sequence."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_sparse_attn import gathered_cp, ring
from oracle import oracle

INT_MAX = 2**31 - 1


class TorchOps:
    def index(self, mask_rows, capacity):
        Bm, Hm, S = mask_rows.shape
        key_pos = torch.full((Bm, Hm, capacity), INT_MAX, dtype=torch.int32)
        mask_c = torch.zeros((Bm, Hm, 1, capacity), dtype=torch.bool)
        for b in range(Bm):
            for h in range(Hm):
                idx = torch.nonzero(mask_rows[b, h]).flatten()
                key_pos[b, h, : idx.numel()] = idx.to(torch.int32)
                mask_c[b, h, 0, : idx.numel()] = True
        return key_pos, mask_c

    @staticmethod
    def _rows(src, key_pos, b, h, heads):  # src (S, d) -> (cap, d), zeros where the slot is not in range
        pos = key_pos[b if key_pos.shape[0] > 1 else 0, h // (heads // key_pos.shape[1])].long()
        ok = (pos >= 0) & (pos < src.shape[0])
        return torch.where(ok.unsqueeze(-1), src[pos.clamp(0, src.shape[0] - 1)], torch.zeros(1, src.shape[1], dtype=src.dtype))

    def gather(self, key, value, bias, key_pos):
        B, S, Hk, d = key.shape
        cap = key_pos.shape[-1]
        k_c, v_c = torch.zeros(B, cap, Hk, d, dtype=key.dtype), torch.zeros(B, cap, Hk, d, dtype=key.dtype)
        for b in range(B):
            for h in range(Hk):
                k_c[b, :, h] = self._rows(key[b, :, h], key_pos, b, h, Hk)
                v_c[b, :, h] = self._rows(value[b, :, h], key_pos, b, h, Hk)
        bias_c = None
        if bias is not None:
            Bc, Hc = max(bias.shape[0], key_pos.shape[0]), max(bias.shape[1], key_pos.shape[1])
            bias_c = torch.zeros(Bc, Hc, 1, cap, dtype=bias.dtype)
            for b in range(Bc):
                for h in range(Hc):
                    src = bias[b if bias.shape[0] > 1 else 0, h if bias.shape[1] > 1 else 0, 0, :S]
                    bias_c[b, h, 0] = self._rows(src.unsqueeze(-1), key_pos, b, h, Hc)[:, 0]
        return k_c, v_c, bias_c

    def scatter(self, src_c, key_pos, rows_full, bias_layout=False):
        if bias_layout:
            Bc, Hc, _, cap = src_c.shape
            full = torch.zeros(Bc, Hc, 1, rows_full, dtype=src_c.dtype)
            for b in range(Bc):
                for h in range(Hc):
                    pos = key_pos[b if key_pos.shape[0] > 1 else 0, h // (Hc // key_pos.shape[1])].long()
                    ok = (pos >= 0) & (pos < rows_full)
                    full[b, h, 0, pos[ok]] = src_c[b, h, 0, ok]
            return full
        B, cap, Hk, d = src_c.shape
        full = torch.zeros(B, rows_full, Hk, d, dtype=src_c.dtype)
        for b in range(B):
            for h in range(Hk):
                pos = key_pos[b if key_pos.shape[0] > 1 else 0, h // (Hk // key_pos.shape[1])].long()
                ok = (pos >= 0) & (pos < rows_full)
                full[b, pos[ok], h] = src_c[b, ok, h]
        return full

    @staticmethod
    def _vis(mask_c, key_pos, Sq, shift, causal):
        vis = mask_c.expand(-1, -1, Sq, -1).clone()                    # (Bm,Hm,Sq,cap)
        if causal:
            rows = torch.arange(Sq).view(1, 1, Sq, 1) + shift
            vis &= key_pos.unsqueeze(2).long() <= rows
        return vis

    def forward(self, q, k_c, v_c, mask_c, bias_c, key_pos, shift, scale, causal, seqlen_k):
        return oracle.attention_forward(q, k_c, v_c, self._vis(mask_c, key_pos, q.shape[1], shift, causal), bias_c, scale,
                                        False)

    def backward(self, dout, q, k_c, v_c, mask_c, bias_c, key_pos, shift, out, lse, scale, causal, seqlen_k):
        vis = self._vis(mask_c, key_pos, q.shape[1], shift, causal)
        with torch.enable_grad():  # called from inside an autograd backward, where grad mode is off
            res = oracle.attention_forward_backward(q, k_c, v_c, vis, bias_c, dout, scale, False)
        return res[2], res[3], res[4], res[5]


def _worker(rank, world, port, causal, mask_heads, bias_heads):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, Hk, d = 1, 4, 2, 16
        S = 2 * world * 64
        q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, bias_heads, 1, S), seed=8) if bias_heads else \
            oracle.make_inputs(B, S, S, H, Hk, d, None, seed=8)
        g = torch.Generator().manual_seed(1)
        src = torch.randn((B, mask_heads, 1, S), generator=g)
        mask = oracle.create_mask(src, None, B, S, S, S // 6, torch.finfo(torch.float32).min)
        want = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, causal)
        loc = lambda t, dim: ring.zigzag_split(t, dim, rank, world).contiguous()
        ql, kl, vl = (loc(t, 1).requires_grad_(True) for t in (q, k, v))
        bl = loc(bias, 3).requires_grad_(True) if bias is not None else None
        out = gathered_cp.gathered_cp_flash_sparse_attn_func(ql, kl, vl, loc(mask, 3), bl, None, causal, ops=TorchOps())
        out.backward(loc(dout, 1))

        def gather(t, dim):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            return ring.zigzag_merge(parts, dim)

        torch.testing.assert_close(gather(out, 1), want[0], atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(gather(ql.grad, 1), want[2], atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(gather(kl.grad, 1), want[3], atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(gather(vl.grad, 1), want[4], atol=1e-4, rtol=1e-4)
        if bias is not None:
            torch.testing.assert_close(gather(bl.grad, 3), want[5], atol=1e-4, rtol=1e-4)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,causal,mask_heads,bias_heads", [(2, True, 2, 2), (2, False, 1, 4), (4, True, 2, 1),
                                                                (2, True, 1, 0)])
def test_gathered_cp_equals_unsharded(world, causal, mask_heads, bias_heads):
    mp.spawn(_worker, args=(world, _free_port(), causal, mask_heads, bias_heads), nprocs=world, join=True)
