"""Multi-GPU launcher: shards independent (batch, kv-head) attention units over the ranks of one node.

An attention unit is one batch element b and one kv head h_k with the G = H / Hk query heads that read it:
Q/O/dO/dQ[b, :, h_k*G:(h_k+1)*G, :], K/V/dK/dV[b, :, h_k, :], mask/bias/dBias[b, h_k]. Units never exchange data in
forward or backward, so each rank (one process per GPU) simply runs the operator on its own units; no collective
is on the data path. `gather=True` adds one all_gather of the outputs for callers that want the full tensor on
every rank. The reference has no multi-GPU code at all (its README lists sequence parallelism as future work).
"""
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch


@dataclass(frozen=True)
class UnitShard:
    """What one rank owns: a batch range and a kv-head range (query heads follow from the kv heads)."""
    batch: Tuple[int, int]
    kv_heads: Tuple[int, int]
    group: int  # query heads per kv head

    @property
    def q_heads(self) -> Tuple[int, int]:
        return self.kv_heads[0] * self.group, self.kv_heads[1] * self.group

    @property
    def n_units(self) -> int:
        return (self.batch[1] - self.batch[0]) * (self.kv_heads[1] - self.kv_heads[0])


def plan_shard(batch: int, heads: int, kv_heads: int, rank: int, world: int) -> UnitShard:
    """Splits batch first (world <= B, B % world == 0), else one batch slice per group of ranks and kv heads
    within it (world = B' * R with B % B' == 0, Hk % R == 0). Raises ValueError when units do not divide."""
    if heads % kv_heads:
        raise ValueError("query heads must be a multiple of kv heads")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    g = heads // kv_heads
    if batch % world == 0:
        per = batch // world
        return UnitShard((rank * per, (rank + 1) * per), (0, kv_heads), g)
    for ranks_per_batch_slice in range(2, world + 1):
        if world % ranks_per_batch_slice:
            continue
        batch_slices = world // ranks_per_batch_slice
        if batch % batch_slices or kv_heads % ranks_per_batch_slice:
            continue
        per_b = batch // batch_slices
        per_h = kv_heads // ranks_per_batch_slice
        bs, hs = divmod(rank, ranks_per_batch_slice)
        return UnitShard((bs * per_b, (bs + 1) * per_b), (hs * per_h, (hs + 1) * per_h), g)
    raise ValueError(f"{batch} x {kv_heads} (batch x kv-head) units cannot be split evenly over {world} ranks")


def _slice_heads(t: torch.Tensor, dim: int, full: int, kv_heads: int, shard: UnitShard) -> torch.Tensor:
    """Head dimension of a mask/bias: extent 1 (shared: keep), Hk (slice kv heads) or H (slice query heads)."""
    n = t.shape[dim]
    if n == 1:
        return t
    lo, hi = shard.kv_heads if n == kv_heads else shard.q_heads
    if n not in (kv_heads, full):
        raise ValueError("mask/bias head dimension must be 1, num_heads_k or num_heads")
    return t.narrow(dim, lo, hi - lo)


def shard_inputs(q, k, v, mask, bias, shard: UnitShard):
    """Views of the rank's units; q (B,Sq,H,d), k/v (B,Sk,Hk,d), mask/bias ({B|1},{H|Hk|1},{Sq|1},Sk)."""
    H, Hk = q.shape[2], k.shape[2]
    b0, b1 = shard.batch
    q0, q1 = shard.q_heads
    h0, h1 = shard.kv_heads
    ql = q[b0:b1, :, q0:q1]
    kl, vl = k[b0:b1, :, h0:h1], v[b0:b1, :, h0:h1]

    def mb(t):
        if t is None:
            return None
        t = t if t.shape[0] == 1 else t[b0:b1]
        return _slice_heads(t, 1, H, Hk, shard)

    return ql, kl, vl, mb(mask), mb(bias)


def attention_sharded(q, k, v, mask=None, bias=None, *, rank: int, world: int, softmax_scale=None, is_causal=None,
                      gather: bool = False, group=None, attn_fn: Optional[Callable] = None) -> torch.Tensor:
    """Runs the operator on this rank's units of the given (full) tensors and returns the local output
    (B_local, Sq, H_local, d), or the full (B, Sq, H, d) output on every rank when gather=True."""
    if attn_fn is None:
        from .flash_sparse_attn_interface import flash_sparse_attn_func as attn_fn
    B, _, H, _ = q.shape
    shard = plan_shard(B, H, k.shape[2], rank, world)
    ql, kl, vl, ml, bl = shard_inputs(q, k, v, mask, bias, shard)
    out = attn_fn(ql, kl, vl, attn_mask=ml, attn_bias=bl, softmax_scale=softmax_scale, is_causal=is_causal)
    if not gather or world == 1:
        return out
    import torch.distributed as dist

    parts = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(parts, out.contiguous(), group=group)
    full = torch.empty((B, q.shape[1], H, q.shape[3]), dtype=out.dtype, device=out.device)
    for r, part in enumerate(parts):
        s = plan_shard(B, H, k.shape[2], r, world)
        full[s.batch[0]:s.batch[1], :, s.q_heads[0]:s.q_heads[1]] = part
    return full
