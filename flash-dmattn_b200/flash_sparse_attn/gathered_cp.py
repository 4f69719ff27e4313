"""Context parallelism for ONE long sequence with a row-broadcast dynamic mask, by gathering the kept keys.

When the mask keeps W keys of the whole sequence for every query (one keep-set per kv head), the keys that matter are
few: W rows of K and V, wherever they sit. Instead of rotating all K/V chunks around a ring (ring.py), every rank
  1. learns the global mask (all-gather of the local mask slices: Sk bytes per mask row),
  2. indexes it (ascending global positions of the kept keys) and gathers the kept rows IT OWNS into their slots of
     a (B, Wp, Hk, d) buffer that is zero elsewhere,
  3. all-reduces those buffers (K, V, bias): every slot is non-zero on exactly one rank, so the sum is the gathered
     tensor, a few MiB,
  4. runs the single-GPU kernels for each of its query chunks over the gathered keys, the causal test on global
     positions (key visible iff key_pos <= chunk offset + local row),
and in the backward pass all-reduces the gradients of the gathered tensors in fp32 and scatters the slots it owns
back into its local dK / dV / dBias. Two small collectives forward, one backward, nothing proportional to Sk*d.

Layout of the local tensors is the zig-zag layout of ring.py: rank r holds chunks r and 2P-1-r of 2P.
The reference has no multi-GPU path. The collectives are torch.distributed (NCCL over NVLink; one process per GPU).
The device work goes through an `ops` object so that the rank logic can run under gloo on CPU with a plain torch
implementation of the same five operations (tests/test_gathered_cp_gloo.py).
"""
from typing import Optional

import torch
import torch.distributed as dist

from .ring import zigzag_chunks, zigzag_merge

__all__ = ["gathered_cp_flash_sparse_attn_func", "CudaOps"]

_INT_MAX = 2**31 - 1


class CudaOps:
    """The five device operations on the kernels of this package (flash_sparse_attn/compaction.py)."""

    def index(self, mask_rows: torch.Tensor, capacity: int):
        from . import compaction

        key_pos, _, mask_c = compaction.index_kept_keys(mask_rows.contiguous(), capacity, check_capacity=False)
        return key_pos, mask_c

    def gather(self, key, value, bias, key_pos):
        from . import compaction

        return compaction.gather_kept_keys(key, value, bias, key_pos)

    def scatter(self, src_c, key_pos, rows_full, bias_layout=False):
        from . import compaction

        return compaction.scatter_kept_rows(src_c, key_pos, rows_full, bias_layout)

    def _ck(self, k_c, v_c, mask_c, bias_c, key_pos, seqlen_k):
        from . import compaction

        return compaction.CompactKeys(k_c, v_c, mask_c, bias_c, key_pos, None, seqlen_k)

    def forward(self, q, k_c, v_c, mask_c, bias_c, key_pos, shift, scale, causal, seqlen_k):
        from . import compaction

        return compaction.compact_forward(q, self._ck(k_c, v_c, mask_c, bias_c, key_pos, seqlen_k), scale, causal, shift)

    def backward(self, dout, q, k_c, v_c, mask_c, bias_c, key_pos, shift, out, lse, scale, causal, seqlen_k):
        from . import compaction

        return compaction.compact_backward(dout, q, self._ck(k_c, v_c, mask_c, bias_c, key_pos, seqlen_k), out, lse,
                                           scale, causal, None, None, causal_shift=shift, scatter=False)


def _all_gather(t: torch.Tensor, group) -> list:
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, t.contiguous(), group=group)
    return parts


class _GatheredCPFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, bias, softmax_scale, is_causal, group, ops):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        B, S2, H, d = q.shape
        Hk = k.shape[2]
        C = S2 // 2
        if S2 % 2 or k.shape[1] != S2:
            raise ValueError("local q/k/v must hold two equally long chunks of the sequence")
        if mask is None or mask.dim() != 4 or mask.shape[2] != 1 or mask.shape[3] != S2 or mask.shape[1] not in (1, Hk):
            raise ValueError("needs a row-broadcast mask of local key length: ({B|1}, {Hk|1}, 1, 2C)")
        if bias is not None and (bias.dim() != 4 or bias.shape[2] != 1 or bias.shape[3] != S2):
            raise ValueError("needs a row-broadcast bias of local key length: ({B|1}, {H|Hk|1}, 1, 2C)")
        scale = d ** -0.5 if softmax_scale is None else softmax_scale
        causal = bool(is_causal)
        S = 2 * C * world
        a, b = zigzag_chunks(rank, world)

        # 1. the global mask, in sequence order, and the positions of its kept keys
        gmask = zigzag_merge([p.to(torch.bool) for p in _all_gather(mask.to(torch.uint8), group)], 3)
        kept = int(gmask.sum(dim=-1, dtype=torch.int32).max().item())
        cap = max(128, (kept + 127) // 128 * 128)
        key_pos, mask_c = ops.index(gmask[:, :, 0], cap)            # (Bm,Hm,cap) global positions, ascending
        # 2. the slots this rank owns, as positions inside its local [chunk a | chunk b] tensors
        chunk = torch.div(key_pos, C, rounding_mode="floor")
        pos_local = torch.where(chunk == a, key_pos - a * C,
                                torch.where(chunk == b, key_pos - b * C + C, torch.full_like(key_pos, _INT_MAX)))
        pos_local = pos_local.to(torch.int32).contiguous()
        k_c, v_c, bias_c = ops.gather(k, v, bias, pos_local)
        # 3. every slot is non-zero on exactly one rank: the sum is the gathered tensor
        for t in (k_c, v_c) + ((bias_c,) if bias_c is not None else ()):
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        # 4. attention of the local query chunks over the gathered keys
        if causal:
            res = [ops.forward(q[:, i * C:(i + 1) * C], k_c, v_c, mask_c, bias_c, key_pos, c * C, scale, True, S)
                   for i, c in enumerate((a, b))]
            out = torch.cat([r[0] for r in res], dim=1)
            lse = torch.cat([r[1] for r in res], dim=2)
        else:
            out, lse = ops.forward(q, k_c, v_c, mask_c, bias_c, key_pos, 0, scale, False, S)
        saved = [q, k_c, v_c, mask_c, key_pos, pos_local, out, lse] + ([bias_c] if bias_c is not None else [])
        ctx.save_for_backward(*saved)
        ctx.meta = (scale, causal, group, ops, C, S, (a, b), tuple(bias.shape) if bias is not None else None, k.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        saved = ctx.saved_tensors
        q, k_c, v_c, mask_c, key_pos, pos_local, out, lse = saved[:8]
        bias_c = saved[8] if len(saved) > 8 else None
        scale, causal, group, ops, C, S, (a, b), bias_shape, kv_dtype = ctx.meta
        dout = dout.contiguous()
        if causal:
            parts = [ops.backward(dout[:, i * C:(i + 1) * C], q[:, i * C:(i + 1) * C], k_c, v_c, mask_c, bias_c, key_pos,
                                  c * C, out[:, i * C:(i + 1) * C], lse[:, :, i * C:(i + 1) * C].contiguous(), scale,
                                  True, S) for i, c in enumerate((a, b))]
            dq = torch.cat([p[0] for p in parts], dim=1)
        else:
            parts = [ops.backward(dout, q, k_c, v_c, mask_c, bias_c, key_pos, 0, out, lse, scale, False, S)]
            dq = parts[0][0]
        # gradients of the gathered tensors: fp32 sum over the local query chunks, then over the ranks
        tot = [sum(p[j].float() for p in parts) if parts[0][j] is not None else None for j in (1, 2, 3)]
        for t in tot:
            if t is not None:
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        dk = ops.scatter(tot[0].to(kv_dtype), pos_local, 2 * C)
        dv = ops.scatter(tot[1].to(kv_dtype), pos_local, 2 * C)
        dbias = None
        if tot[2] is not None:
            full = ops.scatter(tot[2].to(kv_dtype), pos_local, 2 * C, bias_layout=True)
            for dim in (0, 1):  # dimensions the bias broadcast over (the gather widened them) are summed back
                if bias_shape[dim] == 1 and full.shape[dim] != 1:
                    full = full.sum(dim=dim, keepdim=True, dtype=torch.float32).to(kv_dtype)
            dbias = full
        return dq, dk, dv, None, dbias, None, None, None, None


def gathered_cp_flash_sparse_attn_func(query, key, value, attn_mask, attn_bias=None, softmax_scale=None,
                                       is_causal=None, group=None, ops=None):
    """query (B, 2C, H, d); key, value (B, 2C, Hk, d): this rank's two zig-zag chunks of the sequence;
    attn_mask bool ({B|1}, {Hk|1}, 1, 2C) and attn_bias ({B|1}, {H|Hk|1}, 1, 2C): the local key slices of a
    row-broadcast mask / bias. Returns the local (B, 2C, H, d) output; gradients flow to query, key, value and
    attn_bias. The result equals single-device `flash_sparse_attn_func` on the whole sequence."""
    if group is None:
        group = dist.group.WORLD
    return _GatheredCPFunc.apply(query, key, value, attn_mask, attn_bias, softmax_scale, is_causal, group,
                                 ops if ops is not None else CudaOps())
