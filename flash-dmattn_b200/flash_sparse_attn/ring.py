"""KV-ring context parallelism for ONE long sequence spread over the GPUs of a node.

Use when (batch x kv-head) units cannot be sharded (e.g. B = 1, one kv head, S >= 128k): every rank keeps a slice
of the queries and the K/V (+ query-broadcast bias and mask) slices travel around a ring of `torch.distributed`
point-to-point transfers (NCCL over NVLink; one process per GPU). The reference has no multi-GPU path; the merge rule
is the one its split-KV combine kernel uses (csrc/flash_sparse_attn/src/flash_fwd_kernel.h:1695-1727).

Layout ("zig-zag"): the sequence is cut into 2P chunks of C tokens; rank r owns chunks r and 2P-1-r, so under a
causal mask every rank has the same amount of visible work. A (query chunk i, key chunk j) pair is fully visible
(j < i), diagonal (i == j: causal inside the chunk) or invisible (j > i); non-causal attention sees every pair.

Forward: P steps. In step s a rank holds the K/V/bias/mask chunks of rank (r - s) mod P, runs the single-GPU
operator on each visible pair and folds the partial (O, LSE) into its running result
    LSE' = logaddexp(LSE, LSE_p),  O' = exp(LSE - LSE') O + exp(LSE_p - LSE') O_p,
while the next step's chunks are already in flight. Backward: the same rotation, with fp32 dK/dV/dBias accumulators
travelling alongside their chunks; each pair calls the single-GPU backward with the GLOBAL O and LSE of the query
chunk (P = exp(S - LSE) and D = rowsum(dO o O) are then exact), and one extra hop brings the accumulators home.
"""
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------------------------
# zig-zag layout helpers
# ------------------------------------------------------------------------------------------------------------
def zigzag_chunks(rank: int, world: int) -> Tuple[int, int]:
    """The two chunk indices (of 2*world) that `rank` owns."""
    return rank, 2 * world - 1 - rank


def zigzag_split(t: torch.Tensor, dim: int, rank: int, world: int) -> torch.Tensor:
    """Local slice (2 chunks concatenated along `dim`) of a full-sequence tensor."""
    n = t.shape[dim]
    if n % (2 * world):
        raise ValueError(f"sequence length {n} must be a multiple of 2 * world_size = {2 * world}")
    c = n // (2 * world)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([t.narrow(dim, a * c, c), t.narrow(dim, b * c, c)], dim=dim)


def zigzag_merge(parts: List[torch.Tensor], dim: int) -> torch.Tensor:
    """Inverse of zigzag_split over the list of all ranks' local tensors."""
    world = len(parts)
    c = parts[0].shape[dim] // 2
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = zigzag_chunks(r, world)
        chunks[a], chunks[b] = p.narrow(dim, 0, c), p.narrow(dim, c, c)
    return torch.cat(chunks, dim=dim)


# ------------------------------------------------------------------------------------------------------------
# single-GPU compute, replaceable for CPU tests
# ------------------------------------------------------------------------------------------------------------
def _default_fwd(q, k, v, mask, bias, scale, causal):
    out, lse, _ = torch.ops.flash_sparse_attn._flash_sparse_attn_forward(q, k, v, mask, bias, scale, causal, 0.0, False)
    return out, lse


def _default_bwd(dout, q, k, v, mask, bias, out, lse, scale, causal):
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dbias = torch.empty_like(bias) if bias is not None else None
    torch.ops.flash_sparse_attn._flash_sparse_attn_backward(
        dout, q, k, v, mask, bias, out, lse, dq, dk, dv, dbias, scale, causal, 0.0, False)
    return dq, dk, dv, dbias


def _chunk_capacity(mask: Optional[torch.Tensor], group, chunk: int, batch: int, heads_k: int) -> Optional[int]:
    """Largest number of kept keys in any chunk of any rank (one all-reduce and one read-back per call), rounded
    up to 128 -- or None when gathering does not apply or would not pay: no mask, CPU tensors, a mask with one row
    per QUERY head (the gathered K/V are shared by the heads of a kv group, so its rows must be per kv head or
    shared), more than 3/4 of a chunk kept."""
    from . import flash_sparse_attn_interface as iface

    if mask is None or not mask.is_cuda or iface._compaction != "auto":
        return None
    if mask.shape[0] not in (1, batch) or mask.shape[1] not in (1, heads_k):
        return None
    counts = mask.reshape(*mask.shape[:2], 2, chunk).sum(dim=-1, dtype=torch.int32).max().reshape(1)
    dist.all_reduce(counts, op=dist.ReduceOp.MAX, group=group)
    cap = max(128, (int(counts.item()) + 127) // 128 * 128)
    return cap if 4 * cap <= 3 * chunk else None


def _pad_keys(t: Optional[torch.Tensor], keys: int) -> Optional[torch.Tensor]:
    """mask / bias key dimension rounded up to a multiple of 128, as the operator expects."""
    if t is None:
        return None
    want = (keys + 127) // 128 * 128
    if t.shape[-1] == want:
        return t
    return torch.nn.functional.pad(t, [0, want - t.shape[-1]])


def _neg_inf_lse(lse: torch.Tensor) -> torch.Tensor:
    """The operator reports rows without a visible key as LSE = +inf; for merging they weigh nothing."""
    return torch.where(torch.isposinf(lse), torch.full_like(lse, float("-inf")), lse)


def _merge_on_device(o_acc, lse_acc, o_p, lse_p) -> bool:
    """Folds the partial into the accumulators IN PLACE with one kernel (fdma_merge_partials). False when the
    tensors do not fit that kernel (CPU tensors, other dtypes or strides): the caller then uses `_merge`."""
    if not (o_acc.is_cuda and o_acc.is_contiguous() and lse_acc.is_contiguous() and lse_p.is_contiguous()):
        return False
    if o_p.dtype not in (torch.bfloat16, torch.float16) or o_p.stride(-1) != 1 or o_p.shape[-1] % 8 or o_p.shape[-1] > 256:
        return False
    if any(st % 8 for st in o_p.stride()[:3]) or o_p.data_ptr() % 16:
        return False
    import ctypes

    from . import _lib

    B, Sq, H, d = o_p.shape
    mp = _lib.MergeParams()
    mp.acc, mp.lse_acc, mp.part, mp.lse_part = o_acc.data_ptr(), lse_acc.data_ptr(), o_p.data_ptr(), lse_p.data_ptr()
    mp.part_batch_stride, mp.part_row_stride, mp.part_head_stride = o_p.stride()[:3]
    mp.b, mp.seqlen_q, mp.h, mp.d = B, Sq, H, d
    mp.dtype = _lib.FDMA_BF16 if o_p.dtype == torch.bfloat16 else _lib.FDMA_FP16
    with torch.cuda.device(o_acc.device):
        _lib.check(_lib.load().fdma_merge_partials(ctypes.byref(mp), torch.cuda.current_stream().cuda_stream),
                   "fdma_merge_partials")
    return True


def _merge(o_acc, lse_acc, o_p, lse_p):
    """(B,Sq,H,d) fp32 accumulators with (B,H,Sq) LSE; folds in one partial result."""
    lse_p = _neg_inf_lse(lse_p)
    new = torch.logaddexp(lse_acc, lse_p)
    safe = torch.where(torch.isneginf(new), torch.zeros_like(new), new)
    wa = torch.exp(lse_acc - safe).transpose(1, 2).unsqueeze(-1)
    wp = torch.exp(lse_p - safe).transpose(1, 2).unsqueeze(-1)
    return o_acc * wa + o_p.float() * wp, new


class _Ring:
    """Rotation of a list of tensors by one rank per step, with the transfer of step s+1 overlapping step s."""

    def __init__(self, group, tensors: List[torch.Tensor]):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.cur = [t.contiguous() for t in tensors]
        self.nxt = None
        self.reqs = None

    def start(self):
        """Begins sending the held tensors to rank+1 and receiving the next ones from rank-1."""
        if self.world == 1:
            return
        send_to = dist.get_global_rank(self.group, (self.rank + 1) % self.world) if self.group is not None else (self.rank + 1) % self.world
        recv_from = dist.get_global_rank(self.group, (self.rank - 1) % self.world) if self.group is not None else (self.rank - 1) % self.world
        self.nxt = [torch.empty_like(t) for t in self.cur]
        ops = []
        for s, r in zip(self.cur, self.nxt):
            ops.append(dist.P2POp(dist.isend, s, send_to, group=self.group))
            ops.append(dist.P2POp(dist.irecv, r, recv_from, group=self.group))
        self.reqs = dist.batch_isend_irecv(ops)

    def finish(self):
        """Waits for the transfer begun by start() and makes the received tensors current."""
        if self.world == 1:
            return
        for req in self.reqs:
            req.wait()
        self.cur, self.nxt, self.reqs = self.nxt, None, None


def _visible_pairs(q_chunks, k_chunks, causal):
    """Yields (q_slot, k_slot, diagonal) for the visible (query chunk, key chunk) pairs of one ring step."""
    for qs, qi in enumerate(q_chunks):
        for ks, kj in enumerate(k_chunks):
            if not causal or kj < qi:
                yield qs, ks, False
            elif kj == qi:
                yield qs, ks, True


class RingAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, bias, softmax_scale, is_causal, group, fwd_fn, bwd_fn):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        B, S2, H, d = q.shape
        C = S2 // 2
        if S2 % 2 or k.shape[1] != S2:
            raise ValueError("local q/k/v must hold two equally long chunks of the sequence")
        for t in (mask, bias):
            if t is not None and (t.dim() != 4 or t.shape[2] != 1 or t.shape[3] != S2):
                raise ValueError("ring attention takes query-broadcast mask/bias of local key length: (B|1, h, 1, 2C)")
        scale = d ** -0.5 if softmax_scale is None else softmax_scale
        causal = bool(is_causal)
        cap = None  # slots per visiting chunk when the pairs run over gathered keys (compaction.py)
        if fwd_fn is _default_fwd and bwd_fn is _default_bwd and d % 8 == 0:
            cap = _chunk_capacity(mask, group, C, B, k.shape[2])
        if cap is not None:
            from . import compaction
        payload = [torch.stack([k, v])]
        if bias is not None:
            payload.append(bias)
        if mask is not None:
            payload.append(mask.to(torch.uint8))
        ring = _Ring(group, payload)
        o_acc = [torch.zeros((B, C, H, d), dtype=torch.float32, device=q.device) for _ in range(2)]
        lse_acc = [torch.full((B, H, C), float("-inf"), dtype=torch.float32, device=q.device) for _ in range(2)]
        q_chunks = zigzag_chunks(rank, world)
        q_loc = [q[:, :C], q[:, C:]]
        for step in range(world):
            if step + 1 < world:
                ring.start()
            src = (rank - step) % world
            kv = ring.cur[0]
            b_cur = ring.cur[1] if bias is not None else None
            m_cur = ring.cur[-1].to(torch.bool) if mask is not None else None
            gathered = {}  # kept keys of a visiting chunk: gathered once, used by both local query chunks
            for qs, ks, diag in _visible_pairs(q_chunks, zigzag_chunks(src, world), causal):
                sl = slice(ks * C, (ks + 1) * C)
                m_p = _pad_keys(m_cur[..., sl] if m_cur is not None else None, C)
                b_p = _pad_keys(b_cur[..., sl] if b_cur is not None else None, C)
                if cap is not None:
                    # a pair is fully visible or the causal diagonal of two equally long chunks, so plain causal
                    # semantics on the chunk's own key positions apply
                    if ks not in gathered:
                        gathered[ks] = compaction.compact_keys(kv[0][:, sl], kv[1][:, sl], m_p, b_p, cap,
                                                               check_capacity=False)
                    o_p, lse_p = compaction.compact_forward(q_loc[qs], gathered[ks], scale, diag)
                else:
                    o_p, lse_p = fwd_fn(q_loc[qs], kv[0][:, sl], kv[1][:, sl], m_p, b_p, scale, diag)
                if not _merge_on_device(o_acc[qs], lse_acc[qs], o_p, lse_p):
                    o_acc[qs], lse_acc[qs] = _merge(o_acc[qs], lse_acc[qs], o_p, lse_p)
            if step + 1 < world:
                ring.finish()
        out = torch.cat(o_acc, dim=1).to(q.dtype)
        lse = torch.cat(lse_acc, dim=2)
        lse = torch.where(torch.isneginf(lse), torch.full_like(lse, float("inf")), lse)  # operator convention
        ctx.save_for_backward(q, k, v, mask, bias, out, lse)
        ctx.scale, ctx.causal, ctx.group, ctx.bwd_fn, ctx.cap = scale, causal, group, bwd_fn, cap
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, mask, bias, out, lse = ctx.saved_tensors
        group, scale, causal, bwd_fn, cap = ctx.group, ctx.scale, ctx.causal, ctx.bwd_fn, ctx.cap
        if cap is not None:
            from . import compaction
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        B, S2, H, d = q.shape
        C = S2 // 2
        dout = dout.contiguous()
        # travelling payload: K/V chunk pair, (bias), (mask), fp32 dK/dV accumulator, (fp32 dBias accumulator)
        payload = [torch.stack([k, v])]
        if bias is not None:
            payload.append(bias)
        if mask is not None:
            payload.append(mask.to(torch.uint8))
        payload.append(torch.zeros((2,) + tuple(k.shape), dtype=torch.float32, device=k.device))
        if bias is not None:
            payload.append(torch.zeros(bias.shape, dtype=torch.float32, device=bias.device))
        ring = _Ring(group, payload)
        dq_acc = [torch.zeros((B, C, H, d), dtype=torch.float32, device=q.device) for _ in range(2)]
        q_chunks = zigzag_chunks(rank, world)
        sl_q = [slice(0, C), slice(C, 2 * C)]
        for step in range(world):
            src = (rank - step) % world
            kv = ring.cur[0]
            b_cur = ring.cur[1] if bias is not None else None
            m_cur = ring.cur[2 if bias is not None else 1].to(torch.bool) if mask is not None else None
            dkv_acc = ring.cur[-2] if bias is not None else ring.cur[-1]
            db_acc = ring.cur[-1] if bias is not None else None
            gathered = {}
            for qs, ks, diag in _visible_pairs(q_chunks, zigzag_chunks(src, world), causal):
                sl = slice(ks * C, (ks + 1) * C)
                b_p = _pad_keys(b_cur[..., sl] if b_cur is not None else None, C)
                m_p = _pad_keys(m_cur[..., sl] if m_cur is not None else None, C)
                lse_q = lse[:, :, sl_q[qs]].contiguous()
                if cap is not None:
                    if ks not in gathered:
                        gathered[ks] = compaction.compact_keys(kv[0][:, sl], kv[1][:, sl], m_p, b_p, cap,
                                                               check_capacity=False)
                    dq_p, dk_p, dv_p, db_p = compaction.compact_backward(
                        dout[:, sl_q[qs]], q[:, sl_q[qs]], gathered[ks], out[:, sl_q[qs]], lse_q, scale, diag,
                        tuple(kv[0][:, sl].shape), tuple(b_p.shape) if b_p is not None else None)
                else:
                    dq_p, dk_p, dv_p, db_p = bwd_fn(
                        dout[:, sl_q[qs]], q[:, sl_q[qs]], kv[0][:, sl], kv[1][:, sl], m_p, b_p,
                        out[:, sl_q[qs]], lse_q, scale, diag)
                dq_acc[qs] += dq_p.float()
                dkv_acc[0][:, sl] += dk_p.float()
                dkv_acc[1][:, sl] += dv_p.float()
                if db_acc is not None:
                    db_acc[..., sl] += db_p[..., :C].float()
            # the accumulators move with their chunks; after the last step one more hop takes them home
            ring.start()
            ring.finish()
        dkv = ring.cur[-2] if bias is not None else ring.cur[-1]
        dbias = ring.cur[-1].to(bias.dtype) if bias is not None else None
        dq = torch.cat(dq_acc, dim=1).to(q.dtype)
        return dq, dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, dbias, None, None, None, None, None


def ring_flash_sparse_attn_func(query, key, value, attn_mask=None, attn_bias=None, softmax_scale=None, is_causal=None,
                                group=None, fwd_fn: Optional[Callable] = None, bwd_fn: Optional[Callable] = None):
    """Context-parallel dynamic-mask attention over the ranks of `group` (default: the world group).

    query, key, value: this rank's zig-zag slice (see zigzag_split), shapes (B, 2C, H, d) / (B, 2C, Hk, d);
    attn_mask (bool) and attn_bias: query-broadcast, ({B|1}, {H|Hk|1}, 1, 2C), sliced like the keys. Masks with
    at most one row per kv head run over each visiting chunk's gathered kept keys; a mask with one row per query
    head runs over the full chunks.
    Returns this rank's slice of the output; gradients flow to query, key, value and attn_bias.
    C must be a multiple of 128."""
    if not dist.is_initialized():
        raise RuntimeError("ring attention needs an initialised torch.distributed process group")
    C = query.shape[1] // 2
    if C % 128:
        raise ValueError("chunk length (local sequence / 2) must be a multiple of 128")
    return RingAttnFunc.apply(query, key, value, attn_mask, attn_bias, softmax_scale, is_causal, group,
                              fwd_fn or _default_fwd, bwd_fn or _default_bwd)
