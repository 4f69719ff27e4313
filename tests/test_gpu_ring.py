"""KV-ring context parallelism on real GPUs (needs at least two): NCCL ranks as child processes, tcgen05 kernels
underneath (each chunk pair over its full key range, and with the kept keys of the visiting chunk gathered first),
compared with the fp32 oracle on the full sequence."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, causal, route, d, scheme="ring", per_query_head=False):
    import torch.distributed as dist

    from flash_sparse_attn import flash_sparse_attn_interface as iface
    from flash_sparse_attn import ring
    from oracle import oracle

    iface.set_compaction(route)

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, H, Hk = 1, 4, 1
        S = 2 * world * 256
        q, k, v, bias, dout = oracle.make_inputs(B, S, S, H, Hk, d, (B, H if per_query_head else Hk, 1, S), seed=5,
                                                 dtype=torch.bfloat16)
        mask = oracle.create_mask(bias, None, B, S, S, S // 4, torch.finfo(torch.bfloat16).min)
        want = oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, causal)
        loc = lambda t, dim: ring.zigzag_split(t, dim, rank, world).contiguous().to(dev)
        ql, kl, vl = (loc(t, 1).requires_grad_(True) for t in (q, k, v))
        bl = loc(bias, 3).requires_grad_(True)
        if scheme == "ring":
            out = ring.ring_flash_sparse_attn_func(ql, kl, vl, loc(mask, 3), bl, None, causal)
        else:
            from flash_sparse_attn import gathered_cp

            out = gathered_cp.gathered_cp_flash_sparse_attn_func(ql, kl, vl, loc(mask, 3), bl, None, causal)
        out.backward(loc(dout, 1))

        def gather(t, dim):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            return ring.zigzag_merge(parts, dim).float().cpu()

        for name, got, ref, dim in (("out", out, want[0], 1), ("dq", ql.grad, want[2], 1), ("dk", kl.grad, want[3], 1),
                                    ("dv", vl.grad, want[4], 1), ("dbias", bl.grad, want[5], 3)):
            r = oracle.error_report(name, gather(got, dim), ref)
            # under the ring dQ too is a sum: one 16-bit partial per visited chunk pair, added in fp32
            ok, msg = oracle.within_tolerance(r, name in ("dq", "dk", "dv", "dbias"))
            assert ok, msg
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal,route,d", [
    (True, "off", 128), (False, "off", 128), (True, "auto", 128), (False, "auto", 128),
    (True, "auto", 256),   # head dim 256: tcgen05 forward and two-pass backward under the ring
], ids=["causal-tiles", "full-tiles", "causal-compaction", "full-compaction", "causal-compaction-d256"])
def test_ring_two_gpus(causal, route, d):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, causal, route, d), nprocs=2, join=True)


def test_ring_two_gpus_mask_per_query_head():
    """A mask / bias with one row per QUERY head cannot share gathered K/V inside a kv group: the ring must take the
    full-range kernels for it even with gathering enabled, and still match the oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, True, "auto", 128, "ring", True), nprocs=2, join=True)


@pytest.mark.parametrize("causal,d", [(True, 128), (False, 128), (True, 256)])
def test_gathered_keys_context_parallel_two_gpus(causal, d):
    """The same check for the gathered-keys scheme (all-reduce of the kept K/V rows instead of a ring)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, causal, "auto", d, "gathered"), nprocs=2, join=True)
