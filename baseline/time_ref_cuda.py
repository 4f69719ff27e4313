"""Times the reference's own CUDA kernels (the trimmed sm_100 build that baseline/build_ref_cuda.py leaves in
baseline/_ref/) on one batch element of the long-context training shape: B=1, S=32768, Hq=32, Hkv=8, d=128, bf16,
bias (B,Hkv,1,Sk) ~ N(0,1), mask = top-2048 keys per (batch, kv head), causal, forward + backward through the
reference's `flash_sparse_attn_func`. A labelled extra, not bench.py's reference arm: it shows what the unchanged
mma.sync kernels reach on this GPU for the same call.

    python baseline/time_ref_cuda.py [--seq-len 32768] [--window 2048] [--steps 5]

Runs in its own process with ONLY baseline/_ref on the import path (the reference package has the same name as this
repository's). Prints one JSON line; {"unavailable": "..."} if the build is not there."""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--window", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--per-query", action="store_true",
                    help="per-query bias and mask (B,Hkv,Sq,Sk) instead of row-broadcast ones (use --seq-len 8192 "
                         "--window 1024 for the per-query training shape)")
    args = ap.parse_args()
    if not os.path.exists(os.path.join(REF, "flash_sparse_attn_cuda.so")):
        print(json.dumps({"impl": "reference-cuda", "unavailable": "baseline/_ref/flash_sparse_attn_cuda.so not built"}))
        return
    sys.path[:] = [REF] + [p for p in sys.path if p and os.path.abspath(p) not in (os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), "flash-dmattn_b200"))]
    import torch

    try:
        from flash_sparse_attn.flash_sparse_attn_interface import flash_sparse_attn_func
        from flash_sparse_attn.utils.mask import create_mask
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference-cuda", "unavailable": f"import failed: {e!r}"[:300]}))
        return
    dev = torch.device("cuda:0")
    S, W, H, Hk, d = args.seq_len, args.window, 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(1234)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v = rnd(1, S, H, d), rnd(1, S, Hk, d), rnd(1, S, Hk, d)
    bias, dout = rnd(1, Hk, S if args.per_query else 1, S), rnd(1, S, H, d)
    mask = create_mask(bias, None, 1, S, S, W, torch.finfo(torch.bfloat16).min)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True); bias.requires_grad_(True)

    def step():
        out = flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias, is_causal=True)
        out.backward(dout)
        q.grad = k.grad = v.grad = bias.grad = None
        return out

    try:
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            f0.record()
            for _ in range(args.steps):
                flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias, is_causal=True)
            f1.record()
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference-cuda", "unavailable": f"run failed: {e!r}"[:400]}))
        return
    shape = "(B,Hkv,Sq,Sk)" if args.per_query else "(B,Hkv,1,Sk)"
    print(json.dumps({"impl": "reference-cuda", "workload": f"B=1 S={S} W={W} d={d} Hq={H} Hkv={Hk} causal, bias and mask {shape}",
                      "fwd_bwd_ms": e0.elapsed_time(e1) / args.steps, "fwd_ms": f0.elapsed_time(f1) / args.steps,
                      "steps": args.steps, "build": "sm_100, mma.sync kernels unchanged, CUTLASS headers from flashinfer"}))


if __name__ == "__main__":
    main()
