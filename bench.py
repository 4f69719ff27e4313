"""Headline benchmark: forward+backward dynamic-mask attention, TFLOP/s on kept blocks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch-per-gpu B]

Workload (the long-context training shape the headline metric is quoted on): S = Sq = Sk = 32768, top-2048 mask per
(batch, kv head) from a query-broadcast bias (B,Hkv,1,Sk) ~ N(0,1), causal, Hq = 32, Hkv = 8, d = 128, bf16,
dOut ~ N(0,1), seeded synthetic data. One batch element per GPU (8 independent (batch, kv-head) units); with N GPUs
the global batch is N, sharded over ranks with no collective in the data path (weak scaling).

A step = one forward + one backward through the C ABI, the same sequence of calls flash_sparse_attn_func makes
for this mask shape: fdma_gather_rows (K, V, bias) at the positions create_mask wrote, fdma_fwd, fdma_bwd,
fdma_scatter_rows (dK, dV, dBias). The mask is row-broadcast, so the library gathers the kept keys first and the attention kernels
run over W instead of Sk keys (--compaction off times fdma_fwd + fdma_bwd over the full key range; the default
run reports that too, as `tile_path`). create_mask is outside the timed region, as in the reference's benchmarks
(benchmarks/forward_performance.py:185-204). FLOPs are counted only on the tiles the kernels really process, of
the tile shape each kernel uses, from the actual mask (4*d*BM*BN per forward tile, 10*d*BM*BN per backward tile);
both arms use the same count. `value` has inputs resident in HBM; `e2e` goes through flash_sparse_attn_func with
pinned host buffers, copying inputs up and results back inside the timed region.

--impl reference times the reference's eager algorithm (the CPU oracle port, oracle/oracle.py) on the host cores
on a bounded sample of the same workload.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "flash-dmattn_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

S, HQ, HKV, D, WINDOW = 32768, 32, 8, 128, 2048
WORKLOAD = "S=32768 W=2048 d=128 Hq=32 Hkv=8 causal, bias (B,Hkv,1,Sk), B=1 per GPU"


def set_geometry(seq_len: int, window: int, head_dim: int = 128):
    """Other sequence lengths and head dims exist for profiler captures only; the reported benchmark uses the
    defaults."""
    global S, WINDOW, D, WORKLOAD
    S, WINDOW, D = seq_len, window, head_dim
    WORKLOAD = f"S={S} W={WINDOW} d={D} Hq=32 Hkv=8 causal, bias (B,Hkv,1,Sk), B=1 per GPU"


FWD_TILE, BWD_TILE = (128, 128), (64, 128)
NOMINAL_TFLOPS = 2250.0


def workload_config(world: int, batch_per_gpu: int, compaction: str) -> dict:
    """The `config` object of the JSON line; both arms (ours and --impl reference) print exactly this."""
    compact = compaction == "auto"
    return {"workload": WORKLOAD, "global_batch": batch_per_gpu * world, "seq_len": S, "window": WINDOW,
            "parallelism": f"(batch x kv-head) units sharded over {world} GPU(s), no collective",
            "l2": "inputs larger than L2 (Q alone is 256 MiB per batch element)",
            "route": ("gathered kept keys (key compaction)" if compact else "full key range with tile skipping (tile-OR)"),
            "key_compaction": compaction,
            "flops": ("tiles of the gathered kept keys that the kernels process" if compact
                      else "tiles of the full key range that hold a kept key"),
            "tiles": {"fwd": list(FWD_TILE), "bwd": list(BWD_TILE)}}


def metric_name(compaction: str) -> str:
    return ("fwd+bwd TFLOP/s on kept blocks (gathered-keys route)" if compaction == "auto"
            else "fwd+bwd TFLOP/s on kept blocks (tile-OR route)")


# ------------------------------------------------------------------------------------------------------------
# FLOP accounting on kept tiles (host side, from the actual mask)
# ------------------------------------------------------------------------------------------------------------
def kept_tiles_rowbcast(mask_row: torch.Tensor, Sq: int, Sk: int, bm: int, bn: int, causal: bool,
                        compact: bool = False) -> int:
    """Number of (bm x bn) tiles holding at least one kept, causally visible element, for a mask that is the
    same for every query row. mask_row: bool (Sk,). compact: key tiles are runs of bn consecutive KEPT keys (the
    gathered layout) instead of bn consecutive key positions."""
    mt = (Sq + bm - 1) // bm
    big = Sk + Sq + 1
    if compact:
        pos = torch.nonzero(mask_row[:Sk]).flatten()
        kmin = pos[::bn]                                        # first position of each gathered key tile
        nt = kmin.numel()
        if nt == 0:
            return 0
    else:
        nt = (Sk + bn - 1) // bn
        idx = torch.arange(Sk, device=mask_row.device)
        first = torch.where(mask_row[:Sk], idx, torch.full_like(idx, big))
        pad = nt * bn - Sk
        if pad:
            first = torch.cat([first, torch.full((pad,), big, device=first.device, dtype=first.dtype)])
        kmin = first.view(nt, bn).amin(dim=1)                   # first kept key of each key tile
    last_row = torch.clamp((torch.arange(mt, device=mask_row.device) + 1) * bm - 1, max=Sq - 1)
    limit = last_row + (Sk - Sq) if causal else torch.full_like(last_row, big - 1)
    return int((kmin.view(1, nt) <= limit.view(mt, 1)).sum().item())


def count_flops(mask: torch.Tensor, B: int, Sq: int, Sk: int, H: int, Hk: int, d: int, causal: bool,
                compact: bool = False) -> dict:
    """mask (B,Hk,1,Sk) bool. Returns FLOPs per pass under the accounting rules of the metric, for the full-range
    (compact=False) or the gathered-keys (compact=True) tiling."""
    G = H // Hk
    kept_f = kept_b = kept_c = 0
    for b in range(B):
        for hk in range(Hk):
            row = mask[b, hk, 0]
            kept_f += G * kept_tiles_rowbcast(row, Sq, Sk, *FWD_TILE, causal, compact)
            kept_b += G * kept_tiles_rowbcast(row, Sq, Sk, *BWD_TILE, causal, compact)
            kept_c += G * kept_tiles_rowbcast(row, Sq, Sk, 128, 128, causal, compact)
    # element level: kept, causally visible (query, key) pairs
    nnz = 0
    for b in range(B):
        for hk in range(Hk):
            pos = torch.nonzero(mask[b, hk, 0, :Sk]).flatten()
            vis = (Sq - torch.clamp(pos - (Sk - Sq), min=0)) if causal else torch.full_like(pos, Sq)
            nnz += G * int(torch.clamp(vis, min=0).sum().item())
    mt, nt = (Sq + 127) // 128, (Sk + 127) // 128
    causal_tiles = sum(min(nt, max(0, ((i + 1) * 128 + Sk - Sq + 127) // 128)) for i in range(mt)) if causal else mt * nt
    fwd = 4 * d * FWD_TILE[0] * FWD_TILE[1] * kept_f
    bwd = 10 * d * BWD_TILE[0] * BWD_TILE[1] * kept_b
    return {
        "fwd": fwd, "bwd": bwd, "total": fwd + bwd,
        "canonical_128x128": 14 * d * 128 * 128 * kept_c,
        "causal_dense": 14 * d * 128 * 128 * causal_tiles * B * H,
        "element_level": 14 * d * nnz,
    }


# ------------------------------------------------------------------------------------------------------------
# clocks sampler
# ------------------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi polled every 10 ms from before the warm-up until the timed region ends (the tool needs a few
    hundred ms before its first sample, longer than a short timed region). The summary takes the samples between
    `mark()` (start of the timed region, minus the warm-up that directly precedes it) and stop()."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.t_region = None

    def mark(self):
        self.t_region = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "10",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        in_region = 0
        for t_line, ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            if self.t_region is not None and t_line >= self.t_region:
                in_region += 1
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "samples": len(sm),
            "samples_in_timed_region": in_region,
            "window": "warm-up + timed region",
            "reasons": sorted(reasons),
        }


# ------------------------------------------------------------------------------------------------------------
# CPU legs (oracle port of the reference's eager path)
# ------------------------------------------------------------------------------------------------------------
CPU_ROWS = 1024  # query rows of the bounded CPU sample (the last rows of the sequence: full causal extent)


def cpu_sample(steps: int, warmup: int, compact: bool = True, budget_s: float = 1e9) -> dict:
    """Eager fp32 forward+backward of ONE kv head (its 4 query heads) x the last CPU_ROWS query rows against
    all 32768 keys, timed on all host cores; FLOPs counted on that slice's kept 128x128 tiles. Runs `warmup` untimed
    and `steps` timed passes, stopping early (never before one timed pass) once `budget_s` seconds have gone by."""
    from oracle import oracle

    # torchrun exports OMP_NUM_THREADS=1 to its workers: take every host core regardless
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    G = HQ // HKV
    q, k, v, bias, dout = oracle.make_inputs(1, CPU_ROWS, S, G, 1, D, (1, 1, 1, S), seed=0, dtype=torch.bfloat16)
    mask = oracle.create_mask(bias, None, 1, CPU_ROWS, S, WINDOW, torch.finfo(torch.bfloat16).min)
    flops = count_flops(mask, 1, CPU_ROWS, S, G, 1, D, True, compact)
    times, warm_run = [], 0
    t_begin = time.perf_counter()
    for it in range(warmup + steps):
        timed = it >= warmup
        over = time.perf_counter() - t_begin > budget_s
        if over and times:
            break
        if over:
            timed = True  # the budget ran out during the warm-up: the next pass is the timed one
        t0 = time.perf_counter()
        oracle.attention_forward_backward(q, k, v, mask, bias, dout, None, True)
        if timed:
            times.append(time.perf_counter() - t0)
        else:
            warm_run += 1
    sec = sum(times) / len(times)
    flop_ref = flops["canonical_128x128"]
    return {
        "value": flop_ref / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"1 kv head x {G} query heads x last {CPU_ROWS} query rows x {S} keys, fp32 eager, "
                  f"{sec * 1e3:.0f} ms per fwd+bwd, FLOPs on 128x128 tiles of "
                  f"{'the gathered kept keys' if compact else 'the full key range'}",
        "ms_per_step": sec * 1e3, "steps_run": len(times), "warmup_run": warm_run,
    }


def run_reference(args, rank: int, world: int):
    """The reference's eager algorithm on the host cores (rank 0 only; the other ranks exit without work). Each step is
    a bounded sample of the workload (see cpu_sample); --steps / --warmup are honoured up to a two-minute budget, and
    the line reports how many ran."""
    if rank != 0:
        return
    cb = cpu_sample(max(1, args.steps), max(0, args.warmup), args.compaction == "auto", budget_s=120.0)
    line = {
        "impl": "reference", "metric": metric_name(args.compaction), "value": cb["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "steps_run": cb["steps_run"],
        "warmup_run": cb["warmup_run"], "ms_per_step": cb["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus, args.batch_per_gpu, args.compaction),
        "note": "reference eager algorithm (CPU oracle port) on the host cores, bounded sample per step",
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------------
class AttentionStep:
    """Pre-allocated buffers and pre-filled C-ABI parameter blocks for one forward + backward of the workload, over
    the full key range (compact=False: fdma_fwd, fdma_bwd) or over the gathered kept keys (compact=True: the eight
    calls flash_sparse_attn_func makes for a row-broadcast mask whose position list create_mask has written)."""

    def __init__(self, lib, dev, q, k, v, mask, bias, dout, compact: bool, packed=None):
        from flash_sparse_attn import _lib, compaction
        from flash_sparse_attn import flash_sparse_attn_interface as iface

        self.lib, self._lib, self.compact = lib, _lib, compact
        self.stream = torch.cuda.current_stream(dev)
        B, Sq, H, d = q.shape
        Sk, Hk = k.shape[1], k.shape[2]
        self.out = torch.empty_like(q)
        self.lse = torch.empty((B, H, Sq), dtype=torch.float32, device=dev)
        self.dq, self.dk, self.dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        self.dbias = torch.empty_like(bias)
        self.pre, self.post = [], []  # (function, parameter block) run before the forward / after the backward
        kk, vv, mm, bb, dkk, dvv, dbb = k, v, mask, bias, self.dk, self.dv, self.dbias
        if compact:
            # the position list create_mask wrote with the bool mask (the mask itself is not read again)
            kept = iface._cached_kept_keys(mask, Sk)
            assert kept is not None, "create_mask left no position list on the mask"
            self.key_pos = kept.key_pos
            cap = self.key_pos.shape[-1]
            mm = kept.slot_mask
            kk, vv = (torch.empty((B, cap, Hk, d), dtype=q.dtype, device=dev) for _ in range(2))
            bb = torch.empty((bias.shape[0], bias.shape[1], 1, cap), dtype=q.dtype, device=dev)
            dkk, dvv, dbb = torch.empty_like(kk), torch.empty_like(vv), torch.empty_like(bb)
            bst = lambda t: (t.stride(0), 1, t.stride(1))  # a (B, H, 1, keys) bias as rows of one element
            for src, dst in ((k, kk), (v, vv)):
                self.pre.append((lib.fdma_gather_rows, compaction._rows_params(
                    src, dst, self.key_pos, B, Hk, Sk, cap, d, iface._bsh(src), iface._bsh(dst))))
            self.pre.append((lib.fdma_gather_rows, compaction._rows_params(
                bias, bb, self.key_pos, bias.shape[0], bias.shape[1], Sk, cap, 1, bst(bias), bst(bb))))
            for src, dst in ((dkk, self.dk), (dvv, self.dv)):
                self.post.append((lib.fdma_scatter_rows, compaction._rows_params(
                    src, dst, self.key_pos, B, Hk, Sk, cap, d, iface._bsh(src), iface._bsh(dst))))
            self.post.append((lib.fdma_scatter_rows, compaction._rows_params(
                dbb, self.dbias, self.key_pos, bias.shape[0], bias.shape[1], Sk, cap, 1, bst(dbb), bst(self.dbias))))
        self.keep = (kk, vv, mm, bb, dkk, dvv, dbb, packed)
        self.fp = _lib.FwdParams()
        self.bp = _lib.BwdParams()
        for p in (self.fp, self.bp.f):
            iface._fill_fwd(p, q, kk, vv, mm, bb, self.out, self.lse, d ** -0.5, True)
            if packed is not None:  # the mask as one bit per key + tile activity (flash_sparse_attn.packed)
                p.mask, p.mask_bits, p.h_mask = packed.bits.data_ptr(), 1, packed.bits.shape[1]
                p.mask_batch_stride, p.mask_head_stride, p.mask_row_stride = packed.bits.stride()[:3]
                p.tile_activity = packed.activity.data_ptr()
            if compact:
                p.key_pos, p.key_pos_batch_stride = self.key_pos.data_ptr(), self.key_pos.stride(0)
                p.key_pos_head_stride, p.h_pos, p.causal_shift = self.key_pos.stride(1), self.key_pos.shape[1], Sk - Sq
        bp = self.bp
        bp.dout = dout.data_ptr()
        bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride = iface._bsh(dout)
        bp.dq, bp.dk, bp.dv, bp.dbias = self.dq.data_ptr(), dkk.data_ptr(), dvv.data_ptr(), dbb.data_ptr()
        bp.dq_batch_stride, bp.dq_row_stride, bp.dq_head_stride = iface._bsh(self.dq)
        bp.dk_batch_stride, bp.dk_row_stride, bp.dk_head_stride = iface._bsh(dkk)
        bp.dv_batch_stride, bp.dv_row_stride, bp.dv_head_stride = iface._bsh(dvv)
        bp.dbias_batch_stride, bp.dbias_head_stride, bp.dbias_row_stride = dbb.stride()[:3]
        bp.dbias_b, bp.dbias_h, bp.dbias_rows, bp.dbias_keys = dbb.shape
        if compact:  # workspace sizes depend on the positions only through their presence
            self.run_pre()
        ws_f = lib.fdma_fwd_workspace_bytes(ctypes.byref(self.fp))
        ws_b = lib.fdma_bwd_workspace_bytes(ctypes.byref(bp))
        self.ws = torch.empty(max(ws_f, ws_b, 1), dtype=torch.uint8, device=dev)
        self.fp.workspace, self.fp.workspace_bytes = self.ws.data_ptr(), ws_f
        bp.f.workspace, bp.f.workspace_bytes = self.ws.data_ptr(), ws_b
        # launches per step, from the code paths above: gathers 3 | fwd_kernel 1 | bwd_prep, bwd_kernel,
        # convert_dq 3 (+ 3 partial reductions when the backward grid is split) | scatters 3 (their zero fills are memsets)
        self.launches = (3 + 1 + 6 + 3) if compact else 4

    def run_pre(self):
        for fn, prm in self.pre:
            self._lib.check(fn(ctypes.byref(prm), self.stream.cuda_stream), "compaction")

    def __call__(self, ev=None):
        lib, st = self.lib, self.stream.cuda_stream
        self.run_pre()
        if ev is not None:
            lib.fdma_time_next_kernel(ev[0].cuda_event, ev[1].cuda_event)
        self._lib.check(lib.fdma_fwd(ctypes.byref(self.fp), st), "fdma_fwd")
        if ev is not None:
            lib.fdma_time_next_kernel(ev[2].cuda_event, ev[3].cuda_event)
        self._lib.check(lib.fdma_bwd(ctypes.byref(self.bp), st), "fdma_bwd")
        for fn, prm in self.post:
            self._lib.check(fn(ctypes.byref(prm), st), "scatter")


def time_steps(step, steps: int, stream, barrier):
    """K steps between two events on the launching stream, barrier + synchronize on both sides; per-step events
    around the forward and the backward attention kernels. Returns (total ms, mean fwd kernel ms, mean bwd kernel
    ms)."""
    kernel_events = []
    for _ in range(steps):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for e in evs:
            e.record(stream)  # materialises the underlying cudaEvent_t
        kernel_events.append(evs)
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record(stream)
    for i in range(steps):
        step(kernel_events[i])
    t_stop.record(stream)
    barrier()
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in kernel_events)
    bwd_ms = statistics.mean(e[2].elapsed_time(e[3]) for e in kernel_events)
    return t_start.elapsed_time(t_stop), fwd_ms, bwd_ms


def load_peak_file() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


def tensor_peaks(sm_mhz) -> dict:
    """Denominators of the tensor-bound roofline: the measured cuBLAS bf16 burst rate while the SM clock sits at or
    above 1800 MHz during the run (a kernel timed in short bursts), the sustained rate otherwise; both are reported."""
    pk = load_peak_file()
    burst = float(pk.get("bf16_tflops", 1590.0))
    sustained = float(pk.get("bf16_tflops_sustained", 1400.0))
    src = "measured" if pk else "fallback"
    use_burst = sm_mhz is None or sm_mhz >= 1800.0
    return {"peak": burst if use_burst else sustained, "burst": burst, "sustained": sustained,
            "source": f"of {src} (cuBLAS bf16, {'burst' if use_burst else 'sustained'})"}


def hbm_peak():
    pk = load_peak_file()
    return float(pk.get("hbm_gbs", 6650.0)), ("of measured (copy)" if pk else "of fallback (copy)")


def chunked_oracle(q, k, v, mask, bias, dout, rows):
    """fp32 oracle on the device, `rows` query rows at a time (causal: a chunk needs the keys up to its last row).
    Checker only, outside every timed region."""
    from oracle import oracle

    B, Sq, H, d = q.shape
    kf, vf, bf = (t.float().requires_grad_(True) for t in (k, v, bias))
    o_ref = torch.empty((B, Sq, H, d), dtype=torch.float32, device=q.device)
    dq_ref = torch.empty_like(o_ref)
    for r0 in range(0, Sq, rows):
        qc = q[:, r0:r0 + rows].float().requires_grad_(True)
        oc, _ = oracle.attention_forward(qc, kf[:, : r0 + rows], vf[:, : r0 + rows], mask[..., : r0 + rows],
                                         bf[..., : r0 + rows], None, True)
        (oc * dout[:, r0:r0 + rows].float()).sum().backward()
        o_ref[:, r0:r0 + rows] = oc.detach()
        dq_ref[:, r0:r0 + rows] = qc.grad
    return o_ref, dq_ref, kf.grad, vf.grad, bf.grad


def reference_cuda_kernels(extra=()) -> dict:
    """The reference's mma.sync kernels, recompiled unchanged for sm_100 (baseline/build_ref_cuda.py), timed on one
    batch element of this workload through the reference's own flash_sparse_attn_func, in a child process that sees
    only baseline/_ref (baseline/time_ref_cuda.py). Context for `value` and `tile_or`; not the reference arm."""
    script = os.path.join(ROOT, "baseline", "time_ref_cuda.py")
    try:
        cmd = [sys.executable, script, "--steps", "3"] + (list(extra) if extra else
                                                          ["--seq-len", str(S), "--window", str(WINDOW)])
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        return json.loads(lines[-1]) if lines else {"unavailable": (res.stderr or "no output")[-300:]}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:300]}


def parity_report(q, k, v, mask, bias, dout) -> dict:
    """One kv-head group of the timed workload (kv head 0 of batch element 0 with its query heads) through the public
    API, against the fp32 oracle evaluated in chunks of 2048 query rows: per tensor max-abs, mean-abs, the floor that
    one 16-bit rounding of the exact value costs, and the largest error in ulps."""
    from flash_sparse_attn import flash_sparse_attn_func
    from oracle import oracle

    G = HQ // HKV
    qs, ks, vs = q[:1, :, :G].contiguous(), k[:1, :, :1].contiguous(), v[:1, :, :1].contiguous()
    bs, ms, ds = bias[:1, :1].contiguous(), mask[:1, :1].contiguous(), dout[:1, :, :G].contiguous()
    ql, kl, vl, bl = (t.detach().requires_grad_(True) for t in (qs, ks, vs, bs))
    out = flash_sparse_attn_func(ql, kl, vl, attn_mask=ms, attn_bias=bl, is_causal=True)
    out.backward(ds)
    ref = chunked_oracle(qs, ks, vs, ms, bs, ds, 2048)
    rep = {"against": "fp32 oracle, one kv-head group of the timed workload, chunks of 2048 query rows",
           "bounds": {"max_abs": oracle.MAX_ABS, "mean_abs": oracle.MEAN_ABS,
                      "reduced_tensors": f"dk, dv, dbias: + {oracle.FLOOR_FACTOR} x floor_bound (max), "
                                         f"+ {oracle.FLOOR_FACTOR} x floor_mean (mean)"}}
    ok_all = True
    for name, got, want, reduced in zip(("out", "dq", "dk", "dv", "dbias"), (out.detach(), ql.grad, kl.grad, vl.grad, bl.grad),
                                        ref, (False, False, True, True, True)):
        r = oracle.error_report(name, got, want)
        ok, _ = oracle.within_tolerance(r, reduced)
        ok_all = ok_all and ok
        rep[name] = {"max_abs": r["max_abs"], "mean_abs": r["mean_abs"], "floor_max": r["floor_max_abs"],
                     "floor_bound": r["floor_bound"], "floor_mean": r["floor_mean_abs"], "ulp_norm": r["ulp_norm"],
                     "within_bounds": ok}
    rep["green"] = ok_all
    return rep


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist

    from flash_sparse_attn import _lib, flash_sparse_attn_func
    from flash_sparse_attn import flash_sparse_attn_interface as iface
    from flash_sparse_attn.utils.mask import create_mask

    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    lib = _lib.load()
    B = args.batch_per_gpu
    compact = args.compaction == "auto"
    iface.set_compaction(args.compaction)
    # seeded synthetic inputs: Q, K, V, bias, dOut ~ N(0,1) drawn in fp32 then cast to bf16; seed differs per rank
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v = rnd(B, S, HQ, D), rnd(B, S, HKV, D), rnd(B, S, HKV, D)
    bias, dout = rnd(B, HKV, 1, S), rnd(B, S, HQ, D)
    mask = create_mask(bias, None, B, S, S, WINDOW, torch.finfo(torch.bfloat16).min)
    mask_host = mask.cpu()
    flops = count_flops(mask_host, B, S, S, HQ, HKV, D, True, compact)  # on the host: keeps the launch list clean
    stream = torch.cuda.current_stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident timing ----
    step = AttentionStep(lib, dev, q, k, v, mask, bias, dout, compact)
    step_launches = step.launches
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler is not None:
        sampler.start()
    # warm-up: at least W steps, and at least half a second of load so that clocks and the sampler have settled
    t_w = time.time()
    n_w = 0
    while n_w < args.warmup or time.time() - t_w < args.min_warmup_seconds:
        step()
        n_w += 1
        if n_w % 8 == 0:
            torch.cuda.synchronize(dev)
    # the timed region of K steps is taken `repeats` times back to back; the line reports the median region
    barrier()
    if sampler is not None:
        sampler.mark()
    regions = [time_steps(step, args.steps, stream, barrier) for _ in range(max(1, args.repeats))]
    clocks = sampler.stop() if sampler is not None else None
    _lib.check(lib.fdma_last_kernel_status(stream.cuda_stream, None), "kernel status")
    out, dq, dk, dv, dbias = step.out, step.dq, step.dk, step.dv, step.dbias
    med = lambda xs: statistics.median(xs)
    step_ms_all = [r[0] / args.steps for r in regions]
    ms_per_step_local, fwd_ms, bwd_ms = med(step_ms_all), med([r[1] for r in regions]), med([r[2] for r in regions])

    # ---- the same workload over the full key range (tile skipping only), for comparison ----
    tile = None
    if compact and not args.no_tile_path:
        tstep = AttentionStep(lib, dev, q, k, v, mask, bias, dout, False)
        for _ in range(3):
            tstep()
        t_steps = max(1, min(args.steps, 5))
        t_ms, t_fwd, t_bwd = time_steps(tstep, t_steps, stream, barrier)
        t_fl = count_flops(mask_host, B, S, S, HQ, HKV, D, True, False)
        tile = {"ms_per_step": t_ms / t_steps, "fwd_kernel_ms": t_fwd, "bwd_kernel_ms": t_bwd,
                "tflops_on_its_kept_tiles": t_fl["total"] / (t_ms / t_steps * 1e-3) / 1e12,
                "bwd_kernel_tflops": t_fl["bwd"] / (t_bwd * 1e-3) / 1e12,
                "fwd_kernel_tflops": t_fl["fwd"] / (t_fwd * 1e-3) / 1e12,
                "note": "per GPU, rank 0; fdma_fwd + fdma_bwd over all Sk keys, skipping tiles without a kept key; "
                        "never mixed into `value`"}
        _lib.check(lib.fdma_last_kernel_status(stream.cuda_stream, None), "kernel status")
        del tstep

    # ---- the public API on device-resident tensors (allocations, workspaces and the Python layer included) ----
    api_ms = None
    if not args.no_api:
        qa, ka, va, ba = (t.detach().requires_grad_(True) for t in (q, k, v, bias))

        def api_step():
            o = flash_sparse_attn_func(qa, ka, va, attn_mask=mask, attn_bias=ba, is_causal=True)
            o.backward(dout)
            qa.grad = ka.grad = va.grad = ba.grad = None

        for _ in range(3):
            api_step()
        n_api = max(2, min(args.steps, 10))
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for _ in range(n_api):
            api_step()
        a1.record(stream)
        barrier()
        api_ms = a0.elapsed_time(a1) / n_api
        del qa, ka, va, ba

    # ---- parity of the timed workload against the oracle (checker, outside every timed region) ----
    parity = parity_report(q, k, v, mask, bias, dout) if rank == 0 and not args.no_parity else None

    # ---- end to end through the public API with pinned host buffers ----
    # The mask is not an input: as in a model, it is made on the device from the uploaded bias (create_mask, inside
    # the timed region), which also leaves flash_sparse_attn_func the position list it needs to gather keys without
    # a read-back.
    host_in = {n: t.detach().cpu().pin_memory() for n, t in (("q", q), ("k", k), ("v", v), ("bias", bias),
                                                              ("dout", dout))}
    host_out = {n: torch.empty(t.shape, dtype=t.dtype).pin_memory()
                for n, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv), ("dbias", dbias))}
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out.values())

    # Three streams: uploads, compute, downloads. Step i's upload overlaps step i-1's compute and download (PCIe is
    # full duplex); device input buffers and host output buffers come in THREE sets, so that the host only has to wait
    # for the download of step i-3 before it queues the upload of step i (with two sets the upload stream idles for a
    # compute time per step, waiting for the host); every tensor a side stream still reads is kept referenced until
    # that stream's event has completed.
    NB = 3
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    in_names = ("q", "k", "v", "bias", "dout")
    dev_in = [{n: torch.empty_like(host_in[n], device=dev) for n in in_names} for _ in range(NB)]
    host_out2 = [host_out] + [{n: torch.empty_like(t).pin_memory() for n, t in host_out.items()} for _ in range(NB - 1)]
    ev_in = [torch.cuda.Event() for _ in range(NB)]
    ev_comp = [torch.cuda.Event() for _ in range(NB)]
    ev_out = [torch.cuda.Event() for _ in range(NB)]
    live = [None] * NB

    def e2e_step(i: int):
        sl = i % NB
        if i >= NB:
            ev_out[sl].synchronize()      # step i-NB has left the device: its buffers may be reused
            live[sl] = None
        with torch.cuda.stream(s_in):
            if i >= NB:
                s_in.wait_event(ev_comp[sl])
            for n in in_names:
                dev_in[sl][n].copy_(host_in[n], non_blocking=True)
            ev_in[sl].record(s_in)
        stream.wait_event(ev_in[sl])
        q_, k_, v_, b_ = (dev_in[sl][n].detach().requires_grad_(True) for n in ("q", "k", "v", "bias"))
        m_ = create_mask(dev_in[sl]["bias"], None, B, S, S, WINDOW, torch.finfo(torch.bfloat16).min)
        o = flash_sparse_attn_func(q_, k_, v_, attn_mask=m_, attn_bias=b_, is_causal=True)
        o.backward(dev_in[sl]["dout"])
        ev_comp[sl].record(stream)
        res = {"out": o.detach(), "dq": q_.grad, "dk": k_.grad, "dv": v_.grad, "dbias": b_.grad}
        live[sl] = res
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[sl])
            for n, t in res.items():
                host_out2[sl][n].copy_(t, non_blocking=True)
            ev_out[sl].record(s_out)

    e2e_ms = copy_ms = float("nan")
    if not args.no_e2e:
        # enough steps that filling and draining the three-stage pipeline (one upload, one compute and one download
        # that nothing overlaps) weighs little against the steady state
        e2e_steps = max(NB + 1, min(2 * args.steps, 30))
        for i in range(NB):
            e2e_step(i)
        torch.cuda.synchronize(dev)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        s_in.wait_event(e0)
        for i in range(e2e_steps):
            e2e_step(NB + i)
        for ev in ev_out:
            stream.wait_event(ev)
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        live = [None] * NB
        # The ceiling the host sets: the same bytes, up and down at once on two streams, with no compute at all
        # (every rank at the same time, as in the run above).
        res0 = {"out": out, "dq": dq, "dk": dk, "dv": dv, "dbias": dbias}
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record(stream)
        s_in.wait_event(c0)
        s_out.wait_event(c0)
        for i in range(e2e_steps):
            with torch.cuda.stream(s_in):
                for n in in_names:
                    dev_in[i % NB][n].copy_(host_in[n], non_blocking=True)
            with torch.cuda.stream(s_out):
                for n, t in res0.items():
                    host_out2[i % NB][n].copy_(t, non_blocking=True)
        fin_in, fin_out = torch.cuda.Event(), torch.cuda.Event()
        fin_in.record(s_in)
        fin_out.record(s_out)
        stream.wait_event(fin_in)
        stream.wait_event(fin_out)
        c1.record(stream)
        barrier()
        copy_ms = c0.elapsed_time(c1) / e2e_steps

    # ---- secondary workloads (rank 0 of a single-GPU run): short runs of the other benchmark shapes ----
    secondary = None
    if world == 1 and not args.no_secondary:
        del step, host_in, host_out, host_out2, dev_in
        torch.cuda.empty_cache()
        sec_args = argparse.Namespace(**vars(args))
        sec_args.steps, sec_args.warmup = max(3, min(args.steps, 5)), 3
        secondary = {}
        for name, fn in (("per_query_S8192", measure_perquery), ("decode_B32_Sk65536", measure_decode),
                         ("create_mask_65536x8192", measure_mask)):
            ln = fn(sec_args, 0, 1, local_rank)
            secondary[name] = {"metric": ln["metric"], "ms_per_step": ln["ms_per_step"], "value": ln["value"],
                               "unit": ln["unit"], "roofline": ln["roofline"], "workload": ln["config"]["workload"]}
            for extra in ("fwd_ms", "bwd_ms", "decode_kernel_ms", "bool_mask"):
                if extra in ln:
                    secondary[name][extra] = ln[extra]
            torch.cuda.empty_cache()

    # ---- the reference's own CUDA kernels on this GPU (a labelled extra, its own process; single-GPU runs) ----
    ref_cuda = None
    if world == 1 and not args.no_ref_cuda:
        torch.cuda.empty_cache()
        ref_cuda = reference_cuda_kernels()
        if secondary is not None and "unavailable" not in ref_cuda:
            secondary["per_query_S8192"]["reference_cuda_kernels"] = reference_cuda_kernels(
                ("--per-query", "--seq-len", "8192", "--window", "1024"))

    # ---- context parallelism over all ranks for one long sequence (multi-GPU runs only) ----
    cp = None
    if world > 1 and not args.no_cp:
        torch.cuda.empty_cache()
        cp = measure_cp(args, rank, world, local_rank)

    # ---- max over ranks ----
    vals = torch.tensor([ms_per_step_local, e2e_ms, fwd_ms, bwd_ms, copy_ms, min(step_ms_all), max(step_ms_all),
                         api_ms if api_ms is not None else float("nan")], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms_per_step, e2e_ms, fwd_ms, bwd_ms, copy_ms, ms_min, ms_max, api_ms_max = vals.tolist()
    flop_sum = torch.tensor([float(flops["total"]), float(flops["canonical_128x128"]), float(flops["causal_dense"]),
                             float(flops["bwd"]), float(flops["fwd"]), float(flops["element_level"])],
                            dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(flop_sum, op=dist.ReduceOp.SUM)
    if rank != 0:
        return
    tot, canon, dense, bwd_fl, fwd_fl, elem_fl = flop_sum.tolist()
    value = tot / (ms_per_step * 1e-3) / 1e12
    peaks = tensor_peaks(clocks["sm_mhz"] if clocks else None)
    bwd_tflops = (bwd_fl / world) / (bwd_ms * 1e-3) / 1e12  # per launch, per GPU
    fwd_tflops = (fwd_fl / world) / (fwd_ms * 1e-3) / 1e12
    cpu = cpu_sample(1, 1, compact) if world == 1 and not args.no_cpu else None
    line = {
        "metric": metric_name(args.compaction), "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "warmup_steps_run": n_w, "repeats": len(regions),
        "ms_per_step": ms_per_step, "ms_per_step_min": ms_min, "ms_per_step_max": ms_max,
        "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world, B, args.compaction),
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
        "api_ms_per_step": api_ms_max if api_ms is not None else None,
        "tflops_canonical_128x128_tiles": canon / (ms_per_step * 1e-3) / 1e12,
        "tflops_element_level": elem_fl / (ms_per_step * 1e-3) / 1e12,
        "tflops_causal_dense_equivalent": dense / (ms_per_step * 1e-3) / 1e12,
        "utilisation_of_nominal_2250": value / world / NOMINAL_TFLOPS,
        "roofline": {"bound": "tensor", "kernel": "bwd_kernel", "achieved": bwd_tflops, "peak": peaks["peak"],
                     "unit": "TFLOP/s", "frac": bwd_tflops / peaks["peak"], "peak_source": peaks["source"],
                     "frac_sustained": bwd_tflops / peaks["sustained"], "peak_sustained": peaks["sustained"],
                     "frac_of_nominal_2250": bwd_tflops / NOMINAL_TFLOPS,
                     # dram__bytes_read + dram__bytes_write of one bwd_kernel launch of exactly this workload, one ncu
                     # capture (profiles/fwd_bwd_kernel_S32768_compaction_dram_traffic.md); other geometries: null
                     "traffic": (2364e6 if (compact and (S, WINDOW, D, B) == (32768, 2048, 128, 1)) else None),
                     "fwd_kernel_achieved": fwd_tflops, "fwd_kernel_frac": fwd_tflops / peaks["peak"]},
        "e2e": {"value": tot / (e2e_ms * 1e-3) / 1e12 if e2e_ms == e2e_ms else None, "unit": "TFLOP/s",
                "ms_per_step": e2e_ms if e2e_ms == e2e_ms else None,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "copy_only_ms_per_step": copy_ms if copy_ms == copy_ms else None,
                "frac_of_copy_ceiling": (copy_ms / e2e_ms) if e2e_ms == e2e_ms and copy_ms == copy_ms else None,
                "note": "create_mask + flash_sparse_attn_func + backward on pinned host buffers; uploads, compute and "
                        "downloads of consecutive steps overlap on three streams. copy_only = the same bytes up and "
                        "down with no compute, all ranks at once: the host's ceiling for this figure"},
        "gpu_launches": args.steps * len(regions) * step_launches,
        "clocks": clocks,
    }
    if tile is not None:
        line["tile_or"] = {"ms_per_step": tile["ms_per_step"], "tflops_on_its_kept_tiles": tile["tflops_on_its_kept_tiles"],
                           "bwd_kernel_ms": tile["bwd_kernel_ms"], "fwd_kernel_ms": tile["fwd_kernel_ms"],
                           "bwd_kernel_tflops": tile["bwd_kernel_tflops"],
                           "bwd_kernel_frac": tile["bwd_kernel_tflops"] / peaks["peak"],
                           "fwd_kernel_tflops": tile["fwd_kernel_tflops"],
                           "fwd_kernel_frac": tile["fwd_kernel_tflops"] / peaks["peak"],
                           "frac_of_nominal_2250": tile["tflops_on_its_kept_tiles"] / NOMINAL_TFLOPS,
                           "note": tile["note"]}
    if parity is not None:
        line["parity"] = parity
    if secondary is not None:
        line["secondary"] = secondary
    if cp is not None:
        line["cp"] = cp
    if ref_cuda is not None:
        line["reference_cuda_kernels"] = ref_cuda
    if cpu is not None:
        line["cpu_baseline"] = {k_: cpu[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)


def measure_cp(args, rank: int, world: int, local_rank: int) -> dict:
    """Gathered-keys context parallelism over all ranks on the wide-head long-sequence shape (B=1, S=131072, Hq=16,
    Hkv=1, d=256, W=1024, causal, fwd+bwd with dBias), next to the time ONE GPU needs for the same sequence (rank 0
    runs it alone while the others wait). Returned on every rank; only rank 0's copy is printed."""
    import torch.distributed as dist

    from flash_sparse_attn import flash_sparse_attn_func, gathered_cp, ring
    from flash_sparse_attn.utils.mask import create_mask

    dev = torch.device(f"cuda:{local_rank}")
    B, Sr, H, Hk, d, w = 1, 131072, 16, 1, 256, 1024
    g = torch.Generator(device="cpu").manual_seed(7)
    bias_full = torch.randn((B, Hk, 1, Sr), generator=g).to(torch.bfloat16)
    mask_full = create_mask(bias_full.to(dev), None, B, Sr, Sr, w, torch.finfo(torch.bfloat16).min)
    rnd = lambda gen, *shape: torch.randn(shape, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    steps, warm = max(2, min(args.steps, 5)), 2

    def timed(fn):
        for _ in range(warm):
            fn()
        dist.barrier(); torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        dist.barrier(); torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # one GPU alone (rank 0), full sequence
    one_ms = torch.zeros(1, dtype=torch.float64, device=dev)
    if rank == 0:
        g1 = torch.Generator(device=dev).manual_seed(99)
        qf, kf, vf, df = rnd(g1, B, Sr, H, d), rnd(g1, B, Sr, Hk, d), rnd(g1, B, Sr, Hk, d), rnd(g1, B, Sr, H, d)
        qf.requires_grad_(True); kf.requires_grad_(True); vf.requires_grad_(True)
        bf = bias_full.to(dev).requires_grad_(True)

        def one():
            o = flash_sparse_attn_func(qf, kf, vf, attn_mask=mask_full, attn_bias=bf, is_causal=True)
            o.backward(df)
            qf.grad = kf.grad = vf.grad = bf.grad = None

        for _ in range(warm):
            one()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize(dev)
        one_ms[0] = e0.elapsed_time(e1) / steps
        del qf, kf, vf, df, bf
        torch.cuda.empty_cache()
    dist.broadcast(one_ms, 0)

    gl = torch.Generator(device=dev).manual_seed(100 + rank)
    S2 = Sr // world
    q, k, v, dout = rnd(gl, B, S2, H, d), rnd(gl, B, S2, Hk, d), rnd(gl, B, S2, Hk, d), rnd(gl, B, S2, H, d)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    bias = ring.zigzag_split(bias_full, 3, rank, world).contiguous().to(dev).requires_grad_(True)
    mask = ring.zigzag_split(mask_full.cpu(), 3, rank, world).contiguous().to(dev)

    def cp_step():
        out = gathered_cp.gathered_cp_flash_sparse_attn_func(q, k, v, mask, bias, None, True)
        out.backward(dout)
        q.grad = k.grad = v.grad = bias.grad = None

    cp_ms = timed(cp_step)
    return {"scheme": "gathered-keys context parallel (kept K/V rows all-reduced, zig-zag query chunks)",
            "workload": f"B=1 S={Sr} Hq={H} Hkv={Hk} d={d} W={w} causal, fwd+bwd with dBias", "n_gpus": world,
            "ms_per_step": cp_ms, "one_gpu_ms_per_step": one_ms.item(), "speedup_vs_one_gpu": one_ms.item() / cp_ms,
            "scaling": "strong", "steps": steps}


def run_ring(args, rank: int, world: int, local_rank: int):
    """Secondary workload (not the headline line): one long sequence, KV-ring context parallel over all ranks.
    The wide-head MQA long-sequence shape: B=1, S=131072, Hq=16, Hkv=1, d=256, top-1024 query-broadcast mask, causal, fwd+bwd with
    dBias."""
    import torch.distributed as dist

    from flash_sparse_attn import ring
    from flash_sparse_attn.utils.mask import create_mask

    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    iface.set_compaction(args.compaction)
    B, Sr, H, Hk, d, w = 1, args.ring_seq_len, 16, 1, args.ring_head_dim, 1024
    g = torch.Generator(device="cpu").manual_seed(7)
    bias_full = torch.randn((B, Hk, 1, Sr), generator=g).to(torch.bfloat16)
    mask_full = create_mask(bias_full.to(dev), None, B, Sr, Sr, w, torch.finfo(torch.bfloat16).min).cpu()
    gl = torch.Generator(device=dev).manual_seed(100 + rank)
    S2 = Sr // world
    rnd = lambda *shape: torch.randn(shape, generator=gl, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, dout = rnd(B, S2, H, d), rnd(B, S2, Hk, d), rnd(B, S2, Hk, d), rnd(B, S2, H, d)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    bias = ring.zigzag_split(bias_full, 3, rank, world).contiguous().to(dev).requires_grad_(True)
    mask = ring.zigzag_split(mask_full, 3, rank, world).contiguous().to(dev)

    from flash_sparse_attn import gathered_cp

    def step():
        if args.cp_scheme == "gathered":
            out = gathered_cp.gathered_cp_flash_sparse_attn_func(q, k, v, mask, bias, None, True)
        else:
            out = ring.ring_flash_sparse_attn_func(q, k, v, mask, bias, None, True)
        out.backward(dout)
        q.grad = k.grad = v.grad = bias.grad = None

    for _ in range(args.warmup):
        step()
    dist.barrier(); torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    dist.barrier(); torch.cuda.synchronize(dev)
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank != 0:
        return
    fl = count_flops(mask_full, B, Sr, Sr, H, Hk, d, True)
    # tiles the kernels really process: every visible (query chunk, key chunk) pair runs over the gathered kept keys
    # of the key chunk (when the ring took that route: same rule as flash_sparse_attn/ring.py::_chunk_capacity)
    C = Sr // (2 * world)
    kept_per_chunk = mask_full.reshape(B, Hk, 2 * world, C).sum(-1)
    cap = max(128, (int(kept_per_chunk.max()) + 127) // 128 * 128)
    gathered = args.compaction == "auto" and 4 * cap <= 3 * C and args.cp_scheme == "ring"
    tiles = 0
    if gathered:
        for b in range(B):
            for hk in range(Hk):
                for kc in range(2 * world):
                    row = mask_full[b, hk, 0, kc * C:(kc + 1) * C]
                    n_kt = (int(row.sum()) + 127) // 128
                    tiles += (H // Hk) * ((2 * world - 1 - kc) * (C // 128) * n_kt +
                                          kept_tiles_rowbcast(row, C, C, 128, 128, True, True))
    flops_done = 14 * d * 128 * 128 * tiles if gathered else fl["canonical_128x128"]
    if args.cp_scheme == "gathered":  # every query chunk runs over ALL gathered keys of the sequence at once
        flops_done = count_flops(mask_full, B, Sr, Sr, H, Hk, d, True, True)["canonical_128x128"]
    line = {
        "metric": ("fwd+bwd TFLOP/s on kept blocks (gathered-keys context parallel)" if args.cp_scheme == "gathered"
                   else "fwd+bwd TFLOP/s on kept blocks (KV-ring context parallel)"),
        "value": flops_done / (ms.item() * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms.item(),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"ring: B=1 S={Sr} Hq=16 Hkv=1 d={d} W=1024 causal, bias (1,1,1,S)",
                   "parallelism": (f"kept K/V rows all-reduced over {world} ranks, zig-zag query chunks of "
                                   f"{Sr // (2 * world)} tokens" if args.cp_scheme == "gathered" else
                                   f"KV ring over {world} ranks, zig-zag chunks of {Sr // (2 * world)} tokens"),
                   "key_compaction": ("whole sequence" if args.cp_scheme == "gathered" else
                                      "per chunk pair" if gathered else "off"),
                   "flops": ("128x128 tiles of the sequence's gathered kept keys" if args.cp_scheme == "gathered" else
                             "128x128 tiles of each key chunk's gathered kept keys, per visible chunk pair" if gathered
                             else "kept 128x128 tiles of the global mask")},
        "tflops_on_full_range_kept_tiles": fl["canonical_128x128"] / (ms.item() * 1e-3) / 1e12,
    }
    print(json.dumps(line), flush=True)


def measure_decode(args, rank: int, world: int, local_rank: int):
    """Secondary workload (not the headline line): the decode shape, single-query forward over a KV cache,
    B = 32 per GPU (--decode-batch), Sk = 65536, Hq = 32, Hkv = 8, d = 128, top-4096 mask, non-causal. HBM-bound:
    reported as GB/s of the bytes the kernel's skip granule (one key row) makes it read."""
    import torch.distributed as dist

    from flash_sparse_attn import _lib, flash_sparse_attn_func
    from flash_sparse_attn.utils.mask import create_mask

    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    B, Sk, H, Hk, d, w = args.decode_batch, 65536, 32, 8, 128, 4096
    g = torch.Generator(device=dev).manual_seed(4321 + rank)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, bias = rnd(B, 1, H, d), rnd(B, Sk, Hk, d), rnd(B, Sk, Hk, d), rnd(B, Hk, 1, Sk)
    mask = create_mask(bias, None, B, 1, Sk, w, torch.finfo(torch.bfloat16).min)
    kept = int(mask.sum().item())
    nbytes = kept * 2 * d * 2 + mask.numel() + kept * 2 + 2 * q.numel() * 2  # K+V rows, mask bytes, bias, Q, O
    stream = torch.cuda.current_stream(dev)
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kev = []
        for _ in range(args.steps):
            pair = [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)]
            for e in pair:
                e.record(stream)
            kev.append(pair)
        torch.cuda.synchronize(dev)
        lib = _lib.load()
        e0.record(stream)
        for i in range(args.steps):
            lib.fdma_time_next_kernel(kev[i][0].cuda_event, kev[i][1].cuda_event)
            flash_sparse_attn_func(q, k, v, attn_mask=mask, attn_bias=bias)
        e1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
    _lib.check(_lib.load().fdma_last_kernel_status(stream.cuda_stream, None), "kernel status")
    kernel_ms = statistics.mean(a.elapsed_time(b_) for a, b_ in kev)
    vals = torch.tensor([e0.elapsed_time(e1) / args.steps, float(nbytes), kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        ms_t = vals[:1].clone()
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
        dist.all_reduce(vals, op=dist.ReduceOp.SUM)
        vals[0] = ms_t[0]
    if rank != 0:
        return
    ms, total_bytes, kernel_ms = vals.tolist()
    kernel_ms /= world
    peak, src = hbm_peak()
    gbs = total_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "decode forward GB/s of bytes read at key-row granularity", "value": gbs, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"decode: B={B} per GPU, Sq=1, Sk={Sk}, Hq={H}, Hkv={Hk}, d={d}, W={w}, non-causal",
                   "bytes_per_step": total_bytes, "l2": "K/V cache far larger than L2"},
        "decode_kernel_ms": kernel_ms,
        "roofline": {"bound": "hbm", "kernel": "decode_mma_kernel",
                     "achieved": total_bytes / world / (kernel_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": total_bytes / world / (kernel_ms * 1e-3) / 1e9 / peak, "peak_source": src,
                     # one ncu capture of this kernel at B = 8 (profiles/decode_mma_kernel_B8_Sk65536_ncu_full.md):
                     # 146.9 MB of DRAM traffic for 139 MB of algorithmic bytes; traffic grows with the kept rows,
                     # so the ratio is applied to this launch's bytes
                     "traffic": total_bytes / world * (146.9 / 139.0),
                     "traffic_source": "ncu capture at B=8 scaled by algorithmic bytes (x1.057)"},
        "gpu_launches": args.steps * 2,  # decode_kernel + decode_merge_kernel
    }
    return line


def measure_perquery(args, rank: int, world: int, local_rank: int):
    """Secondary workload (not the headline line): the per-query training shape, per-query bias and mask. B=1, S=8192, Hq=32,
    Hkv=8, d=128, bias (B,Hkv,Sq,Sk) ~ N(0,1), mask = top-1024 per query row AND causal, fwd+bwd with a per-query
    dBias, through the C ABI on device-resident tensors. FLOPs on 128x128 (forward) / 64x128 (backward) tiles that
    hold a kept, causally visible element."""
    from flash_sparse_attn import _lib
    from flash_sparse_attn.utils.mask import create_mask

    if rank != 0:
        return
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    lib = _lib.load()
    B, Sq, w = 1, 8192, 1024
    g = torch.Generator(device=dev).manual_seed(99)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v = rnd(B, Sq, HQ, D), rnd(B, Sq, HKV, D), rnd(B, Sq, HKV, D)
    bias, dout = rnd(B, HKV, Sq, Sq), rnd(B, Sq, HQ, D)
    mask = create_mask(bias, None, B, Sq, Sq, w, torch.finfo(torch.bfloat16).min)
    vis = mask & torch.ones(Sq, Sq, dtype=torch.bool, device=dev).tril()
    G = HQ // HKV
    tiles_f = int(vis.view(B, HKV, Sq // 128, 128, Sq // 128, 128).any(dim=5).any(dim=3).sum().item()) * G
    tiles_b = int(vis.view(B, HKV, Sq // 64, 64, Sq // 128, 128).any(dim=5).any(dim=3).sum().item()) * G
    del vis
    flops = 4 * D * 128 * 128 * tiles_f + 10 * D * 64 * 128 * tiles_b
    stream = torch.cuda.current_stream(dev)
    # As flash_sparse_attn_func does for a mask that create_mask made: the kernels read the bit-packed form and the
    # tile activity create_mask wrote in the same launch (cached on the mask tensor) instead of the bool bytes.
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    packed = iface._cached_packed_mask(mask)
    step = AttentionStep(lib, dev, q, k, v, mask, bias, dout, False, packed=packed)
    for _ in range(max(args.warmup, 3)):
        step()
    ms_total, fwd_ms, bwd_ms = time_steps(step, args.steps, stream, lambda: torch.cuda.synchronize(dev))
    _lib.check(lib.fdma_last_kernel_status(stream.cuda_stream, None), "kernel status")
    ms = ms_total / args.steps
    pk = tensor_peaks(None)
    peak, peak_src = pk["peak"], pk["source"]
    bwd_tf = 10 * D * 64 * 128 * tiles_b / (bwd_ms * 1e-3) / 1e12
    line = {
        "metric": "fwd+bwd TFLOP/s on kept blocks (per-query bias and mask)", "value": flops / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"per-query: B=1 S={Sq} Hq={HQ} Hkv={HKV} d={D} W={w} causal, bias and mask (B,Hkv,Sq,Sk)",
                   "l2": "bias (1 GiB) and mask (0.5 GiB bool, 64 MiB bit-packed) are larger than L2",
                   "mask_form": ("bit-packed + tile activity, as create_mask leaves them beside the bool tensor"
                                 if packed is not None else "bool bytes"),
                   "tiles": {"fwd": list(FWD_TILE), "bwd": list(BWD_TILE)}},
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
        "roofline": {"bound": "tensor", "kernel": "bwd_kernel", "achieved": bwd_tf, "peak": peak, "unit": "TFLOP/s",
                     "frac": bwd_tf / peak, "peak_source": peak_src, "frac_sustained": bwd_tf / pk["sustained"],
                     "traffic": None},
        # fwd_kernel, bwd_prep, bwd_kernel, 2 partial reductions, convert_dq (+ 2 tile_activity with a bool mask)
        "gpu_launches": args.steps * (6 if packed is not None else 8),
    }
    if packed is not None:  # the same step reading the bool tensor (what a mask from elsewhere gets)
        try:
            del step
            bstep = AttentionStep(lib, dev, q, k, v, mask, bias, dout, False)
            for _ in range(max(args.warmup, 3)):
                bstep()
            b_total, b_fwd, b_bwd = time_steps(bstep, args.steps, stream, lambda: torch.cuda.synchronize(dev))
            _lib.check(lib.fdma_last_kernel_status(stream.cuda_stream, None), "kernel status")
            line["bool_mask"] = {"what": "same step, kernels read the bool tensor and derive the tile activity themselves",
                                 "ms_per_step": b_total / args.steps, "fwd_ms": b_fwd, "bwd_ms": b_bwd}
        except Exception as e:  # an extra: never let it take the line down
            line["bool_mask"] = {"unavailable": str(e)[:200]}
    return line


def measure_mask(args, rank: int, world: int, local_rank: int):
    """Secondary workload (not the headline line): create_mask alone at the per-query training shape's size, 65536 rows (B=1,
    Hkv=8, Sq=8192) x 8192 keys of bf16 bias, top-1024 per row. HBM-bound: GB/s of bias bytes read + mask bytes
    written. --mask-rows shrinks it for profiler captures."""
    from flash_sparse_attn import _lib
    from flash_sparse_attn.utils.mask import create_mask

    if rank != 0:
        return
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    rows, keys, w = args.mask_rows, 8192, 1024
    g = torch.Generator(device=dev).manual_seed(77)
    bias = torch.randn((1, 8, rows // 8, keys), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    min_dtype = torch.finfo(torch.bfloat16).min
    stream = torch.cuda.current_stream(dev)
    for _ in range(max(args.warmup, 3)):
        mask = create_mask(bias, None, 1, rows // 8, keys, w, min_dtype)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        mask = create_mask(bias, None, 1, rows // 8, keys, w, min_dtype)
    e1.record(stream)
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    assert int(mask[0, 0, 0].sum()) == w
    nbytes = bias.numel() * 2 + mask.numel()
    peak, src = hbm_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "create_mask GB/s (bias read + mask written)", "value": gbs, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"create_mask: {rows} rows x {keys} keys bf16, top-{w} per row", "bytes_per_step": nbytes,
                   "l2": "bias larger than L2"},
        "roofline": {"bound": "hbm", "kernel": "topk16_reg_kernel", "achieved": gbs, "peak": peak, "unit": "GB/s",
                     "frac": gbs / peak, "peak_source": src, "traffic": None},
        "gpu_launches": args.steps,
    }
    return line


def _print_if_line(line):
    if line is not None:
        print(json.dumps(line), flush=True)


def run_decode(args, rank, world, local_rank):
    _print_if_line(measure_decode(args, rank, world, local_rank))


def run_perquery(args, rank, world, local_rank):
    _print_if_line(measure_perquery(args, rank, world, local_rank))


def run_mask(args, rank, world, local_rank):
    _print_if_line(measure_mask(args, rank, world, local_rank))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch-per-gpu", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--seq-len", type=int, default=S, help="profiling only: shorter sequence")
    ap.add_argument("--window", type=int, default=WINDOW, help="profiling only: window for --seq-len")
    ap.add_argument("--head-dim", type=int, default=D, choices=[64, 128, 256], help="profiling only")
    ap.add_argument("--workload", default="sharded", choices=["sharded", "ring", "decode", "mask", "perquery"],
                    help="sharded = the headline benchmark; ring = single long sequence over a KV ring (needs >= 2 "
                         "ranks); decode = single-query forward over a KV cache (HBM-bound)")
    ap.add_argument("--decode-batch", type=int, default=32)
    ap.add_argument("--mask-rows", type=int, default=65536)
    ap.add_argument("--ring-seq-len", type=int, default=131072)
    ap.add_argument("--ring-head-dim", type=int, default=256, help="256 = the wide-head long-sequence shape; 128 for comparison")
    ap.add_argument("--cp-scheme", default="ring", choices=["ring", "gathered"],
                    help="--workload ring: rotate K/V chunks (ring) or all-reduce the kept K/V rows (gathered)")
    ap.add_argument("--compaction", default="auto", choices=["auto", "off"],
                    help="auto = the library's default route for this mask (kept keys gathered first); off = full key range")
    ap.add_argument("--no-tile-path", action="store_true", help="skip the full-key-range comparison leg")
    ap.add_argument("--repeats", type=int, default=5, help="how many times the timed region of K steps is taken "
                                                           "(the line reports the median region, with min and max)")
    ap.add_argument("--no-api", action="store_true", help="skip the public-API leg on device-resident tensors")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison of the timed workload")
    ap.add_argument("--no-secondary", action="store_true", help="skip the short runs of the other benchmark shapes")
    ap.add_argument("--no-cp", action="store_true", help="multi-GPU runs: skip the context-parallel long-sequence leg")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip timing the reference's own CUDA kernels")
    ap.add_argument("--lean", action="store_true", help="profiling runs: only the device-resident timed region")
    ap.add_argument("--min-warmup-seconds", type=float, default=0.5,
                    help="warm-up runs at least this long (0 for profiler captures, where launch counts must be fixed)")
    args = ap.parse_args()
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)
    if args.lean:
        args.no_cpu = args.no_e2e = args.no_tile_path = args.no_api = args.no_parity = args.no_secondary = True
        args.no_cp, args.no_ref_cuda, args.repeats = True, True, 1
    if args.seq_len != S or args.window != WINDOW or args.head_dim != D:
        set_geometry(args.seq_len, args.window, args.head_dim)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    try:
        if args.workload == "ring":
            run_ring(args, rank, world, local_rank)
        elif args.workload == "decode":
            run_decode(args, rank, world, local_rank)
        elif args.workload == "mask":
            run_mask(args, rank, world, local_rank)
        elif args.workload == "perquery":
            run_perquery(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
