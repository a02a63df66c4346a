#!/usr/bin/env python3
"""Benchmark of the FlashAttention-3 backward hot path (shaobo_fa3_bwd_v2).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C2] [--impl reference]

A step is one shaobo_fa3_bwd_v2 call (delta -> fused five-GEMM kernel -> dQ
convert) over one synthetic batch.  The default workload is B=1, H=4, S=2048,
D=128, causal, fp16 per GPU; with N GPUs every rank runs the same workload on
its own batch shard (global batch N, no collective on the data path), so
scaling is weak.  Rank 0 prints one JSON line.

Keys beyond the base contract:
  roofline      five-GEMM kernel: algorithmic FLOPs / CUDA-event time of that
                kernel alone (stage events recorded by the library) against
                the measured dense bf16 peak
  cpu_baseline  the CPU oracle (NumPy restatement of the reference golden)
                timed on this host on the same workload
  e2e           the same call with host (pinned) inputs and outputs: H2D copies,
                the call, D2H copies, all inside the timed region
  also          TFLOP/s of the larger configurations (N=1 only, informative), and at every N
                "C5_strong": the large sharded configuration (B=16,H=32,S=8192,D=128 causal bf16)
                split over the N ranks by batch with no collective -- strong scaling -- with a
                parity flag (every rank checks one (batch, head) slice of its shard against the
                CPU oracle outside the timed region)
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import pathlib
import statistics
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIGS = {
    # name: (batch, heads_q, heads_kv, seqlen, head_dim, dtype, causal, description)
    "C1": (1, 1, 1, 1024, 128, "fp16", True, "B=1,H=1,S=1024,D=128 causal fp16"),
    "C2": (1, 4, 4, 2048, 128, "fp16", True, "B=1,H=4,S=2048,D=128 causal fp16"),
    "C3d128": (4, 16, 16, 4096, 128, "bf16", False, "B=4,H=16,S=4096,D=128 non-causal bf16"),
    "C3d64": (4, 16, 16, 4096, 64, "bf16", False, "B=4,H=16,S=4096,D=64 non-causal bf16"),
    "C4": (2, 32, 8, 8192, 128, "bf16", True, "B=2,Hq=32,Hkv=8,S=8192,D=128 causal bf16 (GQA)"),
    "C5shard": (2, 32, 32, 8192, 128, "bf16", True, "B=2 of 16,H=32,S=8192,D=128 causal bf16 (1/8 shard)"),
    # the large sharded configuration: strong scaling, the (batch x head) range is split over the ranks
    "C5": (16, 32, 32, 8192, 128, "bf16", True, "B=16,H=32,S=8192,D=128 causal bf16, sharded by batch x head"),
    # profiler-sized case: ~0.2 GB on the device, working set above the 126 MB L2
    "P1": (1, 16, 16, 4096, 128, "bf16", False, "B=1,H=16,S=4096,D=128 non-causal bf16 (profiling case)"),
    "P2": (1, 16, 16, 4096, 128, "bf16", True, "B=1,H=16,S=4096,D=128 causal bf16 (profiling case)"),
    "P3": (1, 16, 16, 4096, 64, "bf16", False, "B=1,H=16,S=4096,D=64 non-causal bf16 (profiling case)"),
}
METRIC = "fa3_bwd_tflops"
UNIT = "TFLOP/s"
L2_FLUSH_BYTES = 256 << 20  # larger than the 126 MB L2
WARMUP_SECONDS = 0.3         # least wall-clock time of the warm-up of the back-to-back and end-to-end loops


def bwd_flops(b, hq, s, d, causal):
    f = 10.0 * b * hq * float(s) * float(s) * d
    return f / 2 if causal else f


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"tflops_burst": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ----------------------------------------------------------------------------
# clocks: sampled with NVML while the timed region runs
# ----------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------
# CPU arm: the oracle port timed on the host cores
# ----------------------------------------------------------------------------
def cpu_golden_rate(cfg, min_seconds, max_reps):
    """TFLOP/s of the NumPy golden on (a bounded sample of) the workload."""
    import numpy as np
    from oracle import golden
    b, hq, hkv, s, d, dtype, causal, _ = cfg
    heads = min(b * hq, 4)  # bounded sample: at most four (batch, head) slices per repetition
    q, k, v, do = golden.seeded_inputs(4321, 1, heads, max(1, heads * hkv // hq), s, d, dtype)
    group = heads // k.shape[1]
    scale = 1.0 / float(np.sqrt(d))
    reps, t0 = 0, time.perf_counter()
    while True:
        for h in range(heads):
            golden.head_backward(q[0, h], k[0, h // group], v[0, h // group], do[0, h], causal, scale, dtype)
        reps += 1
        elapsed = time.perf_counter() - t0
        if elapsed >= min_seconds or reps >= max_reps:
            break
    flops = bwd_flops(1, heads, s, d, causal) * reps
    return {"value": flops / elapsed / 1e12, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": f"{heads} (batch,head) slices of the workload x {reps} repetitions, {elapsed:.1f} s, "
                      f"NumPy/BLAS on all host threads; the golden computes the full SxS matrix even when causal"}


LAUNCHES_PER_CALL = 3  # delta, five-GEMM kernel, convert (or delta, dK/dV kernel, dQ kernel)


L2_BYTES = 126 << 20


def tensor_bytes(cfg):
    """Bytes of the nine tensors of one call (q, k, v, dO, O, LSE in; dq, dk, dv out)."""
    b, hq, hkv, s, d, _, _, _ = cfg
    return (5 * hq + 4 * hkv) * b * s * d * 2 + b * hq * s * 4


def rotation_sets(cfg):
    """How many independent copies of the workload the timed calls rotate over.  A workload smaller
    than the L2 is timed as K calls back to back (one pair of CUDA events around all of them), each
    call on the next of so many sets of tensors and workspaces that together they exceed twice the L2:
    no call finds its inputs cached.  0: the workload is larger than the L2 by itself and is timed call
    by call with the L2 flushed in between (long calls run into the power cap when issued back to
    back, so that way of timing them would measure the cooling, not the kernel)."""
    per_set = tensor_bytes(cfg)
    if per_set >= L2_BYTES:
        return 0
    return max(2, -(-2 * L2_BYTES // per_set))


def config_block(desc, strong, b, world, deterministic, cfg):
    """The "config" object of the JSON line: identical for the GPU arm and the reference arm of one
    command line (the L2 protocol is the GPU arm's; the CPU arm has no device cache to flush)."""
    n_sets = rotation_sets(cfg)
    if n_sets:
        l2 = (f"GPU arm: the steps run back to back between one pair of CUDA events, rotating over {n_sets} "
              f"independent sets of tensors and workspaces ({n_sets * tensor_bytes(cfg) >> 20} MiB of tensors, "
              f"L2 = {L2_BYTES >> 20} MiB); isolated_call: L2 flushed before every step, per-step events")
    else:
        l2 = f"GPU arm: flushed before every step ({L2_FLUSH_BYTES >> 20} MiB write + {L2_FLUSH_BYTES >> 20} MiB read, untimed)"
    return {"workload": desc if strong else desc + " per GPU", "global_batch": b if strong else b * world,
            "sharding": "batch (no collective)",
            "path": "deterministic split path" if deterministic else "fused path",
            "l2": l2}


def run_reference_arm(args, cfg, rank, world):
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its workers; this arm is the only work on the host, so it
    # takes every host thread, as a single-process run does (NumPy is first imported below)
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(os.cpu_count())
    b, hq, hkv, s, d, dtype, causal, desc = cfg
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        base = cpu_golden_rate(cfg, 0.0, 1)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    heads = min(b * hq, 4)
    value = bwd_flops(1, heads, s, d, causal) / (ms * 1e-3) / 1e12
    threads = os.environ.get("OMP_NUM_THREADS") or os.cpu_count()
    base.update({"value": value, "cores": int(threads),
                 "sample": f"each step = {heads} (batch,head) slices of the workload through the NumPy golden "
                           f"(oracle port of the reference's CPU path), BLAS threads: {threads} "
                           f"(OMP_NUM_THREADS={os.environ.get('OMP_NUM_THREADS', 'unset')})"})
    config = config_block(desc, args.config == "C5", b, world, args.deterministic, cfg)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": config,
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------
class Workload:
    def __init__(self, cfg, seed, torch, capi, ops, synthetic, deterministic=False):
        self.torch, self.capi = torch, capi
        b, hq, hkv, s, d, dtype, causal, _ = cfg
        self.cfg = cfg
        td = torch.float16 if dtype == "fp16" else torch.bfloat16
        self.q, self.k, self.v, self.do = synthetic.make_inputs(seed, b, hq, hkv, s, d, td)
        # O and LSE come from the library's own forward (set-up, outside every timed region)
        self.out, self.lse = ops.fa3_fwd(self.q, self.k, self.v, causal, sync=True)
        self.lib = capi.load()
        self.p = ops.make_params(self.q, self.k, causal, deterministic=int(deterministic))
        need = self.lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(self.p))
        self.ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        self.p.workspace, self.p.workspace_bytes = self.ws.data_ptr(), need
        self.dq, self.dk, self.dv = torch.empty_like(self.q), torch.empty_like(self.k), torch.empty_like(self.v)
        self.flops = bwd_flops(b, hq, s, d, causal)

        # the argument list of the call, marshalled once: a caller in C passes nine pointers and a struct,
        # and the step should cost the host what that costs, not what building ctypes objects costs
        vp = lambda t: ctypes.c_void_p(t.data_ptr())
        self._call = self.lib.shaobo_fa3_bwd_v2
        self._args = (vp(self.do), vp(self.q), vp(self.k), vp(self.v), vp(self.out), vp(self.lse), vp(self.dq),
                      vp(self.dk), vp(self.dv), None, ctypes.byref(self.p))

    def step(self):
        code = self._call(*self._args)
        if code != 0:
            raise RuntimeError(f"shaobo_fa3_bwd_v2 returned {code} ({self.capi.status_string(code)})")


class ForwardWorkload:
    """The forward kernel on the same inputs (reported under "also"; not the headline metric)."""

    def __init__(self, cfg, seed, torch, capi, ops, synthetic):
        b, hq, hkv, s, d, dtype, causal, _ = cfg
        td = torch.float16 if dtype == "fp16" else torch.bfloat16
        self.q, self.k, self.v, _ = synthetic.make_inputs(seed, b, hq, hkv, s, d, td)
        self.lib, self.capi = capi.load(), capi
        self.p = ops.make_params(self.q, self.k, causal)
        self.out = torch.empty_like(self.q)
        self.lse = torch.empty((b, hq, s), dtype=torch.float32, device="cuda")
        self.flops = 0.4 * bwd_flops(b, hq, s, d, causal)  # 4*B*H*S^2*D, halved when causal

    def step(self):
        vp = lambda t: ctypes.c_void_p(t.data_ptr())
        code = self.lib.shaobo_fa3_b200_fwd(vp(self.q), vp(self.k), vp(self.v), vp(self.out), vp(self.lse),
                                            ctypes.byref(self.p))
        if code != 0:
            raise RuntimeError(f"shaobo_fa3_b200_fwd returned {code} ({self.capi.status_string(code)})")


class L2Flush:
    """Evicts the step's tensors from the 126 MB L2 between iterations: write a 256 MiB buffer, then
    read a second one, so that L2 ends up full of clean lines (a write-only flush leaves ~126 MB of
    dirty lines whose write-back would be charged to the first kernels of the next step)."""

    def __init__(self, torch):
        self.w = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
        self.r = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda")
        self.sink = torch.zeros((), dtype=torch.int64, device="cuda")

    def zero_(self):
        self.w.zero_()
        self.sink += self.r.sum()


def time_steps(torch, wl, steps, warmup, flush):
    """Per-step CUDA-event timing with an L2 flush (untimed) before every step."""
    for _ in range(warmup):
        flush.zero_()
        wl.step()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.zero_()
        starts[i].record()
        wl.step()
        ends[i].record()
    torch.cuda.synchronize()
    return [starts[i].elapsed_time(ends[i]) for i in range(steps)]


def time_back_to_back(torch, sets, steps, warmup, barrier):
    """K calls back to back, call i on set i % len(sets); one pair of CUDA events around all of them,
    bracketed by a barrier and a device synchronisation on both sides.  Returns the milliseconds of the
    K calls together."""
    # warm-up: at least W calls and every set once, and at least WARMUP_SECONDS of wall clock -- the calls are
    # 30 us apart, which the host thread that enqueues them sustains only once its core has clocked up
    t0 = time.perf_counter()
    i = 0
    while i < max(warmup, len(sets)) or time.perf_counter() - t0 < WARMUP_SECONDS:
        sets[i % len(sets)].step()
        i += 1
        if i % 256 == 0:
            torch.cuda.synchronize()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        sets[i % len(sets)].step()
    end.record()
    barrier()
    return start.elapsed_time(end)


def time_stages(torch, wl, steps, flush):
    """CUDA-event time of each of the three launches, averaged over `steps` calls."""
    lib = wl.lib
    lib.shaobo_fa3_b200_stage_timing(1)
    acc = [0.0, 0.0, 0.0]
    buf = (ctypes.c_float * 3)()
    for _ in range(steps):
        flush.zero_()
        wl.step()
        if lib.shaobo_fa3_b200_last_stage_ms(buf) != 0:
            raise RuntimeError("stage timing unavailable")
        for i in range(3):
            acc[i] += buf[i]
    lib.shaobo_fa3_b200_stage_timing(0)
    return [a / steps for a in acc]


def time_e2e(torch, wl, steps, warmup, flush, ops):
    """Host buffers in, host buffers out, through the library's host-tensor call (shaobo_fa3_b200_bwd_v2_host):
    pinned H2D of every input, shaobo_fa3_bwd_v2, D2H of dq/dk/dv, pipelined over (batch, KV head)
    shards.  Every byte crosses PCIe inside the timed region, every step."""
    b, hq, hkv, s, d, dtype, causal, _ = wl.cfg
    dev_in = [wl.q, wl.k, wl.v, wl.do, wl.out, wl.lse]
    hq_, hk_, hv_, hdo_, hout_, hlse_ = [t.cpu().pin_memory() for t in dev_in]
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (wl.dq, wl.dk, wl.dv)]
    call = ops.HostBackwardC(b, hq, hkv, s, d, wl.q.dtype, causal)  # shaobo_fa3_b200_bwd_v2_host
    h2d, d2h = call.h2d_bytes, call.d2h_bytes

    def one():
        call(hdo_, hq_, hk_, hv_, hout_, hlse_, *host_out)

    # warm-up by wall clock as well as by count: the call is bound by copies over PCIe that the host
    # thread must keep fed (18 copies, 6 launches and a dozen event operations per call), and a host core
    # that has idled through the device-bound part of the run needs a while to clock up again (measured on
    # fresh boxes: 0.6-0.9 ms per call in the first second of such calls, 0.37 ms after)
    t0 = time.perf_counter()
    n_warm = 0
    while n_warm < warmup or time.perf_counter() - t0 < 2 * WARMUP_SECONDS:
        one()
        n_warm += 1
        if n_warm % 16 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    times = []
    for _ in range(steps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        one()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    # the pipelined call must give what the plain device call gives
    wl.step()
    torch.cuda.synchronize()
    for h, dref in zip(host_out, (wl.dq, wl.dk, wl.dv)):
        # (not bitwise: dQ is summed with fp32 atomics, whose order differs between the two calls)
        a_, b_ = h.float(), dref.cpu().float()
        if ((a_ - b_).norm() / b_.norm().clamp_min(1e-30)).item() > 2e-3:
            raise RuntimeError("host-tensor call disagrees with the device call")
    return times, h2d, d2h


def oracle_slice_parity(torch, wl, bi, h):
    """One (batch entry, query head) slice of a workload against the CPU oracle.  The slice's O and
    LSE are replaced by the oracle's own (rounded to storage), one more call is made, and dQ of the
    head, dK / dV of its KV head (when the head has it to itself) and delta are gated as in the tests."""
    import numpy as np
    from oracle import golden
    b, hq, hkv, s, d, dtype, causal, _ = wl.cfg
    f = lambda t: t.detach().float().cpu().numpy()
    group = hq // hkv
    kv = h // group
    r = golden.head_backward(f(wl.q[bi, h]), f(wl.k[bi, kv]), f(wl.v[bi, kv]), f(wl.do[bi, h]), causal,
                             1.0 / float(np.sqrt(d)), dtype)
    wl.out[bi, h] = torch.from_numpy(r.out).to(wl.out.dtype).cuda()
    wl.lse[bi, h] = torch.from_numpy(r.lse).cuda()
    wl.step()
    torch.cuda.synchronize()
    checks = {"dq": golden.check_gradient(f(wl.dq[bi, h]), r.dq, dtype)}
    if group == 1:
        checks["dk"] = golden.check_gradient(f(wl.dk[bi, kv]), r.dk, dtype)
        checks["dv"] = golden.check_gradient(f(wl.dv[bi, kv]), r.dv, dtype)
    ok = all(m["pass"] for m in checks.values()) and wl.lib.shaobo_fa3_b200_device_error(1) == 0
    return ok, {k: round(m["rel_l2"], 6) for k, m in checks.items()}


def c5_strong(torch, capi, ops, synthetic, flush, rank, world, dist, steps=10, warmup=3):
    """The large sharded configuration split over the ranks by batch (strong scaling): time per step
    as the max over ranks, aggregate TFLOP/s, and the parity flag of every rank's sampled slice."""
    from flash_attention3_b200 import sharding
    cfg = CONFIGS["C5"]
    b, hq, hkv, s, d, dtype, causal, desc = cfg
    mine = sharding.plan(b, hkv, world)[rank]
    assert len(mine) == 1 and mine[0].kv_head_count == hkv, "C5 shards are whole batches"
    wl = Workload((mine[0].batch_count,) + cfg[1:], 4321 + mine[0].batch_begin, torch, capi, ops, synthetic)
    times = time_steps(torch, wl, steps, warmup, flush)
    ms = sharding.max_over_ranks(sum(times), dist, "cuda") / steps
    ok, rel = oracle_slice_parity(torch, wl, mine[0].batch_count - 1, (7 * rank + 3) % hq)
    all_ok = sharding.max_over_ranks(0.0 if ok else 1.0, dist, "cuda") == 0.0
    tflops = bwd_flops(b, hq, s, d, causal) / (ms * 1e-3) / 1e12
    del wl
    torch.cuda.empty_cache()
    return {"workload": desc, "scaling": "strong", "n_gpus": world, "steps": steps, "ms_per_step": ms,
            "tflops": tflops, "per_gpu_frac_of_measured_peak": tflops / world / measured_peaks()["tflops_burst"],
            "parity_at_n": bool(all_ok), "rank0_slice_rel_l2": rel}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="C2", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip cpu_baseline, e2e and the 'also' configurations")
    ap.add_argument("--deterministic", action="store_true",
                    help="time the atomic-free split path (deterministic=1) instead of the fused path")
    ap.add_argument("--forward-only", action="store_true",
                    help="time the forward kernel alone on --config (one GPU; a profiling aid, not the headline metric)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, cfg, rank, world)
        return

    import torch
    from flash_attention3_b200 import capi, ops, synthetic
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    if args.forward_only:
        flush = L2Flush(torch)
        fw = ForwardWorkload(cfg, 77, torch, capi, ops, synthetic)
        ms = statistics.median(time_steps(torch, fw, args.steps, args.warmup, flush))
        print(json.dumps({"metric": "attention forward throughput", "value": fw.flops / (ms * 1e-3) / 1e12,
                          "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                          "config": {"workload": "forward kernel, " + cfg[7]}, "gpu_launches": args.steps}))
        return

    b, hq, hkv, s, d, dtype, causal, desc = cfg
    strong = args.config == "C5"
    if strong:
        # this rank's contiguous (batch x KV head) range; for B=16 over 1/2/4/8 ranks these are whole batches
        from flash_attention3_b200 import sharding
        mine = sharding.plan(b, hkv, world)[rank]
        assert len(mine) == 1 and mine[0].kv_head_count == hkv, "C5 shards are whole batches"
        cfg = (mine[0].batch_count,) + cfg[1:]
    wl = Workload(cfg, 1234 + rank, torch, capi, ops, synthetic, deterministic=args.deterministic)
    flush = L2Flush(torch)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    n_sets = rotation_sets(cfg)
    sets = [wl] + [Workload(cfg, 4321 + 100 * i + rank, torch, capi, ops, synthetic, deterministic=args.deterministic)
                   for i in range(1, n_sets)]
    barrier()
    with ClockSampler(local_rank) as clocks:
        times = time_steps(torch, wl, args.steps, args.warmup, flush)
        barrier()
        b2b_ms = time_back_to_back(torch, sets, args.steps, args.warmup, barrier) if n_sets else None
    dev_err = wl.lib.shaobo_fa3_b200_device_error(1)
    if dev_err != 0:
        raise SystemExit(f"device error flag {dev_err}")
    from flash_attention3_b200.sharding import max_over_ranks
    job_flops = bwd_flops(b, hq, s, d, causal) if strong else world * wl.flops
    isolated_ms = max_over_ranks(sum(times), dist, "cuda") / args.steps
    isolated = {"ms_per_step": isolated_ms, "value": job_flops / (isolated_ms * 1e-3) / 1e12, "unit": UNIT,
                "method": "L2 flushed before every step (untimed), one pair of CUDA events per step"}
    if n_sets:
        # the headline: K steps between one barrier + synchronise and the next, as the steps of a training
        # loop follow one another; the isolated figure is kept beside it
        total_ms = max_over_ranks(b2b_ms, dist, "cuda")
        del sets[1:]
        torch.cuda.empty_cache()
    else:
        total_ms = isolated_ms * args.steps
    ms_per_step = total_ms / args.steps
    value = job_flops / (ms_per_step * 1e-3) / 1e12

    stage_ms = time_stages(torch, wl, min(args.steps, 20), flush)
    peaks = measured_peaks()
    # fused path: stage 1 is the five-GEMM kernel (all the FLOPs); deterministic path: stage 1 is the
    # four-GEMM dK/dV kernel (8 of the 10 units), stage 2 the three-GEMM dQ kernel
    stage1_flops = wl.flops * (0.8 if args.deterministic else 1.0)
    achieved = stage1_flops / (stage_ms[1] * 1e-3) / 1e12
    traffic = None
    tpath = ROOT / "profiles" / "dram_traffic.json"
    if tpath.exists():  # bytes per launch from a committed ncu capture of this workload, not from this run
        traffic = json.loads(tpath.read_text()).get(args.config, {}).get("fused_bwd_kernel")
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                "frac": achieved / peaks["tflops_burst"], "traffic": traffic,
                "traffic_source": "profiles/dram_traffic.json (ncu capture of this workload, not this run)",
                "kernel": ("fused_bwd_kernel without dQ (S, dP, dV, dK)" if args.deterministic
                           else "fused_bwd_kernel (S, dP, dV, dK, dQ)"),
                "peak_source": peaks["source"] + " (burst bf16 GEMM)", "kernel_ms": stage_ms[1],
                "other_kernels_ms": {"delta_sidecar_kernel": stage_ms[0],
                                     ("dq_bwd_kernel" if args.deterministic else "dq_convert_kernel"): stage_ms[2]}}

    e2e_times, h2d, d2h = time_e2e(torch, wl, max(3, min(args.steps, 30)), 5, flush, ops)
    # median of the steps: a call that shares the host's PCIe switch and cores with other tenants shows
    # single steps far off (the spread is reported beside it)
    e2e_ms = max_over_ranks(statistics.median(e2e_times), dist, "cuda")
    e2e = {"value": job_flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "statistic": f"median of {len(e2e_times)} steps",
           "ms_min": min(e2e_times), "ms_max": max(e2e_times), "ms_mean": sum(e2e_times) / len(e2e_times)}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if strong else "weak",
        "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": config_block(desc, strong, b, world, args.deterministic, CONFIGS[args.config]),
        "isolated_call": isolated,
        "fractions": {"per_gpu_of_measured_peak": value / world / peaks["tflops_burst"],
                      "per_gpu_of_nominal_2250": value / world / 2250.0},
        "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": LAUNCHES_PER_CALL * args.steps, "roofline": roofline,
    }
    also = {}
    if not args.no_extra and not strong and not args.deterministic:
        # the strong-scaling curve of the large sharded configuration, at this N (every rank takes part)
        del wl
        wl = None
        torch.cuda.empty_cache()
        also["C5_strong"] = c5_strong(torch, capi, ops, synthetic, flush, rank, world, dist)
    if rank == 0 and world == 1 and not args.no_extra:
        line["cpu_baseline"] = cpu_golden_rate(cfg, 10.0, 50)
        wl = None
        torch.cuda.empty_cache()
        for name in ("C3d128", "C3d64", "C4", "C5shard"):
            if name == args.config:
                continue
            w2 = Workload(CONFIGS[name], 77, torch, capi, ops, synthetic)
            t2 = time_steps(torch, w2, 10, 3, flush)
            ms = statistics.median(t2)
            also[name] = {"ms_per_step": ms, "tflops": w2.flops / (ms * 1e-3) / 1e12,
                          "workload": CONFIGS[name][7]}
            if name == "C4":
                # the large shape through the host-tensor call: PCIe-bound, eight pipelined shards
                te, h2d, d2h = time_e2e(torch, w2, 5, 3, flush, ops)
                me = statistics.median(te)
                also[name]["e2e"] = {"ms_per_step": me, "tflops": w2.flops / (me * 1e-3) / 1e12,
                                     "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
            del w2
            torch.cuda.empty_cache()
        for name in ("C3d128", "C3d64", "C4"):
            w2 = ForwardWorkload(CONFIGS[name], 77, torch, capi, ops, synthetic)
            t2 = time_steps(torch, w2, 10, 3, flush)
            ms = statistics.median(t2)
            also["forward_" + name] = {"ms_per_step": ms, "tflops": w2.flops / (ms * 1e-3) / 1e12,
                                       "workload": "forward kernel, " + CONFIGS[name][7]}
            del w2
            torch.cuda.empty_cache()
    if also:
        line["also"] = also
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
