"""Per-CTA timeline of one shaobo_fa3_bwd_v2 call, from an instrumented build of the library.

    python -m flash_attention3_b200.timeline [--batch 1 --heads 4 --heads-kv 4 --seqlen 2048 --dim 128
                                              --dtype fp16 --causal 1]

The library is compiled a second time with -DFA3B200_TRACE (in-tree, libfa3bwd_b200_trace.so): the
GEMM kernel then stamps clock64() at the hand-offs of every role of every CTA (set-up, loads, each
MMA group, both softmax phases, the drain, the epilogue) and the two row-wise kernels stamp their
first start and last end with %globaltimer.  This module runs three warm-up calls and one stamped
call (L2 flushed before each, as in bench.py) and prints medians / minima / maxima over the CTAs.
The stamps cost a few hundred cycles per CTA: read the split of the time, not the total.
"""
from __future__ import annotations

import argparse
import ctypes
import pathlib
import statistics
import subprocess
import shutil

import numpy as np
import torch

from . import build as lib_build
from . import capi

TRACE_LIB = lib_build.PKG / "libfa3bwd_b200_trace.so"


def build_trace_library() -> pathlib.Path:
    newest = max(p.stat().st_mtime for p in lib_build.SOURCES + lib_build.HEADERS)
    if TRACE_LIB.exists() and TRACE_LIB.stat().st_mtime > newest:
        return TRACE_LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    flags = [f for f in lib_build.NVCC_FLAGS if f not in ("-Xptxas", "-v")]
    cmd = [nvcc, *flags, "-DFA3B200_TRACE", "-I", str(lib_build.ROOT / "include"), "-I", str(lib_build.CSRC),
           "-o", str(TRACE_LIB), *map(str, lib_build.SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + (proc.stdout + proc.stderr)[-4000:])
    return TRACE_LIB


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--heads-kv", type=int, default=None)
    ap.add_argument("--seqlen", type=int, default=2048)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--causal", type=int, default=1)
    args = ap.parse_args()
    hkv = args.heads if args.heads_kv is None else args.heads_kv
    capi.LIB_PATH = build_trace_library()
    capi._lib = None
    from . import ops, synthetic
    lib = capi.load()
    lib.shaobo_fa3_b200_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    td = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    q, k, v, do = synthetic.make_inputs(1234, args.batch, args.heads, hkv, args.seqlen, args.dim, td)
    out, lse = ops.fa3_fwd(q, k, v, bool(args.causal), sync=True)
    p = ops.make_params(q, k, bool(args.causal))
    need = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p))
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    flush_w = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    flush_r = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")

    def flush():
        flush_w.zero_()
        flush_r.sum()

    def step():
        code = lib.shaobo_fa3_bwd_v2(vp(do), vp(q), vp(k), vp(v), vp(out), vp(lse), vp(dq), vp(dk), vp(dv), None,
                                     ctypes.byref(p))
        if code != 0:
            raise RuntimeError(f"shaobo_fa3_bwd_v2 returned {code}")

    N, R, E = 1024, 4, 64
    buf = np.zeros((N, R, E), np.int64)
    rw = np.zeros(4, np.int64)
    for _ in range(3):
        flush()
        step()
    torch.cuda.synchronize()
    lib.shaobo_fa3_b200_trace_read(buf.ctypes.data, rw.ctypes.data)   # clears the stamps
    flush()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    step()
    e1.record()
    torch.cuda.synchronize()
    label = (f"B={args.batch},Hq={args.heads},Hkv={hkv},S={args.seqlen},D={args.dim} "
             f"{'causal' if args.causal else 'full'} {args.dtype}")
    print(f"== {label}: call {e0.elapsed_time(e1)*1e3:.1f} us (CUDA events)")
    lib.shaobo_fa3_b200_trace_read(buf.ctypes.data, rw.ctypes.data)
    ctas = [c for c in range(N) if buf[c, 0, 0] != 0]
    print("CTAs traced:", len(ctas))
    gt0 = min(buf[c, 0, 1] for c in ctas)
    gt_end = max(buf[c, 0, 62] for c in ctas)
    print(f"fused kernel: first CTA start .. last CTA end = {(gt_end-gt0)/1e3:.2f} us (globaltimer)")
    print(f"delta kernel: start {(rw[0]-gt0)/1e3:+.2f} us, end {(rw[1]-gt0)/1e3:+.2f} us relative to the first fused CTA")
    print(f"convert kernel: first block start {(rw[2]-gt0)/1e3:+.2f} us, last block end {(rw[3]-gt0)/1e3:+.2f} us")
    starts = sorted((buf[c, 0, 1] - gt0) / 1e3 for c in ctas)
    ends = sorted((buf[c, 0, 62] - gt0) / 1e3 for c in ctas)
    print(f"CTA start spread: median {statistics.median(starts):.2f} max {starts[-1]:.2f} us; CTA end: min {ends[0]:.2f} median {statistics.median(ends):.2f} max {ends[-1]:.2f} us")


    def rel(c, role, ev):
        v = buf[c, role, ev]
        return None if v == 0 else int(v - buf[c, 0, 0])


    def stat(name, vals):
        vals = [v for v in vals if v is not None]
        if not vals:
            return
        print(f"  {name:58s} n={len(vals):4d} median {statistics.median(vals):8.0f}  min {min(vals):7.0f}  max {max(vals):7.0f}")


    def diff(c, r1, e1_, r0, e0_):
        a, b = buf[c, r1, e1_], buf[c, r0, e0_]
        return None if a == 0 or b == 0 else int(a - b)


    print("-- set-up (clk from CTA start)")
    stat("index arithmetic done (tile known)", [rel(c, 0, 4) for c in ctas])
    stat("barriers initialised", [rel(c, 0, 2) for c in ctas])
    stat("first loads issued (K,V,Q0,dO0)", [rel(c, 0, 3) for c in ctas])
    stat("set-up barrier passed (TMEM allocated)", [rel(c, 1, 0) for c in ctas])
    stat("K,V,Q(0) landed (seen by MMA warp)", [rel(c, 1, 1) for c in ctas])
    stat("S(0) issued", [rel(c, 1, 2) for c in ctas])
    stat("dP(0) issued", [rel(c, 1, 4) for c in ctas])
    stat("softmax: first A done", [rel(c, 2, 4 + 2) for c in ctas])
    stat("softmax: first dP seen", [rel(c, 2, 4 + 4) for c in ctas])
    stat("softmax: first dS written", [rel(c, 2, 4 + 6) for c in ctas])
    stat("drain: first dQ seen", [rel(c, 3, 4 + 0) for c in ctas])
    print("-- top of step 3, softmax warp 4 (first warpgroup: row statistics bookkeeping)")
    stat("dS(2) handed over -> loop top", [diff(c, 2, 0, 2, 4 + 8 * 2 + 7) for c in ctas])
    stat("tile coordinates of the step", [diff(c, 2, 1, 2, 0) for c in ctas])
    stat("statistics published", [diff(c, 2, 2, 2, 1) for c in ctas])
    stat("next statistics requested", [diff(c, 2, 3, 2, 2) for c in ctas])
    stat("statistics barrier passed", [diff(c, 2, 4 + 8 * 3 + 0, 2, 3) for c in ctas])
    print("-- per step (clk), softmax warp 4")
    for t in range(0, 6):
        tb = 4 + 8 * t
        if not any(buf[c, 2, tb + 6] for c in ctas):
            break
        print(f" step {t}")
        if t > 0:
            stat("  period (dS written(t) - dS written(t-1))", [diff(c, 2, tb + 6, 2, tb - 8 + 6) for c in ctas])
            stat("  wait: stats", [diff(c, 2, tb + 0, 2, tb - 8 + 7) for c in ctas])
        stat("  wait: S full after stats", [diff(c, 2, tb + 1, 2, tb + 0) for c in ctas])
        stat("  phase A (ld, exp2, P store issued)", [diff(c, 2, tb + 2, 2, tb + 1) for c in ctas])
        stat("  P store wait + arrive", [diff(c, 2, tb + 3, 2, tb + 2) for c in ctas])
        stat("  wait: dP full", [diff(c, 2, tb + 4, 2, tb + 3) for c in ctas])
        stat("  wait: dS buffer free", [diff(c, 2, tb + 5, 2, tb + 4) for c in ctas])
        stat("  phase B (ld, dS, smem store)", [diff(c, 2, tb + 6, 2, tb + 5) for c in ctas])
    print("-- per step (clk), MMA warp")
    for t in range(0, 6):
        tb = 8 + 8 * t
        if not any(buf[c, 1, tb + 0] for c in ctas):
            break
        print(f" step {t}")
        stat("  wait P ready (from previous stamp)", [diff(c, 1, tb + 0, 1, tb - 1 if t > 0 else 4) for c in ctas])
        stat("  issue dV", [diff(c, 1, tb + 1, 1, tb + 0) for c in ctas])
        stat("  wait Q(t+1) + issue S(t+1)", [diff(c, 1, tb + 2, 1, tb + 1) for c in ctas])
        stat("  wait dS ready", [diff(c, 1, tb + 3, 1, tb + 2) for c in ctas])
        stat("  issue dQ,dK", [diff(c, 1, tb + 4, 1, tb + 3) for c in ctas])
        stat("  wait dO(t+1)", [diff(c, 1, tb + 5, 1, tb + 4) for c in ctas])
        stat("  wait dQ drained", [diff(c, 1, tb + 6, 1, tb + 5) for c in ctas])
        stat("  issue dP(t+1)", [diff(c, 1, tb + 7, 1, tb + 6) for c in ctas])
    print("-- drain warp 12 (clk)")
    for t in range(0, 6):
        tb = 4 + 4 * t
        if not any(buf[c, 3, tb + 0] for c in ctas):
            break
        stat(f" step {t}: dQ full -> loaded", [diff(c, 3, tb + 1, 3, tb + 0) for c in ctas])
        stat(f" step {t}: loaded -> reduce-adds issued", [diff(c, 3, tb + 2, 3, tb + 1) for c in ctas])
    print("-- tail (clk)")
    stat("MMA warp: last commit issued (from CTA start)", [rel(c, 1, 62) for c in ctas])
    stat("softmax: all MMAs done (dK/dV complete), from CTA start", [rel(c, 2, 60) for c in ctas])
    stat("softmax: epilogue (dK/dV written) duration", [diff(c, 2, 61, 2, 60) for c in ctas])
    stat("drain: all reduce-adds complete, from CTA start", [rel(c, 3, 59) for c in ctas])
    stat("CTA end (after teardown), from CTA start", [rel(c, 0, 63) for c in ctas])
    nsteps = []
    for c in ctas:
        n = 0
        for t in range(7):
            if buf[c, 2, 4 + 8 * t + 6]:
                n = t + 1
        nsteps.append(n)
    print("steps per CTA (traced, <=7):", {n: nsteps.count(n) for n in sorted(set(nsteps))})


if __name__ == "__main__":
    main()
