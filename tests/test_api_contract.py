"""Host-only checks of the C ABI: exports, contract program, workspace formula."""
import ctypes
import subprocess

import pytest

from flash_attention3_b200 import capi
from tests.conftest import ROOT


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    for name in capi.EXPORTS:
        assert getattr(lib, name) is not None, name
    # every prototype in the headers is covered by EXPORTS
    import re
    declared = set()
    for header in ("shaobo_fa3_api.h", "shaobo_fa3_components.h", "shaobo_fa3_b200_ext.h"):
        text = (ROOT / "include" / header).read_text()
        declared |= set(re.findall(r"\b(shaobo_fa3_\w+)\s*\(", text))
    assert declared == set(capi.EXPORTS), declared ^ set(capi.EXPORTS)
    assert ctypes.sizeof(capi.Params) == 296


def test_contract_program(tmp_path):
    capi.load()
    exe = tmp_path / "api_contract"
    subprocess.run(["g++", "-std=c++17", "-I", str(ROOT / "include"), str(ROOT / "tests/contract/api_contract.cpp"),
                    str(capi.LIB_PATH), "-o", str(exe), f"-Wl,-rpath,{capi.LIB_PATH.parent}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "api_contract pass=1" in out.stdout


def test_headers_compile_as_c(tmp_path):
    exe = tmp_path / "header_is_c"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"),
                    str(ROOT / "tests/contract/header_is_c.c"), "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def _params(**kw):
    base = dict(batch=1, seqlen_q=1024, seqlen_k=1024, num_heads_q=4, num_heads_kv=2, head_dim_qk=128,
                head_dim_v=128, causal=1)
    base.update(kw)
    return capi.new_params(**base)


def test_workspace_formula():
    lib = capi.load()
    p = _params()
    rows = 1 * 4 * 1024
    accum = rows * 128 * 4
    # 8 key tiles x 2 KV heads = 16 units < 148 SMs: tiles are split.  Two query heads per KV head give
    # 2 * (8 + 7 + ... + 1) = 72 steps per KV head; 144 one-step CTAs still fit one wave of 148 SMs, and
    # every CTA owns one dK and one dV partial-sum slab of [128][128], fp16 for fp16 inputs (the default
    # dtype of a parameter block) and fp32 for bf16 inputs
    dkv_accum = 144 * 2 * (128 * 128 * 2)
    expected = accum + dkv_accum + ((rows * 4 + 255) // 256) * 256 + rows * 12
    assert lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p)) == expected
    assert lib.shaobo_fa3_bwd_fused5_workspace_bytes(ctypes.byref(p)) == accum + dkv_accum
    pb = _params(dtype=capi.DTYPE_BF16)
    assert lib.shaobo_fa3_bwd_fused5_workspace_bytes(ctypes.byref(pb)) == accum + 2 * dkv_accum
    # the deterministic path never splits and needs no partial-sum slabs
    pd = _params(deterministic=1)
    assert lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(pd)) == expected - dkv_accum
    # linear in S (the reference's per-K-tile partials were quadratic)
    p2 = _params(seqlen_q=8192, seqlen_k=8192, batch=16, num_heads_q=32, num_heads_kv=32)
    w = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(p2))
    assert w == 16 * 32 * 8192 * (128 * 4 + 4 + 12)
    # monotone in every dimension, 256-byte aligned sub-buffers
    prev = 0
    for s in (128, 256, 512, 1024):
        cur = lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(_params(seqlen_q=s, seqlen_k=s, deterministic=1)))
        assert cur > prev
        prev = cur
    for d in (64, 128):
        pd = _params(head_dim_qk=d, head_dim_v=d)
        assert lib.shaobo_fa3_bwd_fused5_workspace_bytes(ctypes.byref(pd)) % 256 == 0
    # overflow-safe: absurd sizes report 0 instead of wrapping
    big = _params(batch=2**31 - 1, num_heads_q=2**31 - 2, num_heads_kv=2**31 - 2, seqlen_q=2**31 - 128,
                  seqlen_k=2**31 - 128)
    assert lib.shaobo_fa3_bwd_v2_workspace_bytes(ctypes.byref(big)) == 0
    # components report 0 for paths without workspace
    assert lib.shaobo_fa3_bwd_dkv_workspace_bytes(ctypes.byref(_params(dkv_path=capi.DKV_PATH_CANONICAL))) == 0
    assert lib.shaobo_fa3_bwd_dq_workspace_bytes(ctypes.byref(_params(dq_path=capi.DQ_PATH_CANONICAL))) == 0


def test_no_spills_in_any_kernel():
    """ptxas report of the last build: no local-memory spills (the role of the
    reference's static no-spill gates, scripts/check_symbol_metadata_gate.py)."""
    from flash_attention3_b200 import build
    build.build(force=not (build.PKG / "build_ptxas.log").exists())
    report = build.ptxas_report()
    assert len(report) >= 20
    for k in report:
        assert k["spill_stores"] == 0 and k["spill_loads"] == 0 and k["stack"] == 0, k
