"""A compiled C++ caller runs the whole lifecycle on the GPU (no Python between it and the C ABI):
tests/contract/lifecycle.cpp is built with the link line INTEGRATION.md gives, fed raw golden files
written by the oracle (the file set of reference scripts/generate_full_bwd_golden.py:113-132 plus
lse.f32) and calls shaobo_fa3_bwd_v2 and the dot_do_o -> dkv -> dq chain the way reference
src/full_bwd_correctness.cpp:367-392 does."""
from __future__ import annotations

import pathlib
import shutil
import subprocess

import numpy as np
import pytest

from flash_attention3_b200 import build as lib_build
from tests import helpers

ROOT = pathlib.Path(__file__).resolve().parents[1]
CUDA = pathlib.Path(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc").resolve().parents[1]


def write_golden_dir(prob: helpers.Problem, path: pathlib.Path) -> None:
    f16 = lambda x: np.ascontiguousarray(x, dtype=np.float32).astype("<f2")
    f32 = lambda x: np.ascontiguousarray(x, dtype="<f4")
    files = {
        "q.f16": f16(prob.q), "k.f16": f16(prob.k), "v.f16": f16(prob.v), "o.f16": f16(prob.ref["out"]),
        "dout.f16": f16(prob.do), "scores_max.f32": f32(prob.ref["scores_max"]),
        "scores_sum.f32": f32(prob.ref["scores_sum"]), "lse.f32": f32(prob.ref["lse"]),
        "delta.f32": f32(prob.ref["delta"]), "packed_sidecar.f32": f32(prob.ref["packed_sidecar"]),
        "dq.f32": f32(prob.ref["dq"]), "dk.f32": f32(prob.ref["dk"]), "dv.f32": f32(prob.ref["dv"]),
    }
    for name, arr in files.items():
        arr.tofile(path / name)


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    lib = lib_build.build()
    exe = tmp_path_factory.mktemp("lifecycle") / "lifecycle"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), "-I", str(CUDA / "include"),
                    str(ROOT / "tests/contract/lifecycle.cpp"), str(lib), "-L", str(CUDA / "lib64"), "-lcudart",
                    f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{CUDA / 'lib64'}", "-o", str(exe)], check=True)
    return exe


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [
    (1, 1, 1, 1024, 128, 1),   # B=1,H=1,S=1024,D=128 causal: the reference's CPU-runnable configuration
    (1, 4, 2, 256, 128, 1),    # GQA: dK/dV reduced over two query heads
    (2, 2, 2, 256, 64, 0),     # full attention, head_dim 64
])
def test_compiled_caller_lifecycle(harness, tmp_path, shape):
    b, hq, hkv, s, d, causal = shape
    prob = helpers.Problem(b, hq, hkv, s, d, "fp16", bool(causal), seed=99)
    write_golden_dir(prob, tmp_path)
    out = subprocess.run([str(harness), str(tmp_path), *map(str, shape)], capture_output=True, text=True)
    print(out.stdout)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("lifecycle ")]
    assert lines[-1] == "lifecycle pass=1"
    paths = {l.split()[1] for l in lines[:-1]}
    assert paths == {"path=v2_fused5", "path=v2_deterministic", "path=seven_gemm", "path=dq_alone_smax_ssum",
                     "path=dq_alone_lse", "path=dq_without_statistics"}
