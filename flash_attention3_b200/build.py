"""Build recipe of the shared library (nvcc, sm_100a only, in-tree output).

    python -m flash_attention3_b200.build            # build if sources are newer
    python -m flash_attention3_b200.build --force
"""
from __future__ import annotations

import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libfa3bwd_b200.so"
SOURCES = [CSRC / "fa3_api.cpp", CSRC / "fa3_launch.cu"]
HEADERS = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((ROOT / "include").glob("*.h"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-diag-suppress", "177",
]


def stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile the library when missing or older than its sources.  Returns the
    path; raises if nvcc is unavailable or compilation fails (there is no
    fallback implementation)."""
    if not force and not stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(ROOT / "include"), "-I", str(CSRC), "-o", str(LIB),
           *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    (PKG / "build_ptxas.log").write_text(log)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + log[-4000:])
    if verbose:
        print(log)
    return LIB


def ptxas_report() -> list[dict]:
    """Per-kernel registers / spills from the last build log (no-spill gate)."""
    import re
    path = PKG / "build_ptxas.log"
    if not path.exists():
        return []
    text = path.read_text()
    out = []
    pat = re.compile(
        r"Compiling entry function '([^']+)' for 'sm_100a'.*?"
        r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads.*?"
        r"Used (\d+) registers", re.S)
    for m in pat.finditer(text):
        out.append({"kernel": m.group(1), "stack": int(m.group(2)), "spill_stores": int(m.group(3)),
                    "spill_loads": int(m.group(4)), "registers": int(m.group(5))})
    return out


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
