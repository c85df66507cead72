"""Build libflare_b200.so (sm_100a) from csrc/ with nvcc.  Objects are cached by content hash."""

from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build", "obj")
LIB = os.path.join(HERE, "libflare_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    *os.environ.get("FLARE_B200_NVCC_FLAGS", "").split(),  # extra flags for experiments (e.g. -DNAME)
]

# (source file, extra defines, object name)
UNITS = [
    ("flare_abi.cu", [], "flare_abi"),
    ("walk_exact.cu", [], "walk_exact_dispatch"),
    *[("walk_exact.cu", [f"-DFLARE_WALK_MM={mm}"], f"walk_exact_mm{mm}") for mm in (2, 8, 16, 32, 64)],
    ("decode_step.cu", [], "decode_step"),
    ("state_ops.cu", [], "state_ops"),
    ("prefill_tc.cu", [], "prefill_tc_host"),
    *[("prefill_tc.cu", [f"-DFLARE_TC_UNIT={u}"], f"prefill_tc_unit{u}") for u in range(8)],
    ("noalloc.cu", [], "noalloc"),
    ("bwd_tc.cu", [], "bwd_tc_host"),
    *[("bwd_tc.cu", [f"-DFLARE_BT_UNIT={u}"], f"bwd_tc_unit{u}") for u in range(3)],
    ("bwd_exact.cu", [], "bwd_exact_dispatch"),
    *[("bwd_exact.cu", [f"-DFLARE_WALK_MM={mm}"], f"bwd_exact_mm{mm}") for mm in (2, 8, 16, 32, 64)],
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libflare_b200.so cannot be built")


def _digest(src: str, defines: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + defines).encode())
    with open(os.path.join(CSRC, src), "rb") as f:
        h.update(f.read())
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    with open(os.path.join(HERE, "..", "include", "flare_b200.h"), "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def _compile(unit, verbose: bool) -> tuple[str, bool]:
    src, defines, name = unit
    obj = os.path.join(OBJ, name + ".o")
    stamp = obj + ".sha"
    dig = _digest(src, defines)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj, False
    cmd = [_nvcc(), *NVCC_FLAGS, *defines, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(f"--- {name}\n{res.stderr}\n")
    with open(stamp, "w") as f:
        f.write(dig)
    return obj, True


def build(verbose: bool = False, jobs: int | None = None) -> str:
    os.makedirs(OBJ, exist_ok=True)
    jobs = jobs or min(len(UNITS), os.cpu_count() or 4)
    with cf.ThreadPoolExecutor(jobs) as pool:
        results = list(pool.map(lambda u: _compile(u, verbose), UNITS))
    objs = [o for o, _ in results]
    if any(changed for _, changed in results) or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
