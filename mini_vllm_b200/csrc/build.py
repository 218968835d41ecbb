"""Build libmini_vllm_b200.so (sm_100a only) with nvcc, in-tree.

    python -m mini_vllm_b200.csrc.build [--force] [--verbose]

The library lands next to the package (``mini_vllm_b200/libmini_vllm_b200.so``) so it
travels with a source snapshot; nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
ROOT = PKG.parent
LIB = PKG / "libmini_vllm_b200.so"
OBJ_DIR = CSRC / "build"
SOURCES = ["api.cu", "pack.cu", "rope_kv_write.cu", "decode_attn.cu", "prefill_attn.cu", "sampler.cu", "fused_ops.cu", "lm_head_argmax.cu"]
HEADERS = ["common.cuh", "host_util.cuh", "scan.cuh", str(ROOT / "include" / "mini_vllm_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", "--extended-lambda",
              "-Xcompiler", "-fPIC", "-I", str(ROOT / "include"), "-I", str(CSRC)]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    hdrs = [Path(h) if os.path.isabs(h) else CSRC / h for h in HEADERS]
    jobs = []
    for src in SOURCES:
        obj = OBJ_DIR / (src[:-3] + ".o")
        if force or _stale(obj, [CSRC / src, *hdrs]):
            cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", str(CSRC / src), "-o", str(obj)]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed: {cmd[-3]}")

    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    objs = [OBJ_DIR / (s[:-3] + ".o") for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run([_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
