"""In-tree build of ``librg_b200.so`` for sm_100a with nvcc (no JIT cache, no torch extension).

``python -m rustgrad_b200.build`` compiles every source under ``csrc/`` in parallel and links one
shared library beside this file.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "librg_b200.so"
SOURCES = ["qgemv.cu", "qgemv_rows.cu", "qgemv_i8.cu", "qgemm_tc.cu", "qgemm_tc_wide.cu", "attn_fused.cu", "tp_fused.cu", "attn_prefill.cu", "attn_prefill_tc.cu", "attn_decode_tc.cu", "ops.cu", "runtime.cc", "ops_abi.cc", "gguf.cc", "comm.cc", "tokenizer.cc", "workflow.cc", "serving.cc"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + list((HERE.parent / "include").glob("*.h")))
    return LIB.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    OBJ.mkdir(exist_ok=True)
    cc = nvcc()
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        cmd = [cc, *ARCH, *COMMON, "-ccbin", "g++", "-x", "cu", "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(compile_one, sources()))
    link = [cc, *ARCH, "-shared", "-ccbin", "g++", "-o", str(LIB), *map(str, objs), "-ldl"]
    r = subprocess.run(link, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
