"""Build libr3d_b200.so (the plugin) in-tree with nvcc for sm_100a.

    python -m libr3d_b200.build

The shared object lands next to this file so that it travels with the source tree; there
is no JIT cache and no installed copy. Objects are rebuilt only when a source or header is
newer. `-fmad=false`: the kernels spell every fused multiply-add they want, because a
contracted mul+add is a different rounding than the arithmetic contract states.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
SO = PKG / "libr3d_b200.so"

SOURCES = [
    "rows_table.cpp",
    "entries_gemm_q.cpp",
    "entries_band.cpp",
    "entries_logits.cpp",
    "entries_w2a8.cpp",
    "planes_cache.cpp",
    "launch.cu",
    "kern_exact.cu",
    "kern_topk.cu",
    "kern_rerank.cu",
    "kern_w2a8.cu",
    "kern_q8x.cu",
    "q8x_static.cu",
    "kern_stream.cu",
    "kern_tc.cu", "kern_tc_mxf4.cu", "kern_tc_q8x.cu", "kern_tc_gemm.cu", "kern_tc_gemm2.cu", "gather.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build_plugin(verbose: bool = False, ptxas_info: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    srcs = [s for s in SOURCES if (CSRC / s).exists()]
    jobs = []
    for s in srcs:
        src = CSRC / s
        obj = OBJ / (src.stem + ".o")
        if _stale(obj, [src] + headers):
            cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((s, cmd))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = {ex.submit(subprocess.run, cmd, capture_output=True, text=True): s for s, cmd in jobs}
            for f in cf.as_completed(futs):
                r = f.result()
                if verbose or r.returncode != 0 or ptxas_info:
                    sys.stderr.write(f"[{futs[f]}]\n{r.stdout}{r.stderr}\n")
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {futs[f]}")
    objs = [OBJ / (Path(s).stem + ".o") for s in srcs]
    if jobs or _stale(SO, objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(SO),
               *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return SO


if __name__ == "__main__":
    build_plugin(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(SO)
