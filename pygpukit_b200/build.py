"""Build libpgk_b200.so in-tree with nvcc for sm_100a (no torch, no cmake).

    python -m pygpukit_b200.build                 # incremental, every source
    python -m pygpukit_b200.build --force
    python -m pygpukit_b200.build --components core,seq

The shared library is the product's only native artefact; the Python package loads it with
ctypes (pygpukit_b200/_lib.py) and fails loudly when it is missing.

`build(components=[...])` links only the named groups of sources (plus whatever the existing
library already holds), so that a program that serves one model family compiles what that family
needs and no more; the list of linked sources is kept beside the library.  `build()` links all.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libpgk_b200.so")
MANIFEST = LIB + ".sources"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]

# quant_nvf4.cu must use the reference's fast-math flags to stay bit-exact (see its header)
SOURCES = {
    "runtime.cu": [],
    "gemv_fp8.cu": [],
    "gemv_nvf4.cu": [],
    "gemv_bf16.cu": [],
    "gemm_w8a16.cu": [],
    "gemm_tc.cu": [],
    "gemm_tc_nvf4.cu": [],
    "gemm_tc_f8.cu": [],
    "elementwise.cu": [],
    "attention.cu": [],
    "moe.cu": [],
    "sampling.cu": [],
    "comm.cu": [],
    "p2p.cu": [],
    "step.cu": [],
    "init.cu": [],
    "quant_nvf4.cu": ["--use_fast_math"],
    "seq_gemm.cu": [],
    "seq_attention.cu": [],
    "seq_layers.cu": [],
    "seq_latent.cu": [],
    "seq_recurrent.cu": [],
    "seq_gated.cu": [],
}

# groups of sources that link on their own (runtime.cu is in every library)
COMPONENTS = {
    "core": ["runtime.cu"],
    # token-major float32-activation models on the paged cache (llm/models/layered.py)
    "seq": ["runtime.cu", "seq_gemm.cu", "seq_attention.cu", "seq_layers.cu", "seq_latent.cu", "seq_recurrent.cu",
            "seq_gated.cu"],
}


def _deps_mtime() -> float:
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            if f.endswith((".cuh", ".h")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def _compile(src: str, extra: list[str], force: bool, hdr_t: float) -> str:
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(path), hdr_t):
        return obj
    cmd = [NVCC, *ARCH, *COMMON, *extra, "-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def linked_sources() -> list[str]:
    """Sources the existing library was linked from ([] when there is none)."""
    if not (os.path.exists(LIB) and os.path.exists(MANIFEST)):
        return []
    with open(MANIFEST, encoding="utf-8") as f:
        return [ln.strip() for ln in f if ln.strip()]


def build(force: bool = False, verbose: bool = True, components: list[str] | None = None) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr_t = _deps_mtime()
    if components is None:
        want = list(SOURCES)
    else:
        need = {s for c in components for s in COMPONENTS[c]} | set(linked_sources())
        want = [s for s in SOURCES if s in need]
    srcs = {s: SOURCES[s] for s in want if os.path.exists(os.path.join(CSRC, s))}
    workers = max(1, min(8, len(srcs), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as ex:
        objs = list(ex.map(lambda kv: _compile(kv[0], kv[1], force, hdr_t), srcs.items()))
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < newest or linked_sources() != list(srcs):
        tmp = LIB + f".tmp{os.getpid()}"
        cmd = [NVCC, *ARCH, "-shared", "-o", tmp, *objs, "-ldl", "-Xlinker", "--no-undefined"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
        with open(MANIFEST, "w", encoding="utf-8") as f:
            f.write("\n".join(srcs) + "\n")
        if verbose:
            print(f"built {LIB} ({len(srcs)} sources)")
    elif verbose:
        print(f"up to date: {LIB}")
    return LIB


if __name__ == "__main__":
    comps = None
    for i, a in enumerate(sys.argv):
        if a == "--components" and i + 1 < len(sys.argv):
            comps = sys.argv[i + 1].split(",")
    build(force="--force" in sys.argv, components=comps)
