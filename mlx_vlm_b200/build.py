"""Build the native libraries (sm_100a only) in-tree with nvcc.

`python -m mlx_vlm_b200.build [target]` or `build(target=...)`; each .so lands next to this file so
it travels with the repo snapshot to the GPU box (it is git-ignored).  Targets:
  b200vlm   the whole C ABI (every model family)
  b200lm    the layer-level ops alone (decoder designs assembled layer by layer on the host): with the
            tcgen05 GEMM they feed: a fresh checkout that only serves such a model compiles five files
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200vlm.so")
LM_SOURCES = ["errors.cu", "layer_ops.cu", "mixer_ops.cu", "gemm_wt.cu", "tower_f32.cu"]
SOURCES = LM_SOURCES + ["engine.cu", "gemm_tcgen05.cu", "rowops.cu", "attention.cu", "decode.cu", "decode_mega.cu",
           "decode_mega_tc.cu", "attention_tc.cu", "attention_fa.cu", "decode_batch.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


TARGETS = {"b200vlm": SOURCES, "b200lm": LM_SOURCES}


def lib_path(target: str = "b200vlm") -> str:
    return os.path.join(HERE, f"lib{target}.so")


def _fingerprint(sources) -> str:
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in sorted(os.listdir(root)):
            if name.endswith((".cuh", ".h")) or name in sources:
                with open(os.path.join(root, name), "rb") as f:
                    h.update(name.encode())
                    h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, target: str = "b200vlm") -> str:
    SOURCES, LIB = TARGETS[target], lib_path(target)
    stamp = LIB + ".stamp"
    fp = _fingerprint(SOURCES)
    if not force and os.path.exists(LIB) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build", target), exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(HERE, "build", target, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {src} ---\n{out.decode()}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError(f"nvcc failed building {os.path.basename(LIB)}")
    tmp = f"{LIB}.{os.getpid()}.tmp"          # concurrent first calls: each links its own file, the rename is atomic
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC"]
    subprocess.check_call(cmd)
    os.replace(tmp, LIB)
    with open(stamp, "w") as f:
        f.write(fp)
    return LIB


if __name__ == "__main__":
    names = [a for a in sys.argv[1:] if not a.startswith("-")] or ["b200vlm"]
    for name in names:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, target=name))
