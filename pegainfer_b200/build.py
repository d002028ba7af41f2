"""In-tree build of the sm_100a CUDA libraries (nvcc cross-compiles without a GPU).

    python -m pegainfer_b200.build            # build everything that is stale
    python -m pegainfer_b200.build --force

Outputs (git-ignored, shipped to the GPU box by gpurun):
    pegainfer_b200/libpegainfer_kernels_b200.so   -- the C-ABI kernel library (include/pegainfer_kernels.h)
    pegainfer_b200/libpegainfer_qwen3_host.so     -- C++ mirror of the reference's Rust host side
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "--std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-ccbin", "/usr/bin/g++"]

KERNEL_LIB = os.path.join(HERE, "libpegainfer_kernels_b200.so")
HOST_LIB = os.path.join(HERE, "libpegainfer_qwen3_host.so")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build failed: {cmd[0]} ... {cmd[-1]}")


# What one design needs when nothing is built yet (a fresh checkout asked to serve that design compiles these files and no
# others): kernel sources, host sources.  A later full build adds the rest and links both libraries again.
PARTS_OF = {
    "Vamadra": (("runtime.cu", "gemm.cu", "gemm2.cu", "gemv.cu", "sampling.cu", "residual32_ops.cu", "gemm_batched_mma.cu", "latent_attention.cu", "latent_attention_mma.cu", "moe.cu", "moe_grouped.cu"),
                ("qwen3_host.cpp", "layered_host.cpp")),
    "Risolorn": (("runtime.cu", "gemm.cu", "gemm2.cu", "gemv.cu", "sampling.cu", "residual32_ops.cu", "gemm_batched_mma.cu", "gqa_attention.cu", "recurrent_mixers.cu", "moe.cu", "moe_grouped.cu"),
                 ("qwen3_host.cpp", "layered_host.cpp")),
    "Nagosun": (("runtime.cu", "gemm.cu", "gemm2.cu", "gemv.cu", "sampling.cu", "residual32_ops.cu", "gemm_batched_mma.cu", "gqa_attention.cu", "latent_attention.cu", "latent_attention_mma.cu"),
                ("qwen3_host.cpp", "layered_host.cpp")),
}
PARTS_OF["Goguzen"] = PARTS_OF["Risolorn"]  # the same files: attention, recurrent mixers, experts on the fp32 residual stream
MANIFEST = os.path.join(OBJ, "linked.txt")


def kernel_sources(only=None) -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu") and (only is None or f in only))


def host_sources(only=None) -> list[str]:
    d = os.path.join(CSRC, "host")
    if not os.path.isdir(d):
        return []
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(".cpp") and (only is None or f in only))


def _linked() -> set:
    try:
        with open(MANIFEST) as f:
            return set(f.read().split())
    except OSError:
        return set()


def build(force: bool = False, verbose: bool = False, parts=None) -> None:
    """Build what is stale.  ``parts`` = (kernel files, host files) restricts a FIRST build to those sources; once libraries
    that hold at least these parts exist, nothing is rebuilt for them (sources newer than their objects still are)."""
    os.makedirs(OBJ, exist_ok=True)
    have = _linked()
    if parts is not None and os.path.exists(KERNEL_LIB) and os.path.exists(HOST_LIB) and set(parts[0]) | set(parts[1]) <= have:
        parts = tuple(sorted(f for f in have if f.endswith(ext)) for ext in (".cu", ".cpp"))  # keep what is linked, refresh if stale
    konly, honly = (None, None) if parts is None else (set(parts[0]), set(parts[1]))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "pegainfer_kernels.h"))
    hdir = os.path.join(CSRC, "host")
    if os.path.isdir(hdir):
        headers += [os.path.join(hdir, f) for f in os.listdir(hdir) if f.endswith((".hpp", ".h"))]

    jobs, objs = [], []
    for src in kernel_sources(konly):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append([NVCC, *ARCH, *NVCC_FLAGS, "-c", src, "-o", obj])
    if verbose and jobs:
        print(f"[pegainfer_b200.build] compiling {len(jobs)} CUDA file(s) for sm_100a", flush=True)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    names = {os.path.basename(p) for p in kernel_sources(konly)} | {os.path.basename(p) for p in host_sources(honly)}
    relink = names != have
    if force or jobs or relink or _stale(KERNEL_LIB, objs):
        _run([NVCC, *ARCH, "-shared", "-o", KERNEL_LIB, *objs, "-lcudart", "-ccbin", "/usr/bin/g++"])

    hsrcs = host_sources(honly)
    if hsrcs and (force or relink or _stale(HOST_LIB, hsrcs + headers)):
        if verbose:
            print("[pegainfer_b200.build] compiling the C++ host mirror", flush=True)
        _run(["/usr/bin/g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread",
              "-I/usr/local/cuda/include", "-I" + os.path.join(HERE, "..", "include"), *hsrcs,
              "-o", HOST_LIB, "-L/usr/local/cuda/lib64", "-lcudart", "-ldl",
              "-Wl,-rpath,/usr/local/cuda/lib64"])
    if relink or not os.path.exists(MANIFEST):
        with open(MANIFEST, "w") as f:
            f.write("\n".join(sorted(names)) + "\n")


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print("ok:", KERNEL_LIB)
