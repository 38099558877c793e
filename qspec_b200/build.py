"""In-tree build of the C-ABI CUDA library (sm_100a only): qspec_b200/_C/libqspec_b200.so.

`python -m qspec_b200.build` or `__graft_entry__.build()`. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_C")
LIB_PATH = os.path.join(OUT_DIR, "libqspec_b200.so")
SOURCES = ["capi.cu", "act_kernels.cu", "hadamard_kernels.cu", "gemm_w4_stream.cu", "attn_kernels.cu", "qwen_kernels.cu"]
# The sequence-mixer kernels (include/qspec_b200_seq.h) are a library of their own, so that a model that needs only them
# builds only them: libqspec_b200_seq.so.
SEQ_SOURCES = ["capi.cu", "seq_kernels.cu", "seq_mma_kernels.cu", "seq_mix_kernels.cu", "seq_state_kernels.cu"]
SEQ_LIB_PATH = os.path.join(OUT_DIR, "libqspec_b200_seq.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newest_source_mtime(sources=None) -> float:
    names = os.listdir(CSRC) if sources is None else list(sources) + ["common.cuh", "seq_common.cuh"]
    paths = [os.path.join(CSRC, f) for f in names]
    paths.append(os.path.join(HERE, "..", "include", "qspec_b200.h"))
    paths.append(os.path.join(HERE, "..", "include", "qspec_b200_seq.h"))
    return max(os.path.getmtime(p) for p in paths)


def build_seq_library(force: bool = False, verbose: bool = False) -> str:
    """libqspec_b200_seq.so: the sequence-mixer kernels only (seconds to compile). Objects are written next to the
    library under a per-process name and moved into place, so that two first calls at once do not clash."""
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(SEQ_LIB_PATH) and os.path.getmtime(SEQ_LIB_PATH) >= _newest_source_mtime(SEQ_SOURCES):
        return SEQ_LIB_PATH
    nvcc = _nvcc()
    tag = f".{os.getpid()}"

    def compile_one(src):
        obj = os.path.join(OUT_DIR, src.replace(".cu", f"_seq{tag}.o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SEQ_SOURCES)) as ex:
        objs = list(ex.map(compile_one, SEQ_SOURCES))
    tmp = SEQ_LIB_PATH + tag
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "shared"],
                       capture_output=True, text=True)
    for o in objs:
        os.remove(o)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, SEQ_LIB_PATH)
    return SEQ_LIB_PATH


def build_variant(suffix: str, defines, verbose: bool = False) -> str:
    """Experiment builds: libqspec_b200<suffix>.so compiled with extra -D flags (select with QSPEC_LIB=<path>)."""
    os.makedirs(OUT_DIR, exist_ok=True)
    lib_path = LIB_PATH.replace(".so", f"{suffix}.so")
    nvcc = _nvcc()

    def compile_one(src):
        obj = os.path.join(OUT_DIR, src.replace(".cu", f"{suffix}.o"))
        r = subprocess.run([nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", os.path.join(CSRC, src), "-o", obj],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    r = subprocess.run([nvcc, "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "shared"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


def build_library(force: bool = False, verbose: bool = False, prof: bool = False, watchdog: bool = False) -> str:
    """prof=True builds libqspec_b200_prof.so with the GEMM cycle counters compiled in (scripts/gpu_gemm_trace.py;
    select it with QSPEC_LIB=<path>); watchdog=True builds libqspec_b200_wd.so whose pipeline waits trap instead of
    hanging (for protocol changes). The product library carries neither."""
    os.makedirs(OUT_DIR, exist_ok=True)
    lib_path = LIB_PATH.replace(".so", "_prof.so") if prof else LIB_PATH.replace(".so", "_wd.so") if watchdog else LIB_PATH
    if not force and os.path.exists(lib_path) and os.path.getmtime(lib_path) >= _newest_source_mtime(SOURCES):
        build_seq_library(force=False, verbose=verbose)
        return lib_path
    build_seq_library(force=force, verbose=verbose)
    nvcc = _nvcc()
    objs = []
    extra = ["-DQSPEC_GEMM_PROF"] if prof else ["-DQSPEC_GEMM_WATCHDOG"] if watchdog else []
    suffix = "_prof.o" if prof else "_wd.o" if watchdog else ".o"

    def compile_one(src):
        obj = os.path.join(OUT_DIR, src.replace(".cu", suffix))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-cudart", "shared"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    if "--seq" in sys.argv:
        print(build_seq_library(force="--force" in sys.argv, verbose=True))
        sys.exit(0)
    print(build_library(force="--force" in sys.argv, verbose=True, prof="--prof" in sys.argv, watchdog="--watchdog" in sys.argv))
