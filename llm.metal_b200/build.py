"""In-tree build of the native libraries (sm_100a only).

    libllmb200.so        CUDA kernels (csrc/*.cu) + C host engine (host/*.c), static cudart
    libllmb200_synth.so  seeded synthetic models (host/synth.c), no CUDA

Sources are compiled only when they are newer than the library, so importing
the package on a machine that received prebuilt libraries costs nothing.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
INC = os.path.join(ROOT, "include")
OBJ = os.path.join(HERE, "build")

LIB = os.path.join(HERE, "libllmb200.so")
LIB_SYNTH = os.path.join(HERE, "libllmb200_synth.so")

CU_SOURCES = ["pack.cu", "matvec.cu", "attention.cu", "decode_token.cu", "lora_decode.cu", "batch_kernels.cu", "gemm_f32.cu", "gemm_tf32.cu", "train_kernels.cu"]
C_SOURCES = ["weights.c", "decode_engine.c", "sft_engine.c", "batch_engine.c"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _nvcc():
    exe = shutil.which("nvcc") or os.path.join(CUDA_HOME, "bin", "nvcc")
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libllmb200 cannot be built")
    return exe


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout)
        raise RuntimeError("build step failed: " + os.path.basename(cmd[0]))
    return r.stdout


def _headers():
    hs = [os.path.join(INC, f) for f in os.listdir(INC) if f.endswith(".h")]
    hs += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    hs += [os.path.join(HOST, f) for f in os.listdir(HOST) if f.endswith(".h")]
    return hs


def build_main(force=False, verbose=False):
    srcs = [os.path.join(CSRC, f) for f in CU_SOURCES] + [os.path.join(HOST, f) for f in C_SOURCES]
    if not force and not _newer(LIB, srcs + _headers()):
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    objs = []
    for f in CU_SOURCES:
        o = os.path.join(OBJ, f + ".o")
        flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
        out = _run([nvcc] + flags + ["-c", os.path.join(CSRC, f), "-o", o])
        if verbose:
            sys.stderr.write(out)
        objs.append(o)
    for f in C_SOURCES:
        o = os.path.join(OBJ, f + ".o")
        _run(["gcc", "-O2", "-std=gnu11", "-fPIC", "-Wall", "-Wno-unused-function",
              "-I", os.path.join(CUDA_HOME, "include"), "-c", os.path.join(HOST, f), "-o", o])
        objs.append(o)
    _run([nvcc, "-shared", "-o", LIB] + objs + ["-cudart", "static", "-lm", "-lpthread", "-ldl", "-lrt"])
    return LIB


def build_synth(force=False):
    src = os.path.join(HOST, "synth.c")
    if not force and not _newer(LIB_SYNTH, [src] + _headers()):
        return LIB_SYNTH
    _run(["gcc", "-O2", "-std=gnu11", "-fPIC", "-shared", "-ffp-contract=off", "-Wall",
          src, "-o", LIB_SYNTH, "-lm", "-lpthread"])
    return LIB_SYNTH


def build_all(force=False, verbose=False):
    return build_main(force, verbose), build_synth(force)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
