"""Builds the sm_100a shared library (and the llama2_q4 command-line program) in-tree with nvcc.

    python -m llama_cu_awq_b200.build [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libq4b200.so")
CLI = os.path.join(HERE, "llama2_q4")
LIB_SOURCES = ["q4_gemv.cu", "q4_ops.cu", "q4_attn.cu", "q4_comm.cu", "q4_model.cu", "q4_fused.cu", "q4_sampler.cu"]
CLI_SOURCES = ["llama2_q4_main.cpp"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _deps():
    out = [os.path.join(HERE, "..", "include", "q4b200.h")]
    for f in os.listdir(CSRC):
        out.append(os.path.join(CSRC, f))
    return out


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "nvcc")
    deps = _deps()
    if force or _newer(LIB, deps):
        cmd = [nvcc] + NVCC_FLAGS + ["-Xcompiler", "-fPIC", "-shared", "-o", LIB] + [os.path.join(CSRC, s) for s in LIB_SOURCES]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.run(cmd, check=True)
    cli_srcs = [os.path.join(CSRC, s) for s in CLI_SOURCES]
    if all(os.path.exists(s) for s in cli_srcs) and (force or _newer(CLI, deps + [LIB])):
        cmd = [nvcc] + NVCC_FLAGS + ["-o", CLI] + cli_srcs + [LIB, "-Xlinker", "-rpath=$ORIGIN", "-lpthread"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
