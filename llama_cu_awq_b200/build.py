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
TEST_LIB = os.path.join(HERE, "libq4b200_test.so")
PACKER = os.path.join(HERE, "weight_packer")   # offline tool, host code only
TEST_BUILD_SOURCES = ["q4_comm.cu", "q4_fused.cu"]   # the sources that look at Q4_TEST_BUILD
LIB_SOURCES = ["q4_gemv.cu", "q4_ops.cu", "q4_attn.cu", "q4_comm.cu", "q4_model.cu", "q4_fused.cu", "q4_sampler.cu", "q4_synth.cu", "q4_tokenizer.cu", "q4_gemm.cu", "q4_skinny.cu", "q4_batch.cu"]
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


def _compile(nvcc, src, obj, extra):
    os.makedirs(os.path.dirname(obj), exist_ok=True)
    subprocess.run([nvcc] + NVCC_FLAGS + extra + ["-Xcompiler", "-fPIC", "-c", "-o", obj, src], check=True)
    return obj


def build(force=False, verbose=False, test=True):
    """Builds libq4b200.so (the product), the llama2_q4 program and, with test=True, libq4b200_test.so: the same
    sources with -DQ4_TEST_BUILD, which adds the measurement switches and host-side fault injectors the tests use."""
    from concurrent.futures import ThreadPoolExecutor
    nvcc = os.environ.get("NVCC", "nvcc")
    deps = _deps()
    objdir = os.path.join(HERE, "build")
    extra = ["-Xptxas=-v"] if verbose else []
    need_lib = force or _newer(LIB, deps)
    need_test = test and (force or _newer(TEST_LIB, deps))
    jobs = []
    if need_lib or need_test:
        for s in LIB_SOURCES:
            jobs.append((os.path.join(CSRC, s), os.path.join(objdir, s + ".o"), extra))
    if need_test:
        for s in TEST_BUILD_SOURCES:
            jobs.append((os.path.join(CSRC, s), os.path.join(objdir, s + ".test.o"), extra + ["-DQ4_TEST_BUILD"]))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _compile(nvcc, *j), jobs))
    link = [nvcc] + NVCC_FLAGS + ["-Xcompiler", "-fPIC", "-shared"]
    if need_lib or need_test:
        subprocess.run(link + ["-o", LIB] + [os.path.join(objdir, s + ".o") for s in LIB_SOURCES] + ["-ldl"], check=True)
    if need_test:
        objs = [os.path.join(objdir, s + (".test.o" if s in TEST_BUILD_SOURCES else ".o")) for s in LIB_SOURCES]
        subprocess.run(link + ["-o", TEST_LIB] + objs + ["-ldl"], check=True)
    cli_srcs = [os.path.join(CSRC, s) for s in CLI_SOURCES]
    if all(os.path.exists(s) for s in cli_srcs) and (force or _newer(CLI, deps + [LIB])):
        cmd = [nvcc] + NVCC_FLAGS + ["-o", CLI] + cli_srcs + [LIB, "-Xlinker", "-rpath=$ORIGIN", "-lpthread"]
        subprocess.run(cmd, check=True)
    packer_src = os.path.join(CSRC, "weight_packer.cpp")
    if os.path.exists(packer_src) and (force or _newer(PACKER, [packer_src])):
        subprocess.run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-o", PACKER, packer_src], check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
