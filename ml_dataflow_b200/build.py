"""Builds the C-ABI library (ml_dataflow_b200/lib/libb200moe.so) with nvcc for sm_100a.

Usage: python -m ml_dataflow_b200.build [--force]
nvcc cross-compiles without a GPU; the .so is kept in-tree next to the sources.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libb200moe.so")
SOURCES = ["router.cu", "permute.cu", "ep_p2p.cu", "gemm_sm100.cu", "moe_block.cu", "model_files.cu", "ep_block.cu", "block_ops.cu", "attention.cu",
           "attention_sm100.cu", "transformer_block.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _newest_source_mtime():
    newest = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for name in os.listdir(root):
            newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def build(force=False, verbose=False):
    os.makedirs(LIB_DIR, exist_ok=True)
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + [
        os.path.join(CSRC, s) for s in SOURCES
    ]
    subprocess.check_call(cmd)
    return LIB_PATH


MICROBENCH = ["mma_queue_probe", "tma_feed_probe"]


def build_microbench(force=False):
    """The two stand-alone probes of the tensor pipe and the TMA feed (csrc/microbench/*.cu) as executables under
    lib/microbench/ (built artefacts, not tracked). They measure the hardware figures the GEMM's design rests on."""
    out_dir = os.path.join(LIB_DIR, "microbench")
    os.makedirs(out_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    paths = []
    for name in MICROBENCH:
        src, exe = os.path.join(CSRC, "microbench", name + ".cu"), os.path.join(out_dir, name)
        newest = max(os.path.getmtime(src), os.path.getmtime(os.path.join(CSRC, "sm100_ptx.cuh")))
        if force or not os.path.exists(exe) or os.path.getmtime(exe) < newest:
            subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
                                   "-o", exe, src])
        paths.append(exe)
    return paths


ADAPTER_SRC = os.path.join(HERE, "backends", "nvidia", "b200_dataflow_ops.c")
ADAPTER_PATH = os.path.join(LIB_DIR, "libb200moe_dataflow.so")


def build_adapter(reference_root=None, force=False):
    """Builds the external-op adapter (C) against the reference's headers in place. Needs the reference tree.

    Returns the path of the .so, or None when the reference tree is not present on this machine.
    """
    reference_root = (reference_root or os.environ.get("REFERENCE_ROOT")
                      or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
    if not os.path.isdir(os.path.join(reference_root, "libdataflowops", "include")):
        return ADAPTER_PATH if os.path.exists(ADAPTER_PATH) else None
    build(force=False)
    if not force and os.path.exists(ADAPTER_PATH) and os.path.getmtime(ADAPTER_PATH) >= max(
            os.path.getmtime(ADAPTER_SRC), os.path.getmtime(LIB_PATH)):
        return ADAPTER_PATH
    inc = [os.path.join(reference_root, p) for p in ("libdataflow/include", "libdataflowops/include",
                                                     "backends/nvidia/include")]
    inc += [os.path.join(os.path.dirname(HERE), "include"), "/usr/local/cuda/include"]
    if not os.path.exists("/usr/include/numa.h"):
        inc.append(os.path.join(HERE, "backends", "nvidia", "compat"))
    cmd = [os.environ.get("HOST_CC", "/usr/bin/gcc"), "-O2", "-fPIC", "-shared", "-w"] + ["-I" + i for i in inc]
    cmd += ["-o", ADAPTER_PATH, ADAPTER_SRC, "-L" + LIB_DIR, "-lb200moe", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    return ADAPTER_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_adapter(force="--force" in sys.argv))
