"""Builds libb200ng.so (sm_100a) in-tree with nvcc.  `python ngraph_python_b200/build.py`."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200ng.so")

SOURCES = ["b2_api.cu", "b2_ew_codegen.cu", "b2_flex.cu", "b2_gemm.cu", "b2_conv.cu",
           "b2_dimshuffle.cu", "b2_rng.cu", "b2_comm.cu"]


def _embed_device_header():
    """The helper header is also handed to NVRTC at run time: wrap it in a raw string."""
    src = open(os.path.join(CSRC, "b2_ew_device.cuh")).read()
    assert ')B2SRC"' not in src
    out = os.path.join(CSRC, "b2_ew_device_src.inc")
    text = 'R"B2SRC(' + src + ')B2SRC"\n'
    if not os.path.exists(out) or open(out).read() != text:
        with open(out, "w") as f:
            f.write(text)


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in os.listdir(root):
            if os.path.getmtime(os.path.join(root, name)) > t:
                return True
    return False


def build(force=False, verbose=False):
    _embed_device_header()
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a", "-fmad=false",
           "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES] + ["-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        print(r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
