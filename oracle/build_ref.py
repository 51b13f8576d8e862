"""Build ``oracle/_ref/``: the reference's own residual-codec kernels, compiled for the CPU.

TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [/path/to/latentQ_LLM]

The kernels of ``utils/cuda_src/multi_random_quant_kernel.cu`` are plain C arithmetic per thread.  This
recipe lifts the kernel definitions and the constant set-up statements of the launchers out of the
reference checkout WHERE IT LIES into ``oracle/_ref/*.inc`` (git-ignored, never committed), and compiles
``ref_codec_driver.cpp`` around them with g++: a host loop plays the thread index, ``ref_codec_shim.h``
supplies the handful of CUDA names the text uses.  Nothing is launched on a GPU (the reference's launcher
passes 0 bytes of dynamic shared memory to kernels that index 40 bytes of it, so the kernel itself must not
run on a shared GPU).

Two libraries are produced because nvcc contracts ``a*b+c`` into an FMA by default and the reference builds
with nvcc's defaults:

    oracle/_ref/libref_codec_fma.so     g++ -ffp-contract=fast -mfma   (what nvcc's default computes)
    oracle/_ref/libref_codec_nofma.so   g++ -ffp-contract=off          (the separately rounded reading)

``tests/golden/gen_golden.py`` runs both and stores their outputs as fixtures; ``tests/test_oracle_golden.py``
pins ``lq_oracle.c`` to the FMA variant and shows where the two differ.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REF = "/root/reference"
KERNEL_FILE = os.path.join("utils", "cuda_src", "multi_random_quant_kernel.cu")


def _body_until(lines, start_pat, stop_pat):
    """Statements of a launcher between its signature line and the first line matching stop_pat."""
    i = next(k for k, ln in enumerate(lines) if re.search(start_pat, ln))
    out = []
    for ln in lines[i + 1:]:
        if re.search(stop_pat, ln):
            break
        out.append(ln)
    return out


def extract(ref_root: str) -> None:
    path = os.path.join(ref_root, KERNEL_FILE)
    lines = open(path).read().split("\n")
    first = next(k for k, ln in enumerate(lines) if ln.startswith("__global__"))
    last = next(k for k, ln in enumerate(lines) if ln.startswith("#define THREADS_PER_BLOCK"))
    parts = {
        "kernels.inc": lines[first:last],
        "launch_quant_consts.inc": _body_until(lines, r"^void launch_quant\(", r"src\.dtype\(\)"),
        "launch_dequant_consts.inc": _body_until(lines, r"^void launch_dequant\(", r"tgt\.dtype\(\)"),
        "launch_quant_linear_consts.inc": _body_until(lines, r"^void launch_quant_linear\(", r"src\.dtype\(\)"),
    }
    os.makedirs(OUT, exist_ok=True)
    for name, body in parts.items():
        with open(os.path.join(OUT, name), "w") as f:
            f.write(f"// extracted at build time from {KERNEL_FILE} of the reference checkout; not committed\n")
            f.write("\n".join(body) + "\n")


VARIANTS = {"fma": ["-ffp-contract=fast", "-mfma"], "nofma": ["-ffp-contract=off"]}


def lib_path(variant: str) -> str:
    return os.path.join(OUT, f"libref_codec_{variant}.so")


def build(ref_root: str = DEFAULT_REF) -> dict:
    extract(ref_root)
    out = {}
    for variant, flags in VARIANTS.items():
        so = lib_path(variant)
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-fwrapv",
                               "-fno-fast-math", *flags, "-I", HERE, "-o", so,
                               os.path.join(HERE, "ref_codec_driver.cpp")])
        out[variant] = so
    return out


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REF))
