"""Build recipe for the test oracle (TEST INFRASTRUCTURE ONLY).

Two artefacts:

* ``oracle/liboracle.so``  -- the C restatement of FastNN's CPU matmul path
  (``fastnn_cpu_oracle.c``), built with gcc, contraction off.
* ``oracle/_ref/libfastnn_ref.so`` -- FastNN's own ``cuda/kernels.cu`` compiled,
  unmodified and from where it lies, for sm_100a and linked against cuBLAS and
  cuRAND.  It is the reference's GPU implementation of the same entry points
  (cuBLAS TF32) and is used only to validate the oracle and as a timed
  comparator.  It is built only when the reference checkout is present; the
  prebuilt file travels with the tree otherwise.

Neither artefact may be loaded by the product path.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libfastnn_ref.so")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "fastnn_cpu_oracle.c")
    if not force and _newer(ORACLE_SO, src, __file__):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fvisibility=hidden",
           "-shared", "-fPIC", "-pthread", "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_reference(reference_root: str | None = None, force: bool = False) -> str | None:
    """Compile the reference's own GPU library when its checkout is available: the directory
    given, else $FASTNN_REFERENCE_ROOT, else a `reference` directory beside this repository."""
    root = reference_root or os.environ.get("FASTNN_REFERENCE_ROOT") or \
        os.path.join(os.path.dirname(HERE), os.pardir, "reference")
    src = os.path.join(root, "cuda", "kernels.cu")
    if not os.path.exists(src):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, src):
        return REF_SO
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(REF_DIR, exist_ok=True)
    # Flags of the reference's build.rs:49-51, with the sm_100a target it lacks.
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math",
           "--extended-lambda", "-O3", "-I", os.path.join(root, "cuda", "include"),
           "-shared", "-Xcompiler", "-fPIC", "-o", REF_SO, src,
           "-lcublas", "-lcurand"]
    subprocess.check_call(cmd)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
