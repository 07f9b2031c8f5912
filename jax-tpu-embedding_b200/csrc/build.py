"""Builds libsc_b200.so (sm_100a only) from the CUDA sources in this directory."""

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(os.path.dirname(_HERE))
SOURCES = ["sc_api.cu", "sc_lookup.cu", "sc_preprocess.cu"]
HEADERS = ["sc_common.cuh", "sc_sort.cuh", os.path.join(_ROOT, "include", "sc_b200.h")]
LIB = os.path.join(os.path.dirname(_HERE), "jax_tpu_embedding", "sparsecore", "libsc_b200.so")


def _newest(paths):
  return max(os.path.getmtime(p if os.path.isabs(p) else os.path.join(_HERE, p)) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
  if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest(SOURCES + HEADERS + [__file__]):
    return LIB
  nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
  cmd = [
      nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
      # Separately rounded multiply and add: sequential float32 sums match a CPU loop.
      "-fmad=false",
      "-Xcompiler", "-fPIC", "-shared", "-I", os.path.join(_ROOT, "include"), "-I", _HERE,
      "-o", LIB,
  ] + [os.path.join(_HERE, s) for s in SOURCES]
  if verbose:
    cmd.insert(1, "-Xptxas")
    cmd.insert(2, "-v")
  subprocess.run(cmd, check=True)
  return LIB


if __name__ == "__main__":
  print(build(force=True, verbose="-v" in sys.argv))
