"""Builds the C restatement of the reference preprocessing (test infrastructure).

TEST INFRASTRUCTURE - NOT THE PRODUCT.  Produces ``oracle/libsc_oracle.so`` from
``oracle/sc_oracle.c`` with plain gcc.  The reference's own C++ preprocessing
cannot be compiled beside it: it needs bazel, abseil, Eigen, XLA/TSL, highway and
highwayhash, none of which exist in this image, so there is no ``oracle/_ref``.
"""

import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(_HERE, "sc_oracle.c")
LIB = os.path.join(_HERE, "libsc_oracle.so")


def build(force: bool = False) -> str:
  """Compiles the oracle if the library is missing or older than its source."""
  if (
      not force
      and os.path.exists(LIB)
      and os.path.getmtime(LIB) >= os.path.getmtime(SRC)
  ):
    return LIB
  # No -march=native: the library is built on one machine and may be loaded on
  # another.  -ffp-contract=off keeps every f32 operation separately rounded,
  # as the restated C++ is on x86-64 without FMA contraction.
  cmd = [
      "gcc", "-O3", "-std=c11", "-ffp-contract=off", "-fPIC", "-shared",
      "-o", LIB, SRC, "-lm", "-lpthread",
  ]
  subprocess.run(cmd, check=True)
  return LIB


if __name__ == "__main__":
  print(build(force=True))
