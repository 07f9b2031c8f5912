"""pytest configuration: import paths and the `gpu` marker."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "jax-tpu-embedding_b200")
for p in (ROOT, PKG, os.path.dirname(os.path.abspath(__file__))):
  if p not in sys.path:
    sys.path.insert(0, p)

# Checkout of the reference project: $SC_REFERENCE_ROOT, else a "reference" directory beside this repository.
REFERENCE = os.environ.get("SC_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def has_gpu() -> bool:
  try:
    import torch

    return torch.cuda.is_available()
  except Exception:  # pylint: disable=broad-except
    return False


def pytest_collection_modifyitems(config, items):
  if has_gpu():
    return
  skip = pytest.mark.skip(reason="no CUDA device")
  for item in items:
    if "gpu" in item.keywords:
      item.add_marker(skip)


@pytest.fixture(scope="session")
def reference_root():
  if not os.path.isdir(REFERENCE):
    pytest.skip("reference checkout not mounted")
  return REFERENCE
