"""Runs unit tests of the reference project against this repository's implementation.

The reference's test modules import `jax_tpu_embedding.sparsecore...`; with this repository's
package first on sys.path those imports resolve to the B200 drop-in.  Modules the tests import
but the hot path does not provide (FDO client, portpicker) are stubbed.  Only usable where the
reference checkout is mounted; nothing here ships.
"""

from __future__ import annotations

import importlib
import importlib.util
import os
import sys
import types
import unittest

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("SC_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference"))
_CORE_TESTS = os.path.join(REFERENCE, "jax_tpu_embedding/sparsecore/lib/core/tests")


def _stub(name, **attrs):
  mod = types.ModuleType(name)
  for k, v in attrs.items():
    setattr(mod, k, v)
  sys.modules[name] = mod
  return mod


def _load(name, path):
  spec = importlib.util.spec_from_file_location(name, path)
  mod = importlib.util.module_from_spec(spec)
  sys.modules[name] = mod
  spec.loader.exec_module(mod)
  return mod


class _NullFdoClient:
  def __init__(self, *a, **k):
    pass

  def record(self, stats):
    pass

  def publish(self):
    pass


def load_pybind_test_module(backend):
  """Imports the reference's pybind_input_preprocessing_test with `backend` as the preprocessor."""
  from absl import flags
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  if not flags.FLAGS.is_parsed():
    flags.FLAGS(["reference_harness"])
  pip.preprocess_sparse_dense_matmul_input = backend
  _stub("portpicker", pick_unused_port=lambda: 0)
  _stub("jax_tpu_embedding.sparsecore.lib.fdo")
  _stub("jax_tpu_embedding.sparsecore.lib.fdo.file_fdo_client", NPZFileFDOClient=_NullFdoClient)
  sys.modules["jax_tpu_embedding.sparsecore.lib.fdo"].file_fdo_client = sys.modules[
      "jax_tpu_embedding.sparsecore.lib.fdo.file_fdo_client"]
  _stub("jax_tpu_embedding.sparsecore.lib.core.tests")
  tu = _load("jax_tpu_embedding.sparsecore.lib.core.tests.test_utils", os.path.join(_CORE_TESTS, "test_utils.py"))
  sys.modules["jax_tpu_embedding.sparsecore.lib.core.tests"].test_utils = tu
  return _load("reference_pybind_input_preprocessing_test",
               os.path.join(_CORE_TESTS, "pybind_input_preprocessing_test.py"))


def load_sparse_coo_test_module(backend):
  """Imports the reference's sparse_coo_input_preprocessing_test: it calls the product's sparse-COO front end, which
  builds row splits on the host and hands them to `backend` through the binding module."""
  load_pybind_test_module(backend)  # same stubs and test_utils
  return _load("reference_sparse_coo_input_preprocessing_test",
               os.path.join(_CORE_TESTS, "sparse_coo_input_preprocessing_test.py"))


def load_fdo_test_module(name: str):
  """Imports the reference's `lib/fdo/<name>.py` test module; it exercises this repository's FDO clients.
  `etils.epath.Path` is pathlib's Path where etils is not installed."""
  import pathlib

  from absl import flags

  if not flags.FLAGS.is_parsed():
    flags.FLAGS(["reference_harness"])
  try:
    import etils.epath  # noqa: F401  pylint: disable=unused-import,g-import-not-at-top
  except ImportError:
    etils = _stub("etils")
    etils.epath = _stub("etils.epath", Path=pathlib.Path)
  for stale in ("jax_tpu_embedding.sparsecore.lib.fdo", "jax_tpu_embedding.sparsecore.lib.fdo.file_fdo_client"):
    mod = sys.modules.get(stale)
    if mod is not None and getattr(mod, "__file__", None) is None:  # a stub left by load_pybind_test_module
      del sys.modules[stale]
  return _load("reference_" + name, os.path.join(REFERENCE, "jax_tpu_embedding/sparsecore/lib/fdo", name + ".py"))


class _StubMesh:
  """Stands in for jax.sharding.Mesh: the tested module reads `devices` only."""

  def __init__(self, devices, axis_names=None):
    import numpy as np

    self.devices = np.asarray(devices, dtype=object)
    self.axis_names = axis_names


def load_python_preprocessing_test_module(backend):
  """Imports the reference's input_preprocessing_test (tests of its pure-Python single-feature module) so that
  `lib.core.input_preprocessing` of this repository is what it exercises, with `backend` as the preprocessor
  behind the product's binding module."""
  from absl import flags
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  if not flags.FLAGS.is_parsed():
    flags.FLAGS(["reference_harness"])
  pip.preprocess_sparse_dense_matmul_input = backend
  if "jax" not in sys.modules:
    jax = _stub("jax")
    jax.sharding = _stub("jax.sharding", Mesh=_StubMesh)
  return _load("reference_input_preprocessing_test", os.path.join(_CORE_TESTS, "input_preprocessing_test.py"))


def set_reference_root(root: str) -> None:
  global REFERENCE, _CORE_TESTS
  REFERENCE = root
  _CORE_TESTS = os.path.join(root, "jax_tpu_embedding/sparsecore/lib/core/tests")


def run_cases(module, skip_classes=("MinibatchingNodeTest",)):
  """Runs every TestCase of `module`; returns (unittest result, number of tests run)."""
  loader = unittest.TestLoader()
  suite = unittest.TestSuite()
  for name in dir(module):
    obj = getattr(module, name)
    if isinstance(obj, type) and issubclass(obj, unittest.TestCase) and name not in skip_classes:
      if obj.__module__ != module.__name__:
        continue
      suite.addTests(loader.loadTestsFromTestCase(obj))
  result = unittest.TextTestRunner(verbosity=0, stream=open(os.devnull, "w")).run(suite)
  return result
