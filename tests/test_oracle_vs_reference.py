"""Pins the CPU oracle (and the spec layer) to the reference project.

1. The reference's own unit tests for the preprocessing binding
   (jax_tpu_embedding/sparsecore/lib/core/tests/pybind_input_preprocessing_test.py: hand-written
   golden buffers, statistics, buffer sizes, error cases) are executed with the oracle behind the
   product's Python interface.
2. The oracle is compared with the reference's pure-Python preprocessing
   (lib/core/input_preprocessing.py) on random single-feature inputs.
3. The reference's unit tests of that pure-Python module run against this repository's module of
   the same name (oracle as the backend).
4. The reference's unit tests of the sparse-COO input run against the product's sparse-COO front end
   (oracle as the backend).
5. The reference's unit tests of its FDO clients run against the FDO clients of this repository.
Both need the reference checkout and are skipped where it is not mounted; the committed
fixtures under tests/golden/ carry the same pin to machines without it.
"""

import importlib.util
import os
import sys
import types

import numpy as np
import pytest

import oracle_backend as ob
from oracle import preprocess_oracle as po


def test_reference_unit_tests_pass_on_oracle(reference_root):
  import reference_harness as rh
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  original = pip.preprocess_sparse_dense_matmul_input
  try:
    module = rh.load_pybind_test_module(ob.oracle_preprocess)
    result = rh.run_cases(module)
  finally:
    pip.preprocess_sparse_dense_matmul_input = original
  assert result.testsRun >= 30
  problems = [str(t) + "\n" + tb for t, tb in result.failures + result.errors]
  assert not problems, "\n".join(problems)[:4000]


@pytest.mark.parametrize("name,count", [("file_fdo_client_test", 5), ("csv_file_fdo_client_test", 6)])
def test_reference_fdo_client_tests_pass_on_these_clients(reference_root, name, count):
  """lib/fdo/file_fdo_client_test.py and csv_file_fdo_client_test.py against `lib/fdo` of this repository."""
  import reference_harness as rh

  result = rh.run_cases(rh.load_fdo_test_module(name))
  assert result.testsRun >= count
  problems = [str(t) + "\n" + tb for t, tb in result.failures + result.errors]
  assert not problems, "\n".join(problems)[:4000]


def test_reference_sparse_coo_tests_pass_on_this_front_end(reference_root):
  """lib/core/tests/sparse_coo_input_preprocessing_test.py (16 cases with hand-written buffers: empty rows, column
  transformations, feature and table stacking on one and several chips) against the product's sparse-COO front end
  (`preprocess_sparse_dense_matmul_sparse_coo_input`), with the oracle behind it."""
  import reference_harness as rh
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  original = pip.preprocess_sparse_dense_matmul_input
  try:
    module = rh.load_sparse_coo_test_module(ob.oracle_preprocess)
    result = rh.run_cases(module)
  finally:
    pip.preprocess_sparse_dense_matmul_input = original
  assert result.testsRun >= 16
  problems = [str(t) + "\n" + tb for t, tb in result.failures + result.errors]
  assert not problems, "\n".join(problems)[:4000]


def test_reference_tests_of_its_python_module_pass_on_this_module(reference_root):
  """lib/core/tests/input_preprocessing_test.py (hand-written expected buffers for one and several id columns,
  error cases) exercises `lib.core.input_preprocessing` of this repository, with the oracle behind the binding
  module.  The minibatching test class is skipped: minibatching is not built."""
  import reference_harness as rh
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  original = pip.preprocess_sparse_dense_matmul_input
  try:
    module = rh.load_python_preprocessing_test_module(ob.oracle_preprocess)
    result = rh.run_cases(module, skip_classes=("InputPreprocessingMinibatchingTest",))
  finally:
    pip.preprocess_sparse_dense_matmul_input = original
  assert result.testsRun >= 7
  problems = [str(t) + "\n" + tb for t, tb in result.failures + result.errors]
  assert not problems, "\n".join(problems)[:4000]


def _load_reference_python_preprocessing(root):
  """Imports lib/core/input_preprocessing.py with numpy standing in for jax.numpy."""
  saved = {k: sys.modules.get(k) for k in ("jax", "jax.numpy", "jax.sharding")}
  jax = types.ModuleType("jax")
  jnp = types.ModuleType("jax.numpy")
  jnp.asarray, jnp.ndarray, jnp.int32, jnp.float32 = np.asarray, np.ndarray, np.int32, np.float32
  sharding = types.ModuleType("jax.sharding")
  sharding.Mesh = object
  jax.numpy, jax.sharding = jnp, sharding
  sys.modules.update({"jax": jax, "jax.numpy": jnp, "jax.sharding": sharding})
  try:
    path = os.path.join(root, "jax_tpu_embedding/sparsecore/lib/core/input_preprocessing.py")
    spec = importlib.util.spec_from_file_location("reference_python_preprocessing", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
  finally:
    for k, v in saved.items():
      if v is None:
        sys.modules.pop(k, None)
      else:
        sys.modules[k] = v
  return mod


class _Mesh:
  def __init__(self, n):
    self.devices = list(range(n))


def test_oracle_matches_reference_python_preprocessing(reference_root):
  ref = _load_reference_python_preprocessing(reference_root)
  rng = np.random.default_rng(0)
  for _ in range(150):
    c, s = int(rng.choice([1, 2, 4])), int(rng.choice([1, 2, 4]))
    batch = s * int(rng.integers(1, 9))
    vocab = int(rng.choice([16, 64, 1000]))
    rows = [rng.integers(0, vocab, size=rng.integers(0, 7)).astype(np.int32) for _ in range(batch)]
    # Power-of-two weights: the reference sums duplicates in double, the C++ (and oracle) in float.
    weights = [rng.choice([0.5, 1.0, 2.0, 0.25], size=len(r)).astype(np.float32) for r in rows]
    rp, ids, sids, gains = ref.preprocess_sparse_dense_matmul_input(
        rows, weights, _Mesh(c), max_ids_per_partition=64, max_unique_ids_per_partition=64, num_sc_per_device=s)
    out = po.preprocess_table([po.FeatureInput(*po.flatten_feature(rows, weights))], local_device_count=1,
                              global_device_count=c, num_sc_per_device=s, combiner="sum", max_ids_per_partition=64,
                              max_unique_ids_per_partition=64)
    assert out["status"] == 0
    ob.written_region_equal(out["row_pointers"][0], rp, [out["embedding_ids"][0], out["sample_ids"][0], out["gains"][0]],
                            [np.asarray(ids), np.asarray(sids), np.asarray(gains, np.float32)], s)
