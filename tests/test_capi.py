"""The C-ABI library loads without a GPU and exports every symbol include/sc_b200.h declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
  text = open(os.path.join(ROOT, "include", "sc_b200.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  return sorted(set(re.findall(r"\b(sc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_all_declared_symbols():
  from jax_tpu_embedding.sparsecore import _native

  if not _native.available():
    import __graft_entry__

    __graft_entry__.build()
  lib = ctypes.CDLL(_native.LIB_PATH)
  names = _declared_symbols()
  assert len(names) >= 15
  for name in names:
    assert hasattr(lib, name), f"{name} is declared in sc_b200.h but not exported"


def test_sizing_functions_match_reference_arithmetic():
  """Values from the reference's PybindBufferSizeTest
  (lib/core/tests/pybind_input_preprocessing_test.py:1990-2057) and input_preprocessing_util_test.cc:99-133."""
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  assert pip.compute_row_pointers_size_per_device(global_device_count=2, num_sc_per_device=4) == 32
  assert pip.compute_row_pointers_size_per_device(global_device_count=1, num_sc_per_device=1) == 8
  assert pip.compute_row_pointers_size_per_device(global_device_count=8, num_sc_per_device=4) == 128
  assert pip.compute_theoretical_max_coo_buffer_size(100, 2, 4) == 104 * 4 * 8
  assert pip.compute_theoretical_max_coo_buffer_size(8, 1, 1) == 8
  with pytest.raises(NotImplementedError):
    pip.compute_row_pointers_size_per_device(1, 1, enable_minibatching=True)


def test_status_names_and_errors():
  from jax_tpu_embedding.sparsecore import _native

  lib = _native.lib()
  assert lib.sc_version() >= 100
  assert lib.sc_status_name(0) == b"OK" and lib.sc_status_name(3) == b"ID_LIMIT_EXCEEDED"
  assert lib.sc_compute_coo_buffer_size_per_device(8, 1, 1, 64) == -1
  assert "theoretical max" in _native.last_error()
  with pytest.raises(ValueError):
    _native.check(_native.SC_INVALID_ARGUMENT)
  with pytest.raises(RuntimeError):
    _native.check(_native.SC_CUDA_ERROR)


def test_operators_fail_loudly_without_gpu():
  import numpy as np
  import torch

  if torch.cuda.is_available():
    pytest.skip("a GPU is present")
  from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_csr as op

  z = np.zeros(8, np.int32)
  with pytest.raises(RuntimeError, match="no CPU fallback"):
    op.tpu_sparse_dense_matmul_csr_primitive.bind(
        z, z, z, np.zeros(8, np.float32), np.int32(1), np.zeros((8, 8), np.float32), device_batch_size=8,
        max_ids_per_partition=8, max_unique_ids_per_partition=8)
