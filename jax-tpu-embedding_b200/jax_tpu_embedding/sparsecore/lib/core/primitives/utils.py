"""Operand validation shared by the SparseCore operators.

Same checks, in the same order and with the same messages, as
`validate_abstract_eval_params` / `ensure_dtype` / `ensure_dim` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/utils.py:62-160); operands are
numpy arrays or torch tensors instead of JAX abstract values.
"""

from __future__ import annotations

from typing import Any

import numpy as np


_DTYPE_CACHE: dict = {}


def _np_dtype(x) -> np.dtype:
  """dtype of a numpy array, numpy/python scalar or torch tensor as a numpy dtype."""
  dt = getattr(x, "dtype", None)
  if dt is None:
    if isinstance(x, bool):
      return np.dtype(bool)
    if isinstance(x, int):
      return np.dtype(np.int32)  # python ints are weakly typed, as in JAX
    if isinstance(x, float):
      return np.dtype(np.float32)
    return np.asarray(x).dtype
  cached = _DTYPE_CACHE.get(dt)
  if cached is None:
    if type(dt).__module__.startswith("torch"):
      cached = np.dtype(str(dt).replace("torch.", ""))
    else:
      cached = np.dtype(dt)
    _DTYPE_CACHE[dt] = cached
  return cached


def _shape(x) -> tuple[int, ...]:
  return tuple(getattr(x, "shape", ()))


def ensure_dtype(check: Any, expected_type: Any, object_name: str):
  if _np_dtype(check) != np.dtype(expected_type):
    raise ValueError(f"{object_name} must have type {expected_type!r}, got {_np_dtype(check)!r}")


def ensure_dim(check: Any, expected_dim: int | tuple[int, ...], object_name: str):
  expected = (expected_dim,) if isinstance(expected_dim, int) else expected_dim
  if len(_shape(check)) not in expected:
    raise ValueError(f"{object_name} must have dim in {expected!r}, got {_shape(check)!r}")


def get_embedding_dim(val) -> int:
  shape = _shape(val)
  return shape[1] if len(shape) > 1 else 1


def validate_abstract_eval_params(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
                                  num_minibatches_per_physical_sparse_core, embedding_table, activations_grad,
                                  max_ids_per_partition: int, max_unique_ids_per_partition: int,
                                  computation_name: str, sharding_strategy: int, min_value: float | None = None,
                                  max_value: float | None = None):
  """Raises ValueError for any operand or attribute the operators cannot accept."""
  ensure_dtype(lhs_row_pointers, np.int32, "lhs_row_pointers")
  ensure_dtype(lhs_local_sample_ids, np.int32, "lhs_local_sample_ids")
  ensure_dtype(lhs_local_embedding_ids, np.int32, "lhs_local_embedding_ids")
  ensure_dtype(lhs_gains, np.float32, "lhs_gains")
  ensure_dtype(num_minibatches_per_physical_sparse_core, np.int32, "num_minibatches_per_physical_sparse_core")
  ensure_dtype(embedding_table, np.float32, "embedding_table")
  ensure_dtype(activations_grad, np.float32, "activations_grad")
  ensure_dim(lhs_row_pointers, 1, "lhs_row_pointers")
  ensure_dim(embedding_table, (1, 2), "embedding_table")
  ensure_dim(num_minibatches_per_physical_sparse_core, 0, "num_minibatches_per_physical_sparse_core")
  ensure_dim(activations_grad, (1, 2), "activations_grad")
  if (_shape(lhs_local_sample_ids) != _shape(lhs_local_embedding_ids)
      or _shape(lhs_gains) != _shape(lhs_local_embedding_ids) or len(_shape(lhs_local_sample_ids)) != 1):
    raise ValueError(
        "LHS sample IDs, embedding IDs, and gains must all have equal rank 1 shapes, got shapes "
        f"{_shape(lhs_local_sample_ids)}, {_shape(lhs_local_embedding_ids)} and {_shape(lhs_gains)}")
  if get_embedding_dim(embedding_table) != get_embedding_dim(activations_grad):
    raise ValueError(
        "embedding_table and activations_grad must have equal feature (minor) dimensions, got "
        f"{_shape(embedding_table)}, {_shape(activations_grad)}")
  if sharding_strategy != 1:
    raise ValueError(f"sharding_strategy must be MOD (1), got {sharding_strategy}")
  if max_ids_per_partition <= 0:
    raise ValueError(f"max_ids_per_partition must be positive, got {max_ids_per_partition}")
  if max_unique_ids_per_partition <= 0:
    raise ValueError(f"max_unique_ids_per_partition must be positive, got {max_unique_ids_per_partition}")
  if not computation_name:
    raise ValueError("computation_name must be non-empty")
  if min_value is not None and max_value is not None and min_value > max_value:
    raise ValueError(f"min_value must be less than or equal to max_value, got {min_value} and {max_value}")


class _Shaped:
  """Stand-in operand with only a shape and a dtype (for checks that need no data)."""

  def __init__(self, shape, dtype):
    self.shape = tuple(shape)
    self.dtype = np.dtype(dtype)
