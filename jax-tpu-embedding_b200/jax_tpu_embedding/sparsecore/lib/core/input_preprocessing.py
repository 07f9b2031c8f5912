"""Single-feature preprocessing with the interface of the reference's `lib/core/input_preprocessing.py`.

The reference keeps a readable pure-Python preprocessing of ONE feature next to its C++ one, for tests
and verification (`preprocess_sparse_dense_matmul_input(features, features_weights, mesh, *,
max_ids_per_partition, max_unique_ids_per_partition, num_sc_per_device, ...)`, lib/core/input_preprocessing.py:294-383):
weights are the gains as given (no combiner), ids are not bounded by a vocabulary, the batch is the batch of one
device of the mesh, and the result is the four flat CSR-wrapped COO arrays of that device.  This module offers the
same call on the GPU: it wraps the feature in a one-table spec and runs the kernels behind
`pybind_input_preprocessing`, so the arrays are those of the production path (same sizes and padding as the
reference's: `round_up(max_ids_per_partition, 8) * num_sc_per_device * num_scs` slots, INT_MAX / NaN padding,
`max(num_scs, 8)` row pointers per SparseCore).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing
from jax_tpu_embedding.sparsecore.lib.nn import embedding
from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec
from jax_tpu_embedding.sparsecore.utils import utils


def _device_count(mesh) -> int:
  """Number of devices of `mesh`: an object with a `devices` collection (jax.sharding.Mesh) or a plain int."""
  if isinstance(mesh, (int, np.integer)):
    return int(mesh)
  devices = mesh.devices
  size = getattr(devices, "size", None)
  return int(size) if size is not None else len(devices)


def _rows(batch, what: str):
  """A 2-D array or a sequence of per-sample sequences -> list of 1-D arrays (one per sample)."""
  if isinstance(batch, np.ndarray) and batch.dtype != object:
    if batch.ndim not in (1, 2):
      raise ValueError(f"{what} must be 1D or 2D, got {batch.ndim}D.")
    if batch.ndim == 2:
      return [row for row in batch]
  return [np.asarray(row).reshape(-1) for row in batch]


def preprocess_sparse_dense_matmul_input(features, features_weights, mesh, *, max_ids_per_partition: int,
                                         max_unique_ids_per_partition: int, num_sc_per_device: int = -1,
                                         sharding_strategy: str = "MOD", enable_minibatching: bool = False):
  """(row_pointers, embedding_ids, sample_ids, gains) of one feature's batch, as numpy arrays.

  `features` / `features_weights`: a [batch, valency] array or one sequence of ids / weights per sample.  The batch
  must be a multiple of `num_sc_per_device` (sample i goes to SparseCore i // (batch / num_sc_per_device)).
  Exceeding `max_ids_per_partition` or `max_unique_ids_per_partition` raises ValueError, as does a sharding strategy
  other than "MOD"; minibatching is not available.
  """
  if max_ids_per_partition <= 0:
    raise ValueError(f"max_ids_per_partition must be positive, got {max_ids_per_partition}.")
  if enable_minibatching:
    raise NotImplementedError("minibatching is not available on this backend")
  if len(features) != len(features_weights):
    raise ValueError("features and features_weights must have the same length.")
  if sharding_strategy != "MOD":
    raise ValueError("Currently only MOD sharding strategy is supported")
  global_device_count = _device_count(mesh)
  if global_device_count <= 0:
    raise ValueError("global_device_count must be positive.")
  if num_sc_per_device <= 0:
    num_sc_per_device = utils.num_sparsecores_per_device()
  id_rows, weight_rows = _rows(features, "features"), _rows(features_weights, "features_weights")
  for i, (ids, weights) in enumerate(zip(id_rows, weight_rows)):
    if len(ids) != len(weights):
      raise ValueError(f"sample {i} has {len(ids)} ids and {len(weights)} weights")
  batch = len(id_rows)
  largest = max((int(np.max(r)) for r in id_rows if len(r)), default=0)
  # One table that holds every id of the batch: stacking leaves ids, sample ids and gains as they are.
  table = embedding_spec.TableSpec(
      name="table", vocabulary_size=largest + 1, embedding_dim=8, initializer=None,
      optimizer=embedding_spec.SGDOptimizerSpec(), combiner="sum", max_ids_per_partition=int(max_ids_per_partition),
      max_unique_ids_per_partition=int(max_unique_ids_per_partition))
  feature = embedding_spec.FeatureSpec(name="feature", table_spec=table, input_shape=[batch * global_device_count, 1],
                                       output_shape=[batch * global_device_count, 8])
  embedding.prepare_feature_specs_for_training([feature], global_device_count=global_device_count,
                                               num_sc_per_device=num_sc_per_device)
  ragged_ids, ragged_weights = np.empty(batch, dtype=object), np.empty(batch, dtype=object)
  for i, (ids, weights) in enumerate(zip(id_rows, weight_rows)):
    ragged_ids[i] = np.asarray(ids, dtype=np.int32)
    ragged_weights[i] = np.asarray(weights, dtype=np.float32)
  rp, ids, sids, gains, _, _ = pybind_input_preprocessing.preprocess_sparse_dense_matmul_input(
      [ragged_ids], [ragged_weights], [feature], 1, global_device_count, num_sc_per_device=num_sc_per_device,
      device_output=False)
  name = table.stacked_table_spec.stack_name
  return (np.asarray(rp[name]).reshape(-1), np.asarray(ids[name]).reshape(-1), np.asarray(sids[name]).reshape(-1),
          np.asarray(gains[name]).reshape(-1))
