"""Adapters that let the CPU oracle stand behind the product's Python interfaces (tests only)."""

from __future__ import annotations

import numpy as np

from oracle import preprocess_oracle as po
from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip


def oracle_preprocess(features, feature_weights, feature_specs, local_device_count, global_device_count, *,
                      num_sc_per_device, sharding_strategy=pip.ShardingStrategy.MOD, has_leading_dimension=False,
                      allow_id_dropping=False, batch_number=0, enable_minibatching=False, all_reduce_interface=None,
                      device_output=False, num_threads=1):
  """Same signature and return value as the product's preprocess function, computed by the oracle."""
  del batch_number, all_reduce_interface, device_output
  if enable_minibatching:
    raise NotImplementedError
  if int(sharding_strategy) != 1:
    raise ValueError("Only mod sharding is supported for now.")
  features = list(features)
  feature_specs = list(feature_specs)
  if (local_device_count <= 0 or global_device_count <= 0 or global_device_count < local_device_count
      or num_sc_per_device <= 0 or (num_sc_per_device * global_device_count) & (num_sc_per_device * global_device_count - 1)):
    _raise_invalid(local_device_count, global_device_count, num_sc_per_device)
  if not features:
    raise ValueError("input_batches cannot be empty.")
  rp, ids, sids, gains = {}, {}, {}, {}
  stats = pip.SparseDenseMatmulInputStats()
  for stack_name, members in pip._group_by_stack(feature_specs).items():  # pylint: disable=protected-access
    stacked = members[0][1].table_spec.stacked_table_spec
    feats = []
    for idx, spec in members:
      w = None if feature_weights is None else feature_weights[idx]
      feature = features[idx]
      if isinstance(feature, pip.RaggedInput):  # flat values + row splits (what the sparse-COO front end builds)
        splits = np.asarray(feature.row_splits).reshape(-1)
        values = np.asarray(feature.values)
        if feature.weights is not None:
          w = [np.asarray(feature.weights)[a:b] for a, b in zip(splits[:-1], splits[1:])]
        feature = [values[a:b] for a, b in zip(splits[:-1], splits[1:])]
      f_ids, f_off, f_w = po.flatten_feature(feature, w)
      row_offset, col_offset, col_shift = pip._transform(spec)  # pylint: disable=protected-access
      feats.append(po.FeatureInput(f_ids, f_off, f_w, row_offset, col_offset, col_shift))
    out = po.preprocess_table(
        feats, local_device_count=local_device_count, global_device_count=global_device_count,
        num_sc_per_device=num_sc_per_device, combiner=stacked.combiner,
        max_ids_per_partition=stacked.max_ids_per_partition,
        max_unique_ids_per_partition=stacked.max_unique_ids_per_partition, allow_id_dropping=allow_id_dropping,
        suggested_coo_buffer_size_per_device=stacked.suggested_coo_buffer_size_per_device, num_threads=num_threads)
    if out["status"] == po.INVALID_ARGUMENT:
      _raise_invalid(local_device_count, global_device_count, num_sc_per_device)
    if out["status"] == po.ID_LIMIT_EXCEEDED:
      raise ValueError(f"Observed max ids per partition for table: {stack_name} is greater than the set limit")
    arrays = [out["row_pointers"], out["embedding_ids"], out["sample_ids"], out["gains"]]
    if not has_leading_dimension:
      arrays = [a.reshape(-1) for a in arrays]
    rp[stack_name], ids[stack_name], sids[stack_name], gains[stack_name] = arrays
    stats.max_ids_per_partition[stack_name] = out["max_ids_per_partition"]
    stats.max_unique_ids_per_partition[stack_name] = out["max_unique_ids_per_partition"]
    stats.required_buffer_sizes[stack_name] = out["required_buffer_sizes"]
    stats.dropped_id_count[stack_name] = out["dropped_id_count"]
  return rp, ids, sids, gains, 1, stats


def _raise_invalid(l, c, s):
  if l <= 0:
    raise ValueError(f"local_device_count must be greater than 0, but got {l}")
  if c <= 0:
    raise ValueError(f"global_device_count must be greater than 0, but got {c}")
  if c < l:
    raise ValueError(f"global_device_count must be greater than or equal to local_device_count, but got {c} vs {l}")
  if s <= 0:
    raise ValueError(f"num_sc_per_device must be greater than 0, but got {s}")
  raise ValueError(f"Total number of SparseCores ({s * c}) must be a power of 2.")


def written_region_equal(rp_a, rp_b, arrays_a, arrays_b, num_sc_slices: int):
  """Bit-exact comparison of two preprocessing results over the region the reference writes:
  all row pointers, and per SparseCore slice the slots before its last row pointer."""
  rp_a, rp_b = np.asarray(rp_a).reshape(-1), np.asarray(rp_b).reshape(-1)
  np.testing.assert_array_equal(rp_a, rp_b)
  per = len(rp_a) // num_sc_slices
  for a, b in zip(arrays_a, arrays_b):
    a, b = np.asarray(a).reshape(-1), np.asarray(b).reshape(-1)
    assert a.shape == b.shape
    coo = len(a) // num_sc_slices
    for s in range(num_sc_slices):
      last = rp_a[s * per + per - 1]
      x, y = a[s * coo:s * coo + last], b[s * coo:s * coo + last]
      if x.dtype.kind == "f":
        np.testing.assert_array_equal(x.view(np.uint32), y.view(np.uint32))
      else:
        np.testing.assert_array_equal(x, y)
