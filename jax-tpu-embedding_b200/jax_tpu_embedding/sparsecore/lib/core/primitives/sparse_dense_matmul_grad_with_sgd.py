"""Backward operator fused with SGD: theta <- theta - lr * g on every touched row.

Mirrors `tpu_sparse_dense_matmul_grad_with_sgd_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_grad_with_sgd.py:32-238).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
          num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, learning_rate, *_,
          max_ids_per_partition: int, max_unique_ids_per_partition: int,
          computation_name: str = "sgd_optimizer_update", sharding_strategy: int = 1,
          enable_minibatching: bool = False, min_value: float | None = None, max_value: float | None = None,
          num_sc_per_device: int | None = None, global_device_count: int | None = None,
          local_device_count: int | None = None):
  utils.ensure_dtype(learning_rate, np.float32, "learning_rate")
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, max_ids_per_partition,
      max_unique_ids_per_partition, computation_name, sharding_strategy, min_value, max_value)
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  return _ops.GradRequest(
      "sgd", lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table, (),
      activations_grad, (_ops.scalar_f32(learning_rate),), min_value=min_value, max_value=max_value,
      num_sc_per_device=num_sc_per_device, global_device_count=global_device_count,
      local_device_count=local_device_count, partition_capacity=max_ids_per_partition,
      exchange_key=computation_name)


tpu_sparse_dense_matmul_grad_with_sgd_primitive = _ops.Primitive(
    "sparse_dense_matmul_grad_with_sgd", _prepare, _ops.run_grad_group, unwrap=lambda r: r[0])
