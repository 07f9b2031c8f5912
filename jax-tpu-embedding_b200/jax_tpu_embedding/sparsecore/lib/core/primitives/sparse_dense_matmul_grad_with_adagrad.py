"""Backward operator fused with Adagrad: a <- a + g^2; theta <- theta - lr * g / sqrt(a).

Mirrors `tpu_sparse_dense_matmul_grad_with_adagrad_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_grad_with_adagrad.py:41-292).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
          num_minibatches_per_physical_sparse_core, embedding_table, accumulator, activations_grad, learning_rate,
          *_, max_ids_per_partition: int, max_unique_ids_per_partition: int,
          computation_name: str = "adagrad_optimizer_update", sharding_strategy: int = 1,
          enable_minibatching: bool = False, min_value: float | None = None, max_value: float | None = None,
          num_sc_per_device: int | None = None, global_device_count: int | None = None,
          local_device_count: int | None = None):
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, max_ids_per_partition,
      max_unique_ids_per_partition, computation_name, sharding_strategy, min_value, max_value)
  utils.ensure_dtype(accumulator, np.float32, "accumulator")
  utils.ensure_dtype(learning_rate, np.float32, "learning_rate")
  if tuple(embedding_table.shape) != tuple(accumulator.shape):
    raise ValueError(
        "embedding_table and accumulator must have equal shapes, got"
        f" {tuple(embedding_table.shape)} and {tuple(accumulator.shape)}")
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  return _ops.GradRequest(
      "adagrad", lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table,
      (accumulator,), activations_grad, (_ops.scalar_f32(learning_rate),), min_value=min_value, max_value=max_value,
      num_sc_per_device=num_sc_per_device, global_device_count=global_device_count,
      local_device_count=local_device_count, partition_capacity=max_ids_per_partition,
      exchange_key=computation_name)


tpu_sparse_dense_matmul_grad_with_adagrad_primitive = _ops.Primitive(
    "sparse_dense_matmul_grad_with_adagrad_primitive", _prepare, _ops.run_grad_group, multiple_results=True)
