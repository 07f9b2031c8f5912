"""Backward operator fused with FTRL.

a' = a + g^2; dp = a'^(-lr_power) - a^(-lr_power); linear <- linear + g - (dp / lr) theta (or its
learning-rate-scaled form); theta <- (clamp(linear, -l1, l1) - linear) / ((a'^(-lr_power) + beta) / lr + 2 l2).
Mirrors `tpu_sparse_dense_matmul_grad_with_ftrl_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_grad_with_ftrl.py:60-406).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
             num_minibatches_per_physical_sparse_core, embedding_table, accumulator, linear, activations_grad,
             learning_rate, learning_rate_power, l1_regularization_strength, l2_regularization_strength, beta, *_, max_ids_per_partition: int, max_unique_ids_per_partition: int,
             computation_name: str = "ftrl_optimizer_update", sharding_strategy: int = 1,
             enable_minibatching: bool = False, min_value: float | None = None, max_value: float | None = None,
             multiply_linear_by_learning_rate: bool = False, num_sc_per_device: int | None = None, global_device_count: int | None = None,
             local_device_count: int | None = None):
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, max_ids_per_partition,
      max_unique_ids_per_partition, computation_name, sharding_strategy, min_value, max_value)
  for value, label in ((accumulator, "accumulator"), (linear, "linear"), (learning_rate, "learning_rate"), (learning_rate_power, "learning_rate_power"), (l1_regularization_strength, "l1_regularization_strength"), (l2_regularization_strength, "l2_regularization_strength"), (beta, "beta")):
    utils.ensure_dtype(value, np.float32, label)
  if tuple(embedding_table.shape) != tuple(accumulator.shape) or tuple(embedding_table.shape) != tuple(linear.shape):
    raise ValueError(
        "embedding_table, accumulator and linear must have equal shapes, got"
        f" {tuple(embedding_table.shape)}, {tuple(accumulator.shape)} and {tuple(linear.shape)}")
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  hyper = tuple(_ops.scalar_f32(h) for h in (learning_rate, learning_rate_power, l1_regularization_strength,
                                              l2_regularization_strength, beta)) + (
      1.0 if multiply_linear_by_learning_rate else 0.0,)
  return _ops.GradRequest(
      "ftrl", lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table,
      (accumulator, linear), activations_grad, hyper, min_value=min_value, max_value=max_value,
      num_sc_per_device=num_sc_per_device, global_device_count=global_device_count,
      local_device_count=local_device_count, partition_capacity=max_ids_per_partition,
      exchange_key=computation_name)


tpu_sparse_dense_matmul_grad_with_ftrl_primitive = _ops.Primitive(
    "sparse_dense_matmul_grad_with_ftrl_primitive", _prepare, _ops.run_grad_group, multiple_results=True)
