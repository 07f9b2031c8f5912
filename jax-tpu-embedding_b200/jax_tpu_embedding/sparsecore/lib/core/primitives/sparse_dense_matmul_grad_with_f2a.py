"""Backward operator fused with frequency-aware Adagrad (F2A).

local_step <- local_step + 1; f = min((max(global_step, 1) / local_step)^rho, max_lr_multiplier);
a <- a + g^2; theta <- theta - lr (f g / sqrt(a) + l1 sign(theta) + l2 theta), on touched rows only.
Mirrors `tpu_sparse_dense_matmul_grad_with_f2a_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_grad_with_f2a.py:60-358).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
             num_minibatches_per_physical_sparse_core, embedding_table, accumulator, local_step, activations_grad,
             learning_rate, rho, l1_regularization_strength, l2_regularization_strength, max_lr_multiplier,
             global_step, *_, max_ids_per_partition: int, max_unique_ids_per_partition: int,
             computation_name: str = "f2a_optimizer_update", sharding_strategy: int = 1,
             enable_minibatching: bool = False, min_value: float | None = None, max_value: float | None = None,
             num_sc_per_device: int | None = None, global_device_count: int | None = None,
             local_device_count: int | None = None):
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, max_ids_per_partition,
      max_unique_ids_per_partition, computation_name, sharding_strategy, min_value, max_value)
  for value, label in ((accumulator, "accumulator"), (local_step, "local_step"), (learning_rate, "learning_rate"), (rho, "rho"), (l1_regularization_strength, "l1_regularization_strength"), (l2_regularization_strength, "l2_regularization_strength"), (max_lr_multiplier, "max_lr_multiplier"), (global_step, "global_step")):
    utils.ensure_dtype(value, np.float32, label)
  if tuple(embedding_table.shape) != tuple(accumulator.shape) or tuple(embedding_table.shape) != tuple(local_step.shape):
    raise ValueError(
        "embedding_table, accumulator and local_step must have equal shapes, got"
        f" {tuple(embedding_table.shape)}, {tuple(accumulator.shape)} and {tuple(local_step.shape)}")
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  hyper = tuple(_ops.scalar_f32(h) for h in (learning_rate, rho, l1_regularization_strength,
                                              l2_regularization_strength, max_lr_multiplier, global_step))
  return _ops.GradRequest(
      "f2a", lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table,
      (accumulator, local_step), activations_grad, hyper, min_value=min_value, max_value=max_value,
      num_sc_per_device=num_sc_per_device, global_device_count=global_device_count,
      local_device_count=local_device_count, partition_capacity=max_ids_per_partition,
      exchange_key=computation_name)


tpu_sparse_dense_matmul_grad_with_f2a_primitive = _ops.Primitive(
    "sparse_dense_matmul_grad_with_f2a_primitive", _prepare, _ops.run_grad_group, multiple_results=True)
