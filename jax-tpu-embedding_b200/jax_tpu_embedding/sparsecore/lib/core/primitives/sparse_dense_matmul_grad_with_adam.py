"""Backward operator fused with (lazy) Adam.

m <- m + (1 - beta_1)(g - m); v <- v + (1 - beta_2)(g^2 - v);
theta <- theta - alpha_t * m / (sqrt(v) + epsilon_hat), on touched rows only.  Mirrors
`tpu_sparse_dense_matmul_grad_with_adam_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_grad_with_adam.py:42-405).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
          num_minibatches_per_physical_sparse_core, embedding_table, momentum, velocity, activations_grad, alpha_t,
          beta_1, beta_2, epsilon_hat, *_, max_ids_per_partition: int, max_unique_ids_per_partition: int,
          computation_name: str = "adam_optimizer_update", sharding_strategy: int = 1,
          enable_minibatching: bool = False, min_value: float | None = None, max_value: float | None = None,
          num_sc_per_device: int | None = None, global_device_count: int | None = None,
          local_device_count: int | None = None):
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, max_ids_per_partition,
      max_unique_ids_per_partition, computation_name, sharding_strategy, min_value, max_value)
  utils.ensure_dtype(alpha_t, np.float32, "alpha_t")
  utils.ensure_dtype(beta_1, np.float32, "beta_1")
  utils.ensure_dtype(beta_2, np.float32, "beta_2")
  utils.ensure_dtype(epsilon_hat, np.float32, "epsilon_hat")
  utils.ensure_dtype(momentum, np.float32, "momentum")
  utils.ensure_dtype(velocity, np.float32, "velocity")
  if tuple(embedding_table.shape) != tuple(velocity.shape):
    raise ValueError(
        "embedding_table and velocity must have equal shapes, got"
        f" {tuple(embedding_table.shape)} and {tuple(velocity.shape)}")
  if tuple(embedding_table.shape) != tuple(momentum.shape):
    raise ValueError(
        "embedding_table and momentum must have equal shapes, got"
        f" {tuple(embedding_table.shape)} and {tuple(momentum.shape)}")
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  hyper = tuple(_ops.scalar_f32(h) for h in (alpha_t, beta_1, beta_2, epsilon_hat))
  return _ops.GradRequest(
      "adam", lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table,
      (momentum, velocity), activations_grad, hyper, min_value=min_value, max_value=max_value,
      num_sc_per_device=num_sc_per_device, global_device_count=global_device_count,
      local_device_count=local_device_count, partition_capacity=max_ids_per_partition,
      exchange_key=computation_name)


tpu_sparse_dense_matmul_grad_with_adam_primitive = _ops.Primitive(
    "sparse_dense_matmul_grad_with_adam_primitive", _prepare, _ops.run_grad_group, multiple_results=True)
