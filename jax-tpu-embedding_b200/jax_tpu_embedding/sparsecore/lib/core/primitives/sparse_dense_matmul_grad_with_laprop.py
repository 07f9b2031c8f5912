"""Backward operator fused with LaProp.

nu <- decay nu + (1 - decay)(g^2 + eps); u = b1 mu + sqrt(1 - b1^2) g / sqrt(nu); mu <- u;
theta <- theta - lr u, on touched rows only.
Mirrors `tpu_sparse_dense_matmul_grad_with_laprop_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_grad_with_laprop.py:60-405).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
             num_minibatches_per_physical_sparse_core, embedding_table, mu, nu, activations_grad,
             learning_rate, b1, decay_rate, eps, *_, max_ids_per_partition: int, max_unique_ids_per_partition: int,
             computation_name: str = "laprop_optimizer_update", sharding_strategy: int = 1,
             enable_minibatching: bool = False, min_value: float | None = None, max_value: float | None = None,
             num_sc_per_device: int | None = None, global_device_count: int | None = None,
             local_device_count: int | None = None):
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, max_ids_per_partition,
      max_unique_ids_per_partition, computation_name, sharding_strategy, min_value, max_value)
  for value, label in ((mu, "mu"), (nu, "nu"), (learning_rate, "learning_rate"), (b1, "b1"), (decay_rate, "decay_rate"), (eps, "eps")):
    utils.ensure_dtype(value, np.float32, label)
  if tuple(embedding_table.shape) != tuple(mu.shape) or tuple(embedding_table.shape) != tuple(nu.shape):
    raise ValueError(
        "embedding_table, mu and nu must have equal shapes, got"
        f" {tuple(embedding_table.shape)}, {tuple(mu.shape)} and {tuple(nu.shape)}")
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  hyper = tuple(_ops.scalar_f32(h) for h in (learning_rate, b1, decay_rate, eps))
  return _ops.GradRequest(
      "laprop", lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table,
      (mu, nu), activations_grad, hyper, min_value=min_value, max_value=max_value,
      num_sc_per_device=num_sc_per_device, global_device_count=global_device_count,
      local_device_count=local_device_count, partition_capacity=max_ids_per_partition,
      exchange_key=computation_name)


tpu_sparse_dense_matmul_grad_with_laprop_primitive = _ops.Primitive(
    "sparse_dense_matmul_grad_with_laprop_primitive", _prepare, _ops.run_grad_group, multiple_results=True)
