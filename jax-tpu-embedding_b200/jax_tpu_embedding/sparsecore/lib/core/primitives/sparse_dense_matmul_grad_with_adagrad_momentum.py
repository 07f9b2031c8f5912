"""Backward operator fused with Adagrad with momentum.

a <- a + g^2 (beta2 == 1) or beta2 a + (1 - beta2) g^2; s = (a + epsilon)^(-1/exponent) g;
m <- momentum m + s; theta <- theta - lr (momentum m + s if use_nesterov else m), on touched rows only.
Mirrors `tpu_sparse_dense_matmul_grad_with_adagrad_momentum_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_grad_with_adagrad_momentum.py:76-382).
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
             num_minibatches_per_physical_sparse_core, embedding_table, accumulator, momentum, activations_grad,
             learning_rate, momentum_param, beta2, epsilon, exponent, use_nesterov=np.bool_(False), *_, max_ids_per_partition: int, max_unique_ids_per_partition: int,
             computation_name: str = "adagrad_momentum_optimizer_update", sharding_strategy: int = 1,
             enable_minibatching: bool = False, min_value: float | None = None, max_value: float | None = None,
             num_sc_per_device: int | None = None, global_device_count: int | None = None,
             local_device_count: int | None = None):
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table, activations_grad, max_ids_per_partition,
      max_unique_ids_per_partition, computation_name, sharding_strategy, min_value, max_value)
  for value, label in ((accumulator, "accumulator"), (momentum, "momentum"), (learning_rate, "learning_rate"), (momentum_param, "momentum_param"), (beta2, "beta2"), (epsilon, "epsilon"), (exponent, "exponent")):
    utils.ensure_dtype(value, np.float32, label)
  utils.ensure_dtype(use_nesterov, np.bool_, "use_nesterov")
  if tuple(embedding_table.shape) != tuple(accumulator.shape) or tuple(embedding_table.shape) != tuple(momentum.shape):
    raise ValueError(
        "embedding_table, accumulator and momentum must have equal shapes, got"
        f" {tuple(embedding_table.shape)}, {tuple(accumulator.shape)} and {tuple(momentum.shape)}")
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  hyper = tuple(_ops.scalar_f32(h) for h in (learning_rate, momentum_param, beta2, epsilon, exponent)) + (
      1.0 if bool(np.asarray(use_nesterov)) else 0.0,)
  return _ops.GradRequest(
      "adagrad_momentum", lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table,
      (accumulator, momentum), activations_grad, hyper, min_value=min_value, max_value=max_value,
      num_sc_per_device=num_sc_per_device, global_device_count=global_device_count,
      local_device_count=local_device_count, partition_capacity=max_ids_per_partition,
      exchange_key=computation_name)


tpu_sparse_dense_matmul_grad_with_adagrad_momentum_primitive = _ops.Primitive(
    "sparse_dense_matmul_grad_with_adagrad_momentum_primitive", _prepare, _ops.run_grad_group, multiple_results=True)
