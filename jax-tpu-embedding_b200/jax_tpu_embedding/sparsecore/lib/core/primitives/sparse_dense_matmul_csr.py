"""Forward operator `sparse_dense_matmul_csr`.

Mirrors `tpu_sparse_dense_matmul_csr_primitive` of the reference
(jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_csr.py:33-207):
same operand order, attributes and validation; the libtpu custom call
"SparseDenseMatmulOp" is replaced by `sc_sparse_dense_matmul_fwd`.
"""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import utils


def _prepare(lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
          num_minibatches_per_physical_sparse_core, embedding_table, *, device_batch_size: int,
          max_ids_per_partition: int, max_unique_ids_per_partition: int, sharding_strategy: int = 1,
          quantization_config: tuple[float, float, int] | None = None, enable_minibatching: bool = False,
          num_sc_per_device: int | None = None, global_device_count: int | None = None,
          local_device_count: int | None = None, max_ids_per_sample: int = 0, forward_plan=None):
  embedding_dim = utils.get_embedding_dim(embedding_table)
  utils.validate_abstract_eval_params(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains,
      num_minibatches_per_physical_sparse_core, embedding_table,
      utils._Shaped((device_batch_size, embedding_dim), np.float32),  # pylint: disable=protected-access
      max_ids_per_partition, max_unique_ids_per_partition, "fwd-pass", sharding_strategy)
  if quantization_config is not None:
    q_min, q_max, q_buckets = quantization_config
    if q_buckets < 2:
      raise ValueError(f"quantization_num_buckets must be at least 2, got {q_buckets}")
    if q_min >= q_max:
      raise ValueError(f"quantization_min_valuemust be less than quantization_max_value, got {q_min} and {q_max}")
    # Activation quantization is a TPU-side numeric option; values are returned unquantized.
  if enable_minibatching:
    raise NotImplementedError("minibatching exists to fit TPU on-chip memory and is not part of the B200 path")
  return _ops.ForwardRequest(
      lhs_row_pointers, lhs_local_embedding_ids, lhs_local_sample_ids, lhs_gains, embedding_table,
      device_batch_size=device_batch_size, num_sc_per_device=num_sc_per_device,
      global_device_count=global_device_count, local_device_count=local_device_count,
      max_ids_per_sample=max_ids_per_sample, forward_plan=forward_plan)


tpu_sparse_dense_matmul_csr_primitive = _ops.Primitive("sparse_dense_matmul_csr", _prepare, _ops.run_forward_group)
