"""The three sources of the forward's sample-major plan give bit-identical activations.

  given   emitted by this package's preprocessing together with the CSR buffers,
  single  one scatter, when every feature of the stack is declared single-valent,
  built   counting sort inside the operator (foreign buffers).

All are compared with the numpy oracle of the lookup (same summation order: ascending slot),
bit for bit, on the buffers the GPU preprocessing produced (themselves bit-exact with the oracle).
"""

import numpy as np
import pytest

import cases
from oracle import lookup_oracle as lo
from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_csr
from jax_tpu_embedding.sparsecore.lib.nn import embedding

pytestmark = pytest.mark.gpu


def _plan_cases():
  out = [c for c in cases.standard_cases() if c.local_device_count == 1 and c.global_device_count == 1]
  out.append(cases.make_case("long_bags_2sc", seed=5, batch=64, num_sc_per_device=2, combiner="sum", tables=[
      dict(vocab=5000, dim=32, features=[dict(kind="ragged", min_len=0, max_len=600)])]))
  out.append(cases.make_case("stacked_single_hot", seed=6, batch=512, num_sc_per_device=2, stack=True, tables=[
      dict(vocab=300, dim=16, features=[dict(kind="dense", valency=1, dist="zipf"), dict(kind="dense", valency=1)]),
      dict(vocab=77, dim=16, features=[dict(kind="dense", valency=1)])]))
  out.append(cases.make_case("dropping_single_hot", seed=7, batch=1024, max_ids=100, max_unique=20,
                             allow_id_dropping=True, tables=[
      dict(vocab=64, dim=8, features=[dict(kind="dense", valency=1)])]))
  return out


CASES = _plan_cases()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_plan_sources_agree_with_the_oracle(case):
  import torch

  s = case.num_sc_per_device
  specs = case.feature_specs
  pre, _ = embedding.preprocess_sparse_dense_matmul_input(case.features, case.weights, specs, 1, 1, num_sc_per_device=s,
                                                          allow_id_dropping=case.allow_id_dropping)
  rps = pre.lhs_row_pointers
  assert rps.forward_plans is not None and set(rps.forward_plans) == set(rps)
  rng = np.random.default_rng(1)
  stacked = embedding.get_stacked_table_specs(specs)
  variables, shards = {}, {}
  for name, spec in stacked.items():
    rows = spec.stack_vocab_size // s
    shards[name] = rng.normal(0, 0.01, size=(s, rows, spec.stack_embedding_dim)).astype(np.float32)
    variables[name] = embedding.EmbeddingVariables(
        torch.from_numpy(shards[name].reshape(-1, spec.stack_embedding_dim)).cuda(), ())
  given = embedding.tpu_sparse_dense_matmul(pre, variables, specs, global_device_count=1, num_sc_per_device=s,
                                            perform_unstacking=False)
  for name, spec in stacked.items():
    bdev = spec.total_sample_count
    csr = [tuple(d[name].cpu().numpy() for d in pre.sparse_dense_matmul_input)]
    want = lo.forward(csr, shards[name], num_sc_per_device=s, device_batch_size=bdev)[0]
    np.testing.assert_array_equal(given[name].cpu().numpy(), want)
    # The bags cover exactly the entries of the buffers.
    bags = rps.forward_plans[name][1].cpu().numpy().reshape(-1, 2).astype(np.int64)
    written = int(np.sum(csr[0][2] != 2**31 - 1))  # every slot without an entry holds the padding value
    assert int((bags[:, 1] - bags[:, 0]).sum()) == written
    operands = [d[name] for d in pre.sparse_dense_matmul_input]
    kw = dict(device_batch_size=bdev, max_ids_per_partition=spec.max_ids_per_partition,
              max_unique_ids_per_partition=spec.max_unique_ids_per_partition, num_sc_per_device=s,
              global_device_count=1, local_device_count=1)
    bind = sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.bind
    built = bind(*operands, np.int32(1), variables[name].table, **kw)
    np.testing.assert_array_equal(built.cpu().numpy(), want)
    members = [f for f in specs if f.table_spec.stacked_table_spec.stack_name == name]
    if all(len(f.input_shape) == 2 and f.input_shape[-1] == 1 for f in members):
      single = bind(*operands, np.int32(1), variables[name].table, max_ids_per_sample=1, **kw)
      np.testing.assert_array_equal(single.cpu().numpy(), want)


def test_foreign_row_pointer_dict_drops_the_plan():
  """Replacing an array of the output invalidates the plan: the operator then builds its own."""
  case = CASES[0]
  pre, _ = embedding.preprocess_sparse_dense_matmul_input(case.features, None, case.feature_specs, 1, 1,
                                                          num_sc_per_device=1)
  rps = pre.lhs_row_pointers
  name = next(iter(rps))
  assert embedding._forward_plans(*pre.sparse_dense_matmul_input) is not None  # pylint: disable=protected-access
  pre.lhs_gains[name] = pre.lhs_gains[name].clone()
  assert embedding._forward_plans(*pre.sparse_dense_matmul_input) is None  # pylint: disable=protected-access
