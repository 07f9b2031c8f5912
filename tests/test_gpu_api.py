"""End-to-end through the public API (preprocess -> lookup -> update) vs first principles.

The expected values come from `dense_reference`: per sample, the combiner-weighted sum of table
rows in float64, i.e. the definition of the operation, independent of any CSR layout.
"""

import numpy as np
import pytest

import cases
from oracle import lookup_oracle as lo
from jax_tpu_embedding.sparsecore.lib.nn import embedding
from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec
from jax_tpu_embedding.sparsecore.lib.nn import initializers
from jax_tpu_embedding.sparsecore.lib.nn import table_stacking

pytestmark = pytest.mark.gpu

CASES = [c for c in cases.standard_cases()
         if c.local_device_count == c.global_device_count and not c.allow_id_dropping]


def _tables(case, seed=1):
  rng = np.random.default_rng(seed)
  specs = {f.table_spec.name: f.table_spec for f in case.feature_specs}
  return specs, {n: rng.normal(0, 0.01, size=(t.vocabulary_size, t.embedding_dim)).astype(np.float32)
                 for n, t in specs.items()}


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_lookup_and_update_match_definition(case):
  import torch

  c, s = case.global_device_count, case.num_sc_per_device
  p = c * s
  tspecs, tables = _tables(case)
  names = sorted(tspecs)
  stacked = table_stacking.stack_and_shard_tables([tspecs[n] for n in names], [tables[n] for n in names], p,
                                                 pad_value=0.0)
  stacks = embedding.get_stacked_table_specs(case.feature_specs)
  variables = {}
  for name, spec in stacks.items():
    tab = torch.from_numpy(stacked[name].reshape(-1, spec.stack_embedding_dim)).cuda()
    slots = tuple(torch.full_like(tab, 0.1) if i == 0 and spec.optimizer.short_name() == "adagrad"
                  else torch.zeros_like(tab) for i in range(spec.optimizer.slot_variables_count()))
    variables[name] = embedding.EmbeddingVariables(tab, slots)

  pre, _ = embedding.preprocess_sparse_dense_matmul_input(
      case.features, case.weights, case.feature_specs, case.local_device_count, c, num_sc_per_device=s)
  acts = embedding.tpu_sparse_dense_matmul(pre, variables, case.feature_specs, global_device_count=c,
                                           num_sc_per_device=s)
  rng = np.random.default_rng(9)
  grads = []
  want_grad = {n: np.zeros_like(tables[n], dtype=np.float64) for n in names}
  for i, (feat, act) in enumerate(zip(case.feature_specs, acts)):
    tname = feat.table_spec.name
    w = None if case.weights is None else case.weights[i]
    combiner = feat.table_spec.combiner
    g = (rng.normal(0, 1, size=tuple(act.shape)) * 1e-2).astype(np.float32)
    want, tg = lo.dense_reference(case.features[i], w, combiner, tables[tname], g)
    np.testing.assert_allclose(act.cpu().numpy(), want, rtol=2e-5, atol=1e-7)
    want_grad[tname] += tg
    grads.append(torch.from_numpy(g).cuda())

  updated = embedding.tpu_sparse_dense_matmul_grad(grads, pre, variables, case.feature_specs,
                                                   global_device_count=c, num_sc_per_device=s, step=0)
  new_tables = table_stacking.unshard_and_unstack_tables(
      {n: tspecs[n] for n in names}, {k: v.table.cpu().numpy() for k, v in updated.items()}, p)
  for n in names:
    opt = tspecs[n].optimizer
    g = want_grad[n]
    old = tables[n].astype(np.float64)
    touched = np.zeros(len(old), bool)
    for i, feat in enumerate(case.feature_specs):
      if feat.table_spec.name == n:
        for row in case.features[i]:
          touched[np.asarray(row).reshape(-1)] = True
    if opt.short_name() == "sgd":
      want = old - 0.01 * g
    elif opt.short_name() == "adagrad":
      want = old - 0.01 * g / np.sqrt(0.1 + g * g)
    else:
      a, b1, b2, eh = (float(x) for x in opt.get_hyperparameters(0))
      m, v = (1 - b1) * g, (1 - b2) * g * g
      want = old - a * m / (np.sqrt(v) + eh)
    want = np.where(touched[:, None], want, old)
    np.testing.assert_allclose(new_tables[n], want, rtol=2e-5, atol=1e-7)


def test_stats_example_from_docstring():
  """Worked example of the reference's SparseDenseMatmulInputStats docstring (embedding.py:105-130)."""
  t = embedding_spec.TableSpec(name="t", vocabulary_size=16, embedding_dim=8, initializer=None,
                               optimizer=embedding_spec.SGDOptimizerSpec(), combiner="sum",
                               max_ids_per_partition=64, max_unique_ids_per_partition=64)
  f = embedding_spec.FeatureSpec(name="f", table_spec=t, input_shape=[2], output_shape=[2, 8])
  embedding.prepare_feature_specs_for_training([f], 1, 2)
  rows = np.empty(2, dtype=object)
  rows[0] = np.array([0, 0, 0, 2, 4, 1], np.int32)
  rows[1] = np.array([1, 1, 1, 3, 3, 5, 5, 7, 7, 0], np.int32)
  w = np.empty(2, dtype=object)
  w[0] = np.arange(1, 7, dtype=np.float32)  # distinct weights would not be merged... same (row, id) are
  w[1] = np.ones(10, np.float32)
  _, stats = embedding.preprocess_sparse_dense_matmul_input([rows], None, [f], 1, 1, num_sc_per_device=2)
  # ids are deduplicated per sample, so counts are of distinct (sample, id) pairs.
  assert stats.max_ids_per_partition["t"].tolist() == [3, 4]
  assert stats.max_unique_ids_per_partition["t"].tolist() == [3, 4]


def test_update_preprocessing_parameters_roundtrip():
  case = cases.make_case("fdo", seed=2, tables=[dict(vocab=1000, dim=16)], batch=256, num_sc_per_device=2)
  _, stats = embedding.preprocess_sparse_dense_matmul_input(case.features, None, case.feature_specs, 1, 1,
                                                            num_sc_per_device=2)
  embedding.update_preprocessing_parameters(case.feature_specs, stats, 2)
  spec = case.feature_specs[0].table_spec.stacked_table_spec
  assert spec.max_ids_per_partition == int(stats.max_ids_per_partition["table_0"].max())
  assert spec.suggested_coo_buffer_size_per_device == int(stats.required_buffer_size_per_sc["table_0"].max()) * 2
  pre, stats2 = embedding.preprocess_sparse_dense_matmul_input(case.features, None, case.feature_specs, 1, 1,
                                                               num_sc_per_device=2)
  assert stats2.id_drop_counters["table_0"] == 0
  assert pre.lhs_embedding_ids["table_0"].shape[0] == spec.suggested_coo_buffer_size_per_device


@pytest.mark.parametrize("kind", ["adagrad_momentum", "ftrl", "laprop", "f2a"])
def test_two_slot_optimizers_through_the_api(kind):
  """Variables created by init_embedding_variables, one update through the public API, checked
  against the float64 definition of each optimizer (fresh slots: accumulator 0.1 or 0, others 0)."""
  import torch

  opt = {"adagrad_momentum": embedding_spec.AdagradMomentumOptimizerSpec(learning_rate=0.05, momentum=0.9, use_nesterov=True),
         "ftrl": embedding_spec.FTRLOptimizerSpec(learning_rate=0.05, l1_regularization_strength=0.001,
                                                  l2_regularization_strength=0.01, beta=0.1,
                                                  multiply_linear_by_learning_rate=True),
         "laprop": embedding_spec.LaPropOptimizerSpec(learning_rate=0.01, b1=0.9, b2=0.95, eps=1e-12),
         "f2a": embedding_spec.F2AOptimizerSpec(learning_rate=0.05, rho=0.5, l2_regularization_strength=0.01)}[kind]
  table = embedding_spec.TableSpec(name="t", vocabulary_size=500, embedding_dim=16,
                                   initializer=initializers.normal(0.05), optimizer=opt, combiner="sum",
                                   max_ids_per_partition=4096, max_unique_ids_per_partition=4096)
  feature = embedding_spec.FeatureSpec(name="f", table_spec=table, input_shape=[128, 3], output_shape=[128, 16])
  embedding.prepare_feature_specs_for_training([feature], 1, 2)
  variables = embedding.init_embedding_variables(7, [table], 1, num_sparsecore_per_device=2)
  name = table.stacked_table_spec.stack_name
  assert type(variables[name].slot)._fields == type(opt.slot_variables_initializers())._fields
  rng = np.random.default_rng(3)
  ids = rng.integers(0, 500, size=(128, 3)).astype(np.int32)
  grad = (rng.normal(size=(128, 16)) * 1e-2).astype(np.float32)
  before = table_stacking.unshard_and_unstack_tables({"t": table}, {name: variables[name].table.cpu().numpy()}, 2)["t"]
  pre, _ = embedding.preprocess_sparse_dense_matmul_input([ids], None, [feature], 1, 1, num_sc_per_device=2)
  updated = embedding.tpu_sparse_dense_matmul_grad([torch.from_numpy(grad).cuda()], pre, variables, [feature],
                                                   global_device_count=1, num_sc_per_device=2, step=4)
  after = table_stacking.unshard_and_unstack_tables({"t": table}, {name: updated[name].table.cpu().numpy()}, 2)["t"]
  g = np.zeros((500, 16))
  for s in range(128):
    for j in range(3):
      g[ids[s, j]] += grad[s]
  touched = np.zeros(500, bool)
  touched[ids.reshape(-1)] = True
  w = before.astype(np.float64)
  if kind == "adagrad_momentum":
    s = g / np.sqrt(0.1 + g * g + 1e-10)
    want = w - 0.05 * (0.9 * s + s)
  elif kind == "ftrl":
    a1 = 0.1 + g * g
    dp = np.sqrt(a1) - np.sqrt(0.1)
    lin = 0.05 * g - dp * w
    want = (np.clip(lin, -0.001 * 0.05, 0.001 * 0.05) - lin) / (np.sqrt(a1) + 2 * 0.05 * 0.01 + 0.1)
  elif kind == "laprop":
    decay = float(opt.get_decay_rate(4))
    nu = (1 - decay) * (g * g + 1e-12)
    want = w - 0.01 * np.sqrt(1 - 0.81) * g / np.sqrt(nu)
  else:
    fa = min((4.0 / 1.0) ** 0.5, 1e6)
    want = w - 0.05 * (g * fa / np.sqrt(0.1 + g * g) + 0.01 * w)
  want = np.where(touched[:, None], want, w)
  np.testing.assert_allclose(after, want, rtol=3e-5, atol=1e-7)
