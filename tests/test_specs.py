"""Spec layer: stacking arithmetic, optimizer hyper-parameters, sharding helpers, pytrees.

Expected numbers restate the reference's own examples: padding rules and stacking offsets of
lib/nn/table_stacking.py (:355-378, :570-613, :731-740), the Adam bias correction of
lib/nn/embedding_spec.py:506-539 and the MOD layout of utils/utils.py:90-136.
"""

import dataclasses

import numpy as np
import pytest

from jax_tpu_embedding.sparsecore import _tree
from jax_tpu_embedding.sparsecore.lib.nn import embedding
from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec as es
from jax_tpu_embedding.sparsecore.lib.nn import table_stacking as ts
from jax_tpu_embedding.sparsecore.utils import utils


def _table(name, vocab, dim, opt=None, combiner="sum", **kw):
  return es.TableSpec(name=name, vocabulary_size=vocab, embedding_dim=dim, initializer=None,
                      optimizer=opt or es.SGDOptimizerSpec(), combiner=combiner, **kw)


def _feature(name, table, batch):
  return es.FeatureSpec(name=name, table_spec=table, input_shape=[batch, 1], output_shape=[batch, table.embedding_dim])


def test_prepare_pads_and_stacks_features_of_one_table():
  t = _table("t", 1001, 12)
  feats = [_feature("b", t, 16), _feature("a", t, 32)]
  embedding.prepare_feature_specs_for_training(feats, global_device_count=2, num_sc_per_device=4)
  st = t.stacked_table_spec
  assert st.stack_vocab_size == 1024 and st.stack_embedding_dim == 16 and st.total_sample_count == 48
  assert t.setting_in_stack.padded_vocab_size == 1024
  # features of one table are ordered by name
  assert feats[1].id_transformation.row_offset == 0 and feats[0].id_transformation.row_offset == 32
  with pytest.raises(AttributeError, match="update_preprocessing_parameters"):
    t.max_ids_per_partition = 7


def test_stack_tables_offsets_and_rotation():
  tables = [_table("a", 100, 8), _table("b", 30, 6), _table("c", 64, 8)]
  feats = [_feature(f"f{i}", t, 16) for i, t in enumerate(tables)]
  ts.stack_tables(feats, ["a", "b", "c"], global_device_count=2, num_sc_per_device=2, stack_name="s")
  shards = 4
  st = tables[0].stacked_table_spec
  assert st.stack_vocab_size == 128 + 32 + 64 and st.stack_embedding_dim == 8 and st.total_sample_count == 48
  assert [t.setting_in_stack.row_offset_in_shard for t in tables] == [0, 32, 40]
  assert [t.setting_in_stack.shard_rotation for t in tables] == [0, 2, 0]
  assert [f.id_transformation.col_offset for f in feats] == [0, 32 * shards, 40 * shards]
  assert [f.id_transformation.col_shift for f in feats] == [0, 2, 0]
  assert [f.id_transformation.row_offset for f in feats] == [0, 16, 32]
  assert st.max_ids_per_partition == 256  # default limits for multi-table stacks
  with pytest.raises(ValueError, match="already stacked"):
    ts.stack_tables(feats, ["a"], 2, 2, stack_name="again")


def test_stack_tables_rejects_mixed_settings():
  feats = [_feature("f0", _table("a", 16, 8), 8), _feature("f1", _table("b", 16, 8, combiner="mean"), 8)]
  with pytest.raises(ValueError, match="different combiners"):
    ts.stack_tables(feats, ["a", "b"], 1, 1)
  feats = [_feature("f0", _table("a", 16, 8), 8), _feature("f1", _table("b", 16, 8, opt=es.AdagradOptimizerSpec()), 8)]
  with pytest.raises(ValueError, match="different optimizers"):
    ts.stack_tables(feats, ["a", "b"], 1, 1)


def test_auto_stack_groups_by_dim_and_memory():
  tables = [_table("a", 100, 8), _table("b", 100, 7), _table("c", 100, 16), _table("d", 100, 8, combiner="mean")]
  feats = [_feature(f"f{i}", t, 64) for i, t in enumerate(tables)]
  embedding.auto_stack_tables(feats, global_device_count=1, num_sc_per_device=1)
  names = [t.stacked_table_spec.stack_name for t in tables]
  assert names[0] == names[1] == "a_b" and names[2] == "c" and names[3] == "d"
  # with a tiny activation budget nothing merges
  tables = [_table("a", 100, 8), _table("b", 100, 8)]
  feats = [_feature(f"f{i}", t, 64) for i, t in enumerate(tables)]
  embedding.auto_stack_tables(feats, 1, 1, activation_mem_bytes_limit=64 * 8 * 4)
  assert tables[0].stacked_table_spec.stack_name != tables[1].stacked_table_spec.stack_name


def test_short_stack_names():
  long = [f"table_with_a_long_name_{i}" for i in range(4)]
  name = ts._get_stack_name(long)  # pylint: disable=protected-access
  assert name.startswith("_".join(long)[:50] + "...") and len(name) == 50 + 3 + 12
  assert ts._get_stack_name(["a", "b"]) == "a_b"  # pylint: disable=protected-access


def test_stack_and_shard_round_trip():
  tables = [_table("a", 20, 8), _table("b", 9, 5)]
  feats = [_feature(f"f{i}", t, 8) for i, t in enumerate(tables)]
  ts.stack_tables(feats, ["a", "b"], global_device_count=2, num_sc_per_device=2, stack_name="s")
  rng = np.random.default_rng(0)
  values = [rng.normal(size=(t.vocabulary_size, t.embedding_dim)).astype(np.float32) for t in tables]
  stacked = ts.stack_and_shard_tables(tables, values, num_shards=4, pad_value=0.0)
  s = stacked["s"]
  assert s.shape == (4, 8 + 8, 8)
  # id i of table a lives on shard i % 4, local row i // 4
  np.testing.assert_array_equal(s[3, 1, :], values[0][7])
  # table b is rotated by 2 shards and offset by 8 rows
  np.testing.assert_array_equal(s[(1 + 2) % 4, 8 + 1, :5], values[1][5])
  phys = ts.compute_physical_row_ids(4, 64, 2, 8, np.array([5]))
  assert phys[0] == 3 * 16 + 8 + 1
  back = ts.unshard_and_unstack_tables(tables, stacked, 4)
  for v, b in zip(values, back):
    np.testing.assert_array_equal(v, b)


def test_shard_emb_table_layout():
  table = np.arange(16 * 2, dtype=np.float32).reshape(16, 2)
  sharded = utils.shard_emb_table(table, num_devices=2, num_sc_per_device=2)
  assert sharded.shape == (2, 8, 2)
  # device c, SparseCore s holds rows {v*4 + c*2 + s}
  np.testing.assert_array_equal(sharded[1, 4:8, 0] // 2, [3, 7, 11, 15])
  np.testing.assert_array_equal(utils.unshard_emb_table(sharded, 2), table)
  assert utils.NUM_SC_PER_DEVICE_MAP["NVIDIA B200"] == 1
  with pytest.raises(ValueError):
    utils.shard_emb_table(table, num_devices=2, num_sc_per_device=2, sharding_strategy="DIV")


def test_optimizer_hyperparameters():
  sgd = es.SGDOptimizerSpec(learning_rate=lambda step: 0.1 / (step + 1))
  assert sgd.get_hyperparameters(1)[0] == np.float32(0.05) and sgd.get_hyperparameters(1)[0].dtype == np.float32
  with pytest.raises(ValueError, match="requires a `step`"):
    sgd.get_hyperparameters(None)
  assert es.SGDOptimizerSpec(lambda: 0.3).get_learning_rate() == np.float32(0.3)
  adam = es.AdamOptimizerSpec(learning_rate=0.001, beta_1=0.9, beta_2=0.999, epsilon=1e-8)
  alpha, b1, b2, eps = adam.get_hyperparameters(9)
  c2 = np.sqrt(1 - 0.999**10)
  np.testing.assert_allclose(alpha, 0.001 * c2 / (1 - 0.9**10), rtol=1e-5)
  np.testing.assert_allclose(eps, 1e-8 * c2, rtol=1e-5)
  assert b1 == np.float32(0.9) and b2 == np.float32(0.999)
  assert adam.slot_variables_count() == 2 and es.AdagradOptimizerSpec().slot_variables_count() == 1
  assert es.SGDOptimizerSpec(0.1) == es.SGDOptimizerSpec(0.1) and es.SGDOptimizerSpec(0.1) != es.SGDOptimizerSpec(0.2)
  assert adam.short_name() == "adam" and es.AdagradOptimizerSpec().short_name() == "adagrad"


def test_two_slot_optimizer_specs():
  """AdagradMomentum, FTRL, LaProp, F2A: hyper-parameter order, slot names, operators, and the oracle's formulas
  on scalars worked out by hand."""
  from oracle import lookup_oracle as lo

  am = es.AdagradMomentumOptimizerSpec(learning_rate=0.1, momentum=0.5, use_nesterov=True)
  hp = am.get_hyperparameters()
  assert [float(h) for h in hp[:5]] == [np.float32(0.1), 0.5, 1.0, np.float32(1e-10), 2.0] and hp[5].dtype == np.bool_
  assert am.slot_variables_initializers()._fields == ("accumulator", "momentum") and am.short_name() == "adagrad_momentum"
  ftrl = es.FTRLOptimizerSpec(learning_rate=0.5, l1_regularization_strength=0.25, beta=1.0)
  assert [float(h) for h in ftrl.get_hyperparameters()] == [0.5, -0.5, 0.25, 0.0, 1.0]
  assert ftrl.slot_variables_initializers()._fields == ("accumulator", "linear")
  lap = es.LaPropOptimizerSpec(b2=0.5)
  np.testing.assert_allclose(lap.get_hyperparameters(2)[2], 0.5 * (1 - 0.25) / (1 - 0.125), rtol=1e-6)
  assert float(lap.get_hyperparameters()[2]) == 0.5 and lap.slot_variables_initializers()._fields == ("mu", "nu")
  with pytest.raises(ValueError, match="rms_clip_threshold"):
    es.LaPropOptimizerSpec(rms_clip_threshold=1.0)
  f2a = es.F2AOptimizerSpec()
  assert float(f2a.get_hyperparameters(7)[5]) == 7.0 and f2a.slot_variables_initializers()._fields == ("accumulator", "local_step")
  for spec in (am, ftrl, lap, f2a):
    assert spec.slot_variables_count() == 2
    assert spec.get_optimizer_primitive().name == f"sparse_dense_matmul_grad_with_{spec.short_name()}_primitive"
    assert spec == type(spec)(**{k: v for k, v in vars(spec).items()})

  one = lambda v: np.full((1, 1, 1), v, np.float32)
  hit = np.ones((1, 1), bool)
  # FTRL, lr 0.5, power -0.5, no regularisation: a' = 1 + 9 = 10... use a = 0, g = 2 -> a' = 4, sqrt = 2,
  # linear' = 0 + 2 - (2 - 0) / 0.5 * w = 2 - 4 w, w' = -linear' / (2 / 0.5) with w = 1 -> linear' = -2, w' = 0.5.
  w, a, l = lo.apply_ftrl(one(1.0), one(0.0), one(0.0), one(2.0), hit, 0.5, -0.5, 0.0, 0.0, 0.0)
  assert (w.item(), a.item(), l.item()) == (0.5, 4.0, -2.0)
  # LaProp, b1 0, decay 0, eps 0: nu' = g^2, update = g / |g| = 1 -> w' = w - lr.
  w, mu, nu = lo.apply_laprop(one(1.0), one(5.0), one(7.0), one(-3.0), hit, 0.25, 0.0, 0.0, 0.0)
  assert (w.item(), mu.item(), nu.item()) == (1.25, -1.0, 9.0)
  # Adagrad momentum, beta2 1, exponent 2, eps 0, a = 3, g = 1 -> a' = 4, s = 0.5; m' = 0.5 * 2 + 0.5 = 1.5;
  # nesterov: 0.5 * 1.5 + 0.5 = 1.25 -> w' = 1 - 0.1 * 1.25.
  w, a, m = lo.apply_adagrad_momentum(one(1.0), one(3.0), one(2.0), one(1.0), hit, 0.1, 0.5, 1.0, 0.0, 2.0, True)
  np.testing.assert_allclose([w.item(), a.item(), m.item()], [0.875, 4.0, 1.5], rtol=1e-6)
  # F2A, rho 1, global step 8, local step 3 -> multiplier 8 / 4 = 2; a = 0, g = 3 -> g f / sqrt(a') = 2;
  # l1 0.5 sign(w) + l2 0.25 w with w = 2 -> 1.0; w' = 2 - 0.1 * 3.
  w, a, s = lo.apply_f2a(one(2.0), one(0.0), one(3.0), one(3.0), hit, 0.1, 1.0, 0.5, 0.25, 1e6, 8.0)
  np.testing.assert_allclose([w.item(), a.item(), s.item()], [1.7, 9.0, 4.0], rtol=1e-6)
  # Untouched rows keep everything.
  w, a, s = lo.apply_f2a(one(2.0), one(0.0), one(3.0), one(3.0), ~hit, 0.1, 1.0, 0.5, 0.25, 1e6, 8.0)
  assert (w.item(), a.item(), s.item()) == (2.0, 0.0, 3.0)


def test_quantization_config_validation():
  with pytest.raises(ValueError):
    es.QuantizationConfig(min_value=0.0, max_value=1.0, num_buckets=1)
  with pytest.raises(ValueError):
    es.QuantizationConfig(min_value=1.0, max_value=1.0, num_buckets=4)
  assert es.QuantizationConfig(min_value=0.0, max_value=1.0, num_buckets=4).as_tuple() == (0.0, 1.0, 4)


def test_stats_required_buffer_helpers():
  st = embedding.SparseDenseMatmulInputStats({"t": np.array([5, 9])}, {"t": np.array([3, 4])},
                                             {"t": np.array([16, 24])}, {"t": 0})
  assert st.get_required_buffer_size_per_device("t") == 48
  assert st.get_required_buffer_size_per_device("t", 4) == 96
  assert st.get_required_buffer_size_per_device("missing") is None
  st.set_required_buffer_size_per_device("u", 64, 2)
  np.testing.assert_array_equal(st.required_buffer_size_per_sc["u"], [32, 32])


def test_update_preprocessing_parameters():
  t = _table("t", 64, 8)
  f = _feature("f", t, 8)
  embedding.prepare_feature_specs_for_training([f], 1, 2)
  st = embedding.SparseDenseMatmulInputStats({"t": np.array([5, 9])}, {"t": np.array([3, 4])}, {"t": np.array([16, 24])})
  embedding.update_preprocessing_parameters([f], st, 2)
  spec = t.stacked_table_spec
  assert (spec.max_ids_per_partition, spec.max_unique_ids_per_partition) == (9, 4)
  assert spec.suggested_coo_buffer_size_per_device == 48


def test_tree_helpers_follow_sorted_dict_order():
  tree = {"b": [1, 2], "a": (3, None), "c": {"z": 4}}
  assert _tree.leaves(tree) == [3, 1, 2, 4]
  doubled = _tree.tree_map(lambda x: 2 * x, tree)
  assert doubled == {"b": [2, 4], "a": (6, None), "c": {"z": 8}}
  flat, proto = _tree.flatten(tree)
  assert _tree.unflatten(proto, flat) == tree
  with pytest.raises(ValueError):
    _tree.assert_same_structure({"a": 1}, {"b": 1})
  with pytest.raises(ValueError, match="do not match"):
    embedding._assert_same_structure([np.zeros(1)], [np.zeros(1), np.zeros(1)], "x", "y")  # pylint: disable=protected-access


def test_eval_shape_and_spec_lookups():
  tables = [_table("a", 100, 8, max_ids_per_partition=64), _table("b", 30, 8, max_ids_per_partition=20)]
  feats = {"x": _feature("fa", tables[0], 16), "y": _feature("fb", tables[1], 16)}
  with pytest.raises(ValueError, match="prepare_feature_specs_for_training was not called"):
    embedding.get_stacked_table_specs(feats)
  embedding.prepare_feature_specs_for_training(feats, 2, 2)
  assert set(embedding.get_stacked_table_specs(feats)) == {"a", "b"}
  assert set(embedding.get_table_specs(feats)) == {"a", "b"}
  shapes = embedding.eval_preprocess_sparse_dense_matmul_input_shape(feats, 1, 2, num_sc_per_device=2)
  assert shapes.lhs_row_pointers["a"].shape == (16,)
  assert shapes.lhs_embedding_ids["a"].shape == (64 * 2 * 4,) and shapes.lhs_gains["b"].shape == (24 * 2 * 4,)
  dup = [_feature("same", tables[0], 16), _feature("same", tables[1], 16)]
  with pytest.raises(ValueError, match="already defined"):
    embedding.get_table_specs(dup)


def test_spec_facts_are_remembered_per_tree_and_follow_restacking():
  """The per-tree facts are memoised by the identity of the tree; stacking the tables again must not reuse them."""
  tables = [_table("a", 100, 8), _table("b", 30, 8)]
  feats = [_feature(f"f{i}", t, 16) for i, t in enumerate(tables)]
  embedding.prepare_feature_specs_for_training(feats, global_device_count=1, num_sc_per_device=1)
  first = embedding._spec_info(feats)  # pylint: disable=protected-access
  assert embedding._spec_info(feats) is first  # pylint: disable=protected-access
  assert set(first.stacked) == {"a", "b"} and first.flat_stack_names == ["a", "b"]
  # The same list object, other stacked specs: the memo must notice.
  ts.stack_tables(feats, ["a", "b"], global_device_count=1, num_sc_per_device=1, stack_name="ab")
  second = embedding._spec_info(feats)  # pylint: disable=protected-access
  assert second is not first and set(second.stacked) == {"ab"}
  # A longer list that starts with the same features is another tree.
  extra = _feature("g", _table("c", 50, 8), 16)
  embedding.prepare_feature_specs_for_training([extra], global_device_count=1, num_sc_per_device=1)
  third = embedding._spec_info(feats + [extra])  # pylint: disable=protected-access
  assert set(third.stacked) == {"ab", "c"}
  embedding.clear_caches()
  assert embedding._spec_info(feats) is not second  # pylint: disable=protected-access
