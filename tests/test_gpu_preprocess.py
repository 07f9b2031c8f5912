"""GPU preprocessing vs the CPU oracle: bit-exact buffers, row pointers and statistics."""

import numpy as np
import pytest

import cases
import oracle_backend as ob
from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip
from jax_tpu_embedding.sparsecore.lib.nn import embedding

pytestmark = pytest.mark.gpu

CASES = cases.standard_cases()


def _compare(case, got, want):
  slices = case.local_device_count * case.num_sc_per_device
  for name in want[0]:
    ob.written_region_equal(got[0][name], want[0][name], [got[i][name] for i in (1, 2, 3)],
                            [want[i][name] for i in (1, 2, 3)], slices)
    gs, ws = got[5], want[5]
    np.testing.assert_array_equal(gs.max_ids_per_partition[name], ws.max_ids_per_partition[name])
    np.testing.assert_array_equal(gs.max_unique_ids_per_partition[name], ws.max_unique_ids_per_partition[name])
    np.testing.assert_array_equal(gs.required_buffer_sizes[name], ws.required_buffer_sizes[name])
    assert gs.dropped_id_count[name] == ws.dropped_id_count[name]


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
@pytest.mark.parametrize("leading", [False, True])
def test_preprocess_matches_oracle(case, leading):
  kw = dict(num_sc_per_device=case.num_sc_per_device, has_leading_dimension=leading,
            allow_id_dropping=case.allow_id_dropping)
  got = pip.preprocess_sparse_dense_matmul_input(case.features, case.weights, case.feature_specs,
                                                 case.local_device_count, case.global_device_count, **kw)
  want = ob.oracle_preprocess(case.features, case.weights, case.feature_specs, case.local_device_count,
                              case.global_device_count, **kw)
  _compare(case, got, want)
  if leading:
    for name in want[0]:
      assert got[1][name].shape == want[1][name].shape


def test_tail_is_padding():
  case = CASES[0]
  rp, ids, sids, gains, _, _ = pip.preprocess_sparse_dense_matmul_input(
      case.features, None, case.feature_specs, 1, 1, num_sc_per_device=1)
  for name in rp:
    last = rp[name][-1]
    assert (ids[name][last:] == 2**31 - 1).all() and (sids[name][last:] == 2**31 - 1).all()
    assert np.isnan(gains[name][last:]).all()


def test_id_limit_raises_value_error():
  case = cases.make_case("limit", seed=1, tables=[dict(vocab=64, dim=8)], batch=64, max_ids=4, max_unique=4)
  with pytest.raises(ValueError, match="is greater than the set max"):
    pip.preprocess_sparse_dense_matmul_input(case.features, None, case.feature_specs, 1, 1, num_sc_per_device=1)


def test_unity_weights_same_as_none():
  for combiner in ("sum", "mean", "sqrtn"):
    case = cases.make_case("u", seed=5, tables=[dict(vocab=500, dim=8, features=[dict(kind="dense", valency=6)])],
                           batch=128, combiner=combiner, dup_prob=0.2)
    ones = [np.ones_like(case.features[0], dtype=np.float32)]
    a = pip.preprocess_sparse_dense_matmul_input(case.features, None, case.feature_specs, 1, 1, num_sc_per_device=1)
    b = pip.preprocess_sparse_dense_matmul_input(case.features, ones, case.feature_specs, 1, 1, num_sc_per_device=1)
    for name in a[0]:
      np.testing.assert_array_equal(a[0][name], b[0][name])
      last = a[0][name][-1]
      np.testing.assert_array_equal(a[1][name][:last], b[1][name][:last])
      np.testing.assert_allclose(a[3][name][:last], b[3][name][:last], rtol=1e-6)


def test_ragged_input_leaf_and_device_output():
  import torch

  case = CASES[3]
  rows = case.features[0]
  lens = np.array([len(r) for r in rows])
  splits = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
  ragged = embedding.RaggedInput(np.concatenate(list(rows)).astype(np.int32), splits)
  pre_a, stats_a = embedding.preprocess_sparse_dense_matmul_input(
      [ragged], None, case.feature_specs, 1, 1, num_sc_per_device=1)
  pre_b, stats_b = embedding.preprocess_sparse_dense_matmul_input(
      case.features, None, case.feature_specs, 1, 1, num_sc_per_device=1, device_output=False)
  for name in pre_b.lhs_row_pointers:
    assert isinstance(pre_a.lhs_embedding_ids[name], torch.Tensor) and pre_a.lhs_embedding_ids[name].is_cuda
    np.testing.assert_array_equal(pre_a.lhs_row_pointers[name].cpu().numpy(), pre_b.lhs_row_pointers[name])
    np.testing.assert_array_equal(pre_a.lhs_embedding_ids[name].cpu().numpy(), pre_b.lhs_embedding_ids[name])
    np.testing.assert_array_equal(stats_a.max_ids_per_partition[name], stats_b.max_ids_per_partition[name])


def test_invalid_arguments():
  case = CASES[0]
  with pytest.raises(ValueError, match="local_device_count must be greater than 0"):
    pip.preprocess_sparse_dense_matmul_input(case.features, None, case.feature_specs, 0, 1, num_sc_per_device=1)
  with pytest.raises(ValueError, match="must be a power of 2"):
    pip.preprocess_sparse_dense_matmul_input(case.features, None, case.feature_specs, 1, 3, num_sc_per_device=1)
  with pytest.raises(ValueError, match="cannot be empty"):
    pip.preprocess_sparse_dense_matmul_input([], None, [], 1, 1, num_sc_per_device=1)


@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("stack", [False, True])
def test_dense_device_inputs_take_the_cached_plan(weighted, stack):
  """Dense int32 CUDA tensors use prebuilt launch descriptors; results equal the general path and the oracle,
  also when the plan is reused with new data, and the outputs carry a buffer token."""
  import torch

  def make(seed):
    return cases.make_case(
        "dense_plan", seed=seed, batch=256, num_sc_per_device=2, combiner="mean", stack=stack, max_ids=4096,
        max_unique=4096, weights=True if weighted else None,
        tables=[dict(vocab=3000, dim=16, features=[dict(kind="dense", valency=3, dist="zipf"), dict(kind="dense", valency=1)]),
                dict(vocab=500, dim=16, features=[dict(kind="dense", valency=2)])])

  case = make(31)
  kw = dict(num_sc_per_device=2, has_leading_dimension=False)
  for seed in (31, 32):  # the second round reuses the plan of the first
    data = make(seed)
    feats = [torch.from_numpy(f).cuda() for f in data.features]
    weights = None if data.weights is None else [torch.from_numpy(w).cuda() for w in data.weights]
    got = pip.preprocess_sparse_dense_matmul_input(feats, weights, case.feature_specs, 1, 1, device_output=True, **kw)
    want = ob.oracle_preprocess(data.features, data.weights, case.feature_specs, 1, 1, **kw)
    assert isinstance(got[0], pip.BufferDict) and got[0].token is not None and got[3].token is not None
    host = tuple({k: v.cpu().numpy() for k, v in d.items()} for d in got[:4]) + got[4:]
    _compare(case, host, want)
    general = pip.preprocess_sparse_dense_matmul_input(data.features, data.weights, case.feature_specs, 1, 1, **kw)
    _compare(case, general, want)
  got[0]["extra"] = None
  assert got[0].token is None


def test_sparse_coo_input_equals_ragged_input():
  """The same bags as sparse tensors (indices, values, dense shape) give the same buffers as ragged rows."""
  case = cases.make_case("coo", seed=77, batch=64, num_sc_per_device=2, combiner="mean", stack=True, max_ids=2048,
                         max_unique=2048,
                         tables=[dict(vocab=900, dim=16, features=[dict(kind="ragged", min_len=0, max_len=7)]),
                                 dict(vocab=300, dim=16, features=[dict(kind="ragged", max_len=4, dist="zipf")])])
  indices, values, shapes = [], [], []
  for feat in case.features:
    idx = [(r, j) for r, row in enumerate(feat) for j in range(len(row))]
    indices.append(np.asarray(idx, dtype=np.int64).reshape(-1, 2))
    values.append(np.concatenate([np.asarray(row, np.int32) for row in feat]))
    shapes.append(np.asarray([len(feat), max(len(row) for row in feat)], dtype=np.int64))
  kw = dict(num_sc_per_device=2)
  got = pip.preprocess_sparse_dense_matmul_sparse_coo_input(indices, values, shapes, case.feature_specs, 1, 1, **kw)
  want = ob.oracle_preprocess(case.features, None, case.feature_specs, 1, 1, **kw)
  _compare(case, got, want)
  pre, stats = embedding.preprocess_sparse_dense_matmul_input_from_sparse_tensor(
      indices, values, shapes, case.feature_specs, 1, 1, num_sc_per_device=2)
  for name in want[0]:
    np.testing.assert_array_equal(pre.lhs_row_pointers[name].cpu().numpy(), want[0][name])
  assert pre.num_minibatches.dtype == np.int32
  with pytest.raises(ValueError, match="row-major"):
    pip.preprocess_sparse_dense_matmul_sparse_coo_input([indices[0][::-1]], [values[0]], [shapes[0]],
                                                        case.feature_specs[:1], 1, 1, **kw)


def test_deferred_statistics_equal_the_synchronous_ones_and_raise_late():
  """sync_stats=False: same buffers and statistics, no wait inside the call; a violated limit raises when the
  statistics are read, or at the next call."""
  import torch

  case = cases.make_case("deferred", seed=21, batch=512, tables=[
      dict(vocab=5000, dim=16, features=[dict(kind="dense", valency=3, dist="zipf")]),
      dict(vocab=300, dim=16, features=[dict(kind="dense", valency=1)])])
  feats = [torch.from_numpy(f).cuda() for f in case.features]
  want, want_stats = embedding.preprocess_sparse_dense_matmul_input(feats, None, case.feature_specs, 1, 1, num_sc_per_device=1)
  got, got_stats = embedding.preprocess_sparse_dense_matmul_input(feats, None, case.feature_specs, 1, 1, num_sc_per_device=1,
                                                                  sync_stats=False)
  for a, b in zip(got.sparse_dense_matmul_input, want.sparse_dense_matmul_input):
    for name in b:
      assert torch.equal(a[name].view(torch.int32), b[name].view(torch.int32))
  assert set(got_stats.max_ids_per_partition) == set(want_stats.max_ids_per_partition)
  for name in want_stats.max_ids_per_partition:
    np.testing.assert_array_equal(got_stats.max_ids_per_partition[name], want_stats.max_ids_per_partition[name])
    np.testing.assert_array_equal(got_stats.max_unique_ids_per_partition[name], want_stats.max_unique_ids_per_partition[name])
    np.testing.assert_array_equal(got_stats.required_buffer_size_per_sc[name], want_stats.required_buffer_size_per_sc[name])
    assert got_stats.id_drop_counters[name] == want_stats.id_drop_counters[name]
  # A limit below what the batch needs: the synchronous call raises at once, the deferred one when asked.
  tight = cases.make_case("deferred_tight", seed=21, batch=512, max_ids=16, max_unique=16, tables=[
      dict(vocab=5000, dim=16, features=[dict(kind="dense", valency=3, dist="zipf")])])
  tfeats = [torch.from_numpy(f).cuda() for f in tight.features]
  with pytest.raises(ValueError, match="max ids per partition"):
    embedding.preprocess_sparse_dense_matmul_input(tfeats, None, tight.feature_specs, 1, 1, num_sc_per_device=1)
  _, late = embedding.preprocess_sparse_dense_matmul_input(tfeats, None, tight.feature_specs, 1, 1, num_sc_per_device=1,
                                                           sync_stats=False)
  with pytest.raises(ValueError, match="max ids per partition"):
    len(late.max_ids_per_partition)
  _, late2 = embedding.preprocess_sparse_dense_matmul_input(tfeats, None, tight.feature_specs, 1, 1, num_sc_per_device=1,
                                                            sync_stats=False)
  torch.cuda.synchronize()
  with pytest.raises(ValueError, match="max ids per partition"):  # the previous call's violation surfaces here
    embedding.preprocess_sparse_dense_matmul_input(tfeats, None, tight.feature_specs, 1, 1, num_sc_per_device=1,
                                                   sync_stats=False)
  del late2
