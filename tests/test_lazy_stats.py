"""Host-side pieces of the step's fast path: deferred statistics dicts and the flat-list shortcuts."""

import numpy as np
import pytest

from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip
from jax_tpu_embedding.sparsecore.lib.nn import embedding
from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec


class _Deferred:
  """Stands in for the statistics block on its way to the host."""

  def __init__(self, fields=None, error=None):
    self.fields, self.error, self.calls = fields, error, 0

  def resolve(self):
    self.calls += 1
    if self.error is not None:
      raise self.error
    return self.fields


def test_lazy_dict_fills_once_on_first_use():
  d = _Deferred(fields=({"t": np.array([3, 4])}, {"t": np.array([1, 2])}, {"t": np.array([16])}, {"t": 0}))
  ids = pip.LazyStatsDict(deferred=d, field=0)
  uniq = pip.LazyStatsDict(deferred=d, field=1)
  assert d.calls == 0
  assert "t" in ids and list(ids) == ["t"] and len(ids) == 1
  np.testing.assert_array_equal(ids["t"], [3, 4])
  assert d.calls == 1
  np.testing.assert_array_equal(dict(uniq)["t"], [1, 2])
  assert d.calls == 2  # one resolve per dict, none afterwards
  assert uniq.get("missing") is None and d.calls == 2
  # dataclasses.asdict (used by the FDO clients) walks the dict through items().
  stats = embedding.SparseDenseMatmulInputStats(max_ids_per_partition=ids, max_unique_ids_per_partition=uniq)
  import dataclasses

  np.testing.assert_array_equal(dataclasses.asdict(stats)["max_ids_per_partition"]["t"], [3, 4])


def test_lazy_dict_raises_the_deferred_error_on_use():
  lazy = pip.LazyStatsDict(deferred=_Deferred(error=ValueError("Observed max ids per partition: 9")), field=0)
  with pytest.raises(ValueError, match="max ids per partition"):
    lazy["t"]


def test_flat_lists_take_the_shortcut_and_nested_trees_do_not():
  t = embedding_spec.TableSpec(name="t", vocabulary_size=16, embedding_dim=8, initializer=None,
                               optimizer=embedding_spec.SGDOptimizerSpec(), combiner="sum")
  f = [embedding_spec.FeatureSpec(name=f"f{i}", table_spec=t, input_shape=[4, 1], output_shape=[4, 8]) for i in range(3)]
  arrays = [np.zeros((4, 1), np.int32) for _ in range(3)]
  assert embedding._flat_leaves(f) and embedding._flat_leaves(tuple(arrays))  # pylint: disable=protected-access
  assert not embedding._flat_leaves({"a": f[0]}) and not embedding._flat_leaves([f[0], [f[1]]])  # pylint: disable=protected-access
  assert embedding._leaves(f) == f and embedding._leaves({"b": f[1], "a": f[0]}) == [f[0], f[1]]  # pylint: disable=protected-access
  embedding._assert_same_structure(f, arrays)  # pylint: disable=protected-access
  with pytest.raises(ValueError, match="do not match"):
    embedding._assert_same_structure(f, arrays[:2])  # pylint: disable=protected-access
