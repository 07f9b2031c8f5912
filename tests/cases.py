"""Seeded synthetic workloads shared by the parity tests (shapes follow the benchmark configs)."""

from __future__ import annotations

import dataclasses

import numpy as np

from jax_tpu_embedding.sparsecore.lib.nn import embedding
from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec
from jax_tpu_embedding.sparsecore.lib.nn import table_stacking


@dataclasses.dataclass
class Case:
  name: str
  feature_specs: list
  features: list
  weights: list | None
  global_device_count: int
  num_sc_per_device: int
  local_device_count: int
  allow_id_dropping: bool = False


def zipf_ids(rng, vocab, size, a):
  """Bounded Zipf: P(k) ~ (k + 1)^-a for k in [0, vocab), by inverse CDF."""
  ranks = np.arange(1, vocab + 1, dtype=np.float64)
  cdf = np.cumsum(ranks ** (-a))
  cdf /= cdf[-1]
  return np.searchsorted(cdf, rng.random(size), side="left").astype(np.int32)


def _optimizer(kind):
  if kind == "sgd":
    return embedding_spec.SGDOptimizerSpec(learning_rate=0.01)
  if kind == "adagrad":
    return embedding_spec.AdagradOptimizerSpec(learning_rate=0.01, initial_accumulator_value=0.1)
  return embedding_spec.AdamOptimizerSpec(learning_rate=1e-3, beta_1=0.9, beta_2=0.999)


def make_case(name, *, seed, tables, batch, global_device_count=1, num_sc_per_device=1, local_device_count=None,
              combiner="sum", optimizer="sgd", weights=None, stack=False, max_ids=None, max_unique=None,
              allow_id_dropping=False, suggested=None, dup_prob=0.0):
  """tables: list of dict(vocab, dim, features=[dict(kind='dense'|'ragged', valency|max_len, dist)])."""
  rng = np.random.default_rng(seed)
  c, s = global_device_count, num_sc_per_device
  l = c if local_device_count is None else local_device_count
  local_batch = batch // c * l
  specs, feats, wts = [], [], []
  opt = _optimizer(optimizer)
  for ti, t in enumerate(tables):
    tspec = embedding_spec.TableSpec(
        name=f"table_{ti}", vocabulary_size=t["vocab"], embedding_dim=t["dim"], initializer=None, optimizer=opt,
        combiner=combiner, max_ids_per_partition=max_ids or 1 << 15, max_unique_ids_per_partition=max_unique or 1 << 15,
        suggested_coo_buffer_size_per_device=suggested)
    for fi, f in enumerate(t.get("features", [dict(kind="ragged", max_len=8)])):
      valency = f.get("valency")
      specs.append(embedding_spec.FeatureSpec(
          name=f"feature_{ti}_{fi}", table_spec=tspec, input_shape=[batch, valency] if valency else [batch],
          output_shape=[batch, t["dim"]]))
      dist = f.get("dist", "uniform")
      def draw(n):
        if dist == "zipf":
          return zipf_ids(rng, t["vocab"], n, f.get("a", 1.05))
        return rng.integers(0, t["vocab"], size=n).astype(np.int32)
      if f.get("kind", "ragged") == "dense":
        arr = draw(local_batch * valency).reshape(local_batch, valency)
        if dup_prob:
          dup = rng.random(arr.shape) < dup_prob
          arr = np.where(dup, arr[:, :1], arr)
        feats.append(arr)
        wts.append(rng.uniform(0.5, 1.5, size=arr.shape).astype(np.float32))
      else:
        lo, hi = f.get("min_len", 1), f.get("max_len", 8)
        lens = rng.integers(lo, hi + 1, size=local_batch)
        flat = draw(int(lens.sum()))
        rows = np.empty(local_batch, dtype=object)
        wrows = np.empty(local_batch, dtype=object)
        pos = 0
        for i, n in enumerate(lens):
          row = flat[pos:pos + n].copy()
          if dup_prob and n > 1:
            dup = rng.random(n) < dup_prob
            row[dup] = row[0]
          rows[i] = row
          wrows[i] = rng.uniform(0.5, 1.5, size=n).astype(np.float32)
          pos += n
        feats.append(rows)
        wts.append(wrows)
  if stack:
    table_stacking.stack_tables(specs, [f"table_{i}" for i in range(len(tables))], c, s,
                                stack_to_max_ids_per_partition=lambda n, b: max_ids or 1 << 15,
                                stack_to_max_unique_ids_per_partition=lambda n, b: max_unique or 1 << 15,
                                activation_mem_bytes_limit=1 << 40)
    if suggested is not None:
      for f in specs:
        f.table_spec.stacked_table_spec = dataclasses.replace(
            f.table_spec.stacked_table_spec, suggested_coo_buffer_size_per_device=suggested)
  else:
    embedding.prepare_feature_specs_for_training(specs, c, s)
  use_weights = weights if weights is not None else False
  return Case(name, specs, feats, wts if use_weights else None, c, s, l, allow_id_dropping)


def standard_cases():
  """A spread of layouts: combiners, weights, stacking, virtual SparseCores and devices, limits."""
  t1 = [dict(vocab=4096, dim=16, features=[dict(kind="ragged", max_len=8)])]
  out = [
      make_case("c1_small_sum_sgd", seed=101, tables=t1, batch=64),
      make_case("dense_single_hot_zipf", seed=202, tables=[dict(vocab=50000, dim=128, features=[dict(kind="dense", valency=1, dist="zipf")])],
                batch=4096, optimizer="adagrad"),
      make_case("multi_hot_weighted_sqrtn", seed=303, tables=[dict(vocab=20000, dim=64, features=[dict(kind="ragged", max_len=64, dist="zipf", a=1.1)])],
                batch=1024, combiner="sqrtn", optimizer="adagrad", weights=True, dup_prob=0.2),
      make_case("mean_unity_dups", seed=404, tables=[dict(vocab=300, dim=32, features=[dict(kind="ragged", max_len=32, dist="zipf")])],
                batch=512, combiner="mean", optimizer="adam", dup_prob=0.3),
      make_case("sqrtn_unity", seed=405, tables=[dict(vocab=1000, dim=24, features=[dict(kind="dense", valency=5)])],
                batch=256, combiner="sqrtn", dup_prob=0.3),
      make_case("mean_weighted", seed=406, tables=[dict(vocab=1000, dim=8, features=[dict(kind="dense", valency=7)])],
                batch=256, combiner="mean", weights=True, dup_prob=0.3, optimizer="adam"),
      make_case("stacked_features_4sc", seed=505,
                tables=[dict(vocab=777, dim=32, features=[dict(kind="ragged", max_len=16), dict(kind="dense", valency=3)]),
                        dict(vocab=123, dim=30, features=[dict(kind="ragged", max_len=5)]),
                        dict(vocab=4000, dim=32, features=[dict(kind="ragged", min_len=0, max_len=9)])],
                batch=256, num_sc_per_device=4, combiner="mean", optimizer="adam", stack=True),
      make_case("two_devices_two_sc", seed=606,
                tables=[dict(vocab=5000, dim=16, features=[dict(kind="ragged", max_len=12, dist="zipf")]),
                        dict(vocab=900, dim=16, features=[dict(kind="ragged", max_len=4)])],
                batch=512, global_device_count=2, num_sc_per_device=2, optimizer="adagrad", stack=True),
      make_case("eight_devices", seed=707, tables=[dict(vocab=100000, dim=128, features=[dict(kind="ragged", max_len=32, dist="zipf")])],
                batch=1024, global_device_count=8, combiner="mean", optimizer="adagrad"),
      make_case("id_dropping", seed=808, tables=[dict(vocab=64, dim=8, features=[dict(kind="ragged", max_len=20)])],
                batch=128, num_sc_per_device=2, max_ids=40, max_unique=9, allow_id_dropping=True, dup_prob=0.3),
      make_case("static_buffer_overflow", seed=909, tables=[dict(vocab=512, dim=8, features=[dict(kind="ragged", max_len=20)])],
                batch=128, num_sc_per_device=2, global_device_count=2, local_device_count=2, max_ids=1000, max_unique=1000,
                suggested=600, allow_id_dropping=True),
  ]
  return out
