"""Launch descriptors that are cached by the layout of a preprocessing output and moved to new buffers.

CPU part: the pointer arithmetic of `_ops._CsrFields` on ctypes descriptor arrays (no GPU call).
GPU part: a loop over DIFFERENT batches of one layout whose buffers are all kept alive (so every batch lives at
other addresses) must replay the cached descriptors, and every step must give what a fresh process state gives.
"""

import ctypes

import numpy as np
import pytest

from jax_tpu_embedding.sparsecore import _native
from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops


def _items(item_type, n, ibase, fbase, with_plan):
  items = (item_type * n)()
  for j in range(n):
    items[j].csr.row_pointers = ibase + 1000 * j
    items[j].csr.embedding_ids = ibase + 1000 * j + 64
    items[j].csr.sample_ids = ibase + 1000 * j + 512
    items[j].csr.gains = fbase + 400 * j
    if with_plan and j != 1:  # the second descriptor has no plan: its null pointers must stay null
      items[j].plan_slots = ibase + 50000 + 100 * j
      items[j].plan_bags = ibase + 60000 + 100 * j
  return items


@pytest.mark.parametrize("item_type,with_plan", [(_native.FwdItem, True), (_native.GradItem, False)])
def test_rebase_moves_every_csr_pointer_and_nothing_else(item_type, with_plan):
  n, ibase, fbase = 3, 0x7F0000000000, 0x7F1000000000
  items = _items(item_type, n, ibase, fbase, with_plan)
  before = bytes(items)
  fields = _ops._CsrFields(items, item_type, n, (ibase, fbase), with_plan)  # pylint: disable=protected-access
  fields.rebase((ibase, fbase))
  assert bytes(items) == before
  new_i, new_f = 0x7E0000001000, 0x7F2000000400
  fields.rebase((new_i, new_f))
  want = _items(item_type, n, new_i, new_f, with_plan)
  assert bytes(items) == bytes(want)
  fields.rebase((ibase, fbase))
  assert bytes(items) == before
  assert ctypes.sizeof(items) == n * ctypes.sizeof(item_type)


@pytest.mark.gpu
def test_replayed_descriptors_follow_the_buffers_of_each_batch():
  import torch

  import cases
  from jax_tpu_embedding.sparsecore.lib.nn import embedding

  def make(seed):
    return cases.make_case("rebase", seed=seed, batch=512, optimizer="adagrad", max_ids=4096, max_unique=4096, tables=[
        dict(vocab=3000, dim=32, features=[dict(kind="dense", valency=3, dist="zipf", a=1.1)]),
        dict(vocab=500, dim=128, features=[dict(kind="dense", valency=1, dist="uniform")])])

  first = make(1)
  specs = first.feature_specs
  stacks = embedding.get_stacked_table_specs(specs)
  rng = np.random.default_rng(0)

  def variables():
    out = {}
    gen = np.random.default_rng(5)
    for name, spec in stacks.items():
      rows = spec.stack_vocab_size
      tab = torch.from_numpy(gen.normal(0, 0.01, size=(rows, spec.stack_embedding_dim)).astype(np.float32)).cuda()
      out[name] = embedding.EmbeddingVariables(tab, (torch.full_like(tab, 0.1),))
    return out

  def step(case, var, keep):
    feats = [torch.from_numpy(np.ascontiguousarray(f, dtype=np.int32)).cuda() for f in case.features]
    pre, _ = embedding.preprocess_sparse_dense_matmul_input(feats, None, specs, 1, 1, num_sc_per_device=1)
    keep.append(pre)  # alive: the next batch cannot get these addresses
    acts = embedding.tpu_sparse_dense_matmul(pre, var, specs, global_device_count=1, num_sc_per_device=1)
    grads = [torch.full_like(a, 0.01) * (i + 1) for i, a in enumerate(acts)]
    embedding.tpu_sparse_dense_matmul_grad(grads, pre, var, specs, global_device_count=1, num_sc_per_device=1, step=0)
    torch.cuda.synchronize()
    return [a.cpu().numpy() for a in acts]

  batches = [make(seed) for seed in (1, 2, 3, 4, 5)]
  for b in batches[1:]:
    b.feature_specs = specs  # same spec objects: one layout, one cached descriptor set
  # Reference: every step with freshly built descriptors.
  ref_var, ref_acts = variables(), []
  for b in batches:
    embedding.clear_caches()
    ref_acts.append(step(b, ref_var, []))
  # Same steps with the caches on and all buffers kept alive.
  embedding.clear_caches()
  var, keep = variables(), []
  before = dict(embedding.CALL_CACHE_STATS)
  got_acts = [step(b, var, keep) for b in batches]
  built = embedding.CALL_CACHE_STATS["built"] - before["built"]
  replayed = embedding.CALL_CACHE_STATS["replayed"] - before["replayed"]
  assert built == 2 and replayed == 2 * (len(batches) - 1), (built, replayed)
  addresses = {p.sparse_dense_matmul_input[0].token[:2] for p in keep}
  assert len(addresses) == len(batches), "every batch must live in buffers of its own"
  for got, want in zip(got_acts, ref_acts):
    for g, w in zip(got, want):
      np.testing.assert_array_equal(g, w)
  for name in stacks:
    np.testing.assert_array_equal(var[name].table.cpu().numpy(), ref_var[name].table.cpu().numpy())
    np.testing.assert_array_equal(var[name].slot[0].cpu().numpy(), ref_var[name].slot[0].cpu().numpy())
  del rng


def test_csr_key_separates_layout_from_buffer_addresses():
  """Two outputs of one layout share the cache key and differ in `bases`; a replaced array drops the token."""
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip
  from jax_tpu_embedding.sparsecore.lib.nn import embedding

  layout = object()

  def output(ibase, fbase):
    dicts = []
    for i in range(4):
      d = pip.BufferDict({"t": np.zeros(4)})
      d.token = (ibase, fbase, layout, False, i)
      dicts.append(d)
    return dicts

  a, b = output(1 << 40, 2 << 40), output(3 << 40, 4 << 40)
  key_a, bases_a = embedding._csr_key(*a, ["t"])  # pylint: disable=protected-access
  key_b, bases_b = embedding._csr_key(*b, ["t"])  # pylint: disable=protected-access
  assert key_a == key_b and bases_a == (1 << 40, 2 << 40) and bases_b == (3 << 40, 4 << 40)
  # Dicts of two different outputs mixed in one call: no common pair of buffers, the full tokens key the cache.
  mixed_key, mixed_bases = embedding._csr_key(a[0], b[1], a[2], a[3], ["t"])  # pylint: disable=protected-access
  assert mixed_bases is None and mixed_key != key_a
  # Replacing an array drops the token: the dict is described by its arrays (here: not device tensors -> no caching).
  a[1]["t"] = np.ones(4)
  assert a[1].token is None
  assert embedding._csr_key(*a, ["t"]) == (None, None)  # pylint: disable=protected-access
