"""Forward and fused backward kernels vs the numpy oracle, on oracle-produced CSR buffers.

Tolerance: 1e-5 relative (float32).  Sums whose terms cancel have no elementwise relative bound,
so the absolute floor is 1e-6 of the largest magnitude of the expected array.  Where all terms are
added in the oracle's order (the whole forward pass) the results are compared bit for bit.
"""

import numpy as np
import pytest

import cases
import oracle_backend as ob
from oracle import lookup_oracle as lo
from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_csr
from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_grad_with_adagrad
from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_grad_with_adam
from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_grad_with_sgd

pytestmark = pytest.mark.gpu

RTOL = 1e-5


def assert_close(got, want):
  want = np.asarray(want)
  np.testing.assert_allclose(np.asarray(got).reshape(want.shape), want, rtol=RTOL,
                             atol=1e-6 * float(np.abs(want).max()) + 1e-12)

CASES = [c for c in cases.standard_cases() if c.local_device_count == c.global_device_count]


def _setup(case, seed=0, dim_override=None):
  """Oracle CSR per stack plus random shards / gradients."""
  import torch

  out = ob.oracle_preprocess(case.features, case.weights, case.feature_specs, case.local_device_count,
                             case.global_device_count, num_sc_per_device=case.num_sc_per_device,
                             allow_id_dropping=case.allow_id_dropping, has_leading_dimension=True)
  rng = np.random.default_rng(seed)
  stacks = {}
  p = case.global_device_count * case.num_sc_per_device
  for name in out[0]:
    spec = next(f.table_spec.stacked_table_spec for f in case.feature_specs
                if f.table_spec.stacked_table_spec.stack_name == name)
    rows = spec.stack_vocab_size // p
    dim = dim_override or spec.stack_embedding_dim
    bdev = spec.total_sample_count // case.global_device_count
    shards = rng.normal(0, 0.01, size=(p, rows, dim)).astype(np.float32)
    csr = [tuple(out[i][name][d] for i in range(4)) for d in range(case.local_device_count)]
    grads = [(rng.normal(0, 1, size=(bdev, dim)) * 1e-2).astype(np.float32) for _ in csr]
    stacks[name] = dict(spec=spec, shards=shards, csr=csr, grads=grads, bdev=bdev, flat=[
        torch.from_numpy(np.concatenate([c[i] for c in csr])).cuda() for i in range(4)])
  return stacks


def _kw(case, spec):
  return dict(max_ids_per_partition=spec.max_ids_per_partition,
              max_unique_ids_per_partition=spec.max_unique_ids_per_partition,
              num_sc_per_device=case.num_sc_per_device, global_device_count=case.global_device_count,
              local_device_count=case.local_device_count)


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_forward_matches_oracle(case):
  import torch

  for name, st in _setup(case).items():
    want = np.concatenate(lo.forward(st["csr"], st["shards"], num_sc_per_device=case.num_sc_per_device,
                                     device_batch_size=st["bdev"]))
    table = torch.from_numpy(st["shards"].reshape(-1, st["shards"].shape[-1])).cuda()
    got = sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.bind(
        *st["flat"], np.int32(1), table, device_batch_size=st["bdev"], **_kw(case, st["spec"]))
    got2 = sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.bind(
        *st["flat"], np.int32(1), table, device_batch_size=st["bdev"], **_kw(case, st["spec"]))
    assert torch.equal(got, got2), "forward is not run-to-run reproducible"
    # Same summation order as the oracle (ascending shard, row): identical bits.
    np.testing.assert_array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("opt", ["sgd", "adagrad", "adam"])
@pytest.mark.parametrize("clip", [None, (-0.012, 0.011)])
@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_backward_matches_oracle(case, opt, clip):
  import torch

  rng = np.random.default_rng(7)
  for name, st in _setup(case).items():
    shards = st["shards"]
    g, touched = lo.table_gradient(st["csr"], st["grads"], shards.shape, num_sc_per_device=case.num_sc_per_device)
    lo_, hi_ = clip if clip else (None, None)
    slot0 = rng.uniform(0.05, 0.2, size=shards.shape).astype(np.float32)
    slot1 = rng.uniform(0.0, 1e-4, size=shards.shape).astype(np.float32)
    dev = lambda a: torch.from_numpy(a.reshape(-1, a.shape[-1]).copy()).cuda()
    grad = torch.from_numpy(np.concatenate(st["grads"])).cuda()
    kw = dict(_kw(case, st["spec"]), min_value=lo_, max_value=hi_)
    if opt == "sgd":
      want = lo.apply_sgd(shards, g, touched, 0.01, lo_, hi_)
      got = (sparse_dense_matmul_grad_with_sgd.tpu_sparse_dense_matmul_grad_with_sgd_primitive.bind(
          *st["flat"], np.int32(1), dev(shards), grad, np.float32(0.01), **kw),)
    elif opt == "adagrad":
      want = lo.apply_adagrad(shards, slot0, g, touched, 0.01, lo_, hi_)
      got = sparse_dense_matmul_grad_with_adagrad.tpu_sparse_dense_matmul_grad_with_adagrad_primitive.bind(
          *st["flat"], np.int32(1), dev(shards), dev(slot0), grad, np.float32(0.01), **kw)
    else:
      hyp = lo.adam_hyperparameters(1e-3, 0.9, 0.999, 1e-8, 3)
      want = lo.apply_adam(shards, slot0, slot1, g, touched, *hyp, lo_, hi_)
      got = sparse_dense_matmul_grad_with_adam.tpu_sparse_dense_matmul_grad_with_adam_primitive.bind(
          *st["flat"], np.int32(1), dev(shards), dev(slot0), dev(slot1), grad, *hyp, **kw)
    for a, b in zip(got, want):
      assert_close(a.cpu().numpy(), b)
    # Untouched rows must be bit-identical to the inputs.
    untouched = ~touched
    np.testing.assert_array_equal(got[0].cpu().numpy().reshape(shards.shape)[untouched], shards[untouched])


_TWO_SLOT = [
    ("adagrad_momentum", (0.05, 0.9, 1.0, 1e-10, 2.0, False), {}),
    ("adagrad_momentum", (0.05, 0.8, 0.95, 1e-6, 3.0, True), {}),
    ("ftrl", (0.05, -0.5, 0.0, 0.0, 0.0), {"multiply_linear_by_learning_rate": False}),
    ("ftrl", (0.05, -0.5, 0.001, 0.01, 0.1), {"multiply_linear_by_learning_rate": True}),
    ("ftrl", (0.05, -0.4, 0.002, 0.0, 0.0), {"multiply_linear_by_learning_rate": False}),
    ("laprop", (0.01, 0.9, 0.73, 1e-30), {}),
    ("f2a", (0.05, 0.5, 0.001, 0.002, 1e6, 40.0), {}),
]


@pytest.mark.parametrize("clip", [None, (-0.012, 0.011)])
@pytest.mark.parametrize("which", range(len(_TWO_SLOT)))
@pytest.mark.parametrize("case", [c for c in CASES if c.name in ("dense_single_hot_zipf", "mean_unity_dups", "sqrtn_unity")],
                         ids=lambda c: c.name)
def test_two_slot_optimizers_match_oracle(case, which, clip):
  """AdagradMomentum, FTRL, LaProp and F2A epilogues of the fused update."""
  import importlib
  import torch

  name, hyper, flags = _TWO_SLOT[which]
  prim = getattr(importlib.import_module(
      f"jax_tpu_embedding.sparsecore.lib.core.primitives.sparse_dense_matmul_grad_with_{name}"),
      f"tpu_sparse_dense_matmul_grad_with_{name}_primitive")
  apply = getattr(lo, f"apply_{name}")
  rng = np.random.default_rng(17)
  for st in _setup(case).values():
    shards = st["shards"]
    g, touched = lo.table_gradient(st["csr"], st["grads"], shards.shape, num_sc_per_device=case.num_sc_per_device)
    lo_, hi_ = clip if clip else (None, None)
    slot0 = rng.uniform(0.05, 0.2, size=shards.shape).astype(np.float32)
    slot1 = rng.uniform(0.0, 3.0 if name == "f2a" else 1e-2, size=shards.shape).astype(np.float32)
    if name == "f2a":
      slot1 = np.floor(slot1)
    dev = lambda a: torch.from_numpy(a.reshape(-1, a.shape[-1]).copy()).cuda()
    grad = torch.from_numpy(np.concatenate(st["grads"])).cuda()
    want = apply(shards, slot0, slot1, g, touched, *hyper, *flags.values(), lo_, hi_)
    operands = [np.float32(h) if not isinstance(h, bool) else np.bool_(h) for h in hyper]
    got = prim.bind(*st["flat"], np.int32(1), dev(shards), dev(slot0), dev(slot1), grad, *operands,
                    **dict(_kw(case, st["spec"]), min_value=lo_, max_value=hi_, **flags))
    for a, b in zip(got, want):
      assert_close(a.cpu().numpy(), b)
    untouched = ~touched
    for a, b in zip(got, (shards, slot0, slot1)):
      np.testing.assert_array_equal(a.cpu().numpy().reshape(shards.shape)[untouched], b[untouched])


def test_backward_is_reproducible_and_hot_rows():
  """One row hit by thousands of entries: chunked partial sums stay deterministic and accurate."""
  import torch

  case = cases.make_case("hot", seed=11, tables=[dict(vocab=64, dim=128, features=[dict(kind="dense", valency=1, dist="zipf", a=2.0)])],
                         batch=8192, optimizer="adagrad")
  st = _setup(case)["table_0"]
  g, touched = lo.table_gradient(st["csr"], st["grads"], st["shards"].shape, num_sc_per_device=1)
  acc = np.full(st["shards"].shape, 0.1, np.float32)
  want = lo.apply_adagrad(st["shards"], acc, g, touched, 0.01)
  outs = []
  for _ in range(2):
    table = torch.from_numpy(st["shards"][0].copy()).cuda()
    accd = torch.from_numpy(acc[0].copy()).cuda()
    grad = torch.from_numpy(st["grads"][0]).cuda()
    outs.append(sparse_dense_matmul_grad_with_adagrad.tpu_sparse_dense_matmul_grad_with_adagrad_primitive.bind(
        *st["flat"], np.int32(1), table, accd, grad, np.float32(0.01), **_kw(case, st["spec"])))
  assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
  assert_close(outs[0][0].cpu().numpy(), want[0][0])
  assert_close(outs[0][1].cpu().numpy(), want[1][0])


@pytest.mark.parametrize("opt", ["sgd", "adagrad", "adam"])
@pytest.mark.parametrize("dim", [3, 6, 20, 30, 32, 48, 50, 64, 100, 130, 256, 384, 512, 1024])
def test_row_length_classes(dim, opt):
  """Every row-length variant of the kernels (odd dims included) with 0, 1 and 2 slot variables."""
  import torch

  case = cases.make_case("dims", seed=dim, batch=256, optimizer="adagrad", num_sc_per_device=2, tables=[
      dict(vocab=700, dim=8, features=[dict(kind="ragged", max_len=12, dist="zipf")])])
  st = _setup(case, dim_override=dim)["table_0"]
  shards = st["shards"]
  kw = _kw(case, st["spec"])
  want = np.concatenate(lo.forward(st["csr"], shards, num_sc_per_device=2, device_batch_size=st["bdev"]))
  dev = lambda a: torch.from_numpy(a.reshape(-1, a.shape[-1]).copy()).cuda()
  got = sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.bind(
      *st["flat"], np.int32(1), dev(shards), device_batch_size=st["bdev"], **kw)
  np.testing.assert_array_equal(got.cpu().numpy(), want)
  g, touched = lo.table_gradient(st["csr"], st["grads"], shards.shape, num_sc_per_device=2)
  acc = np.full(shards.shape, 0.1, np.float32)
  vel = np.full(shards.shape, 1e-4, np.float32)
  grad = torch.from_numpy(np.concatenate(st["grads"])).cuda()
  if opt == "sgd":
    want_all = lo.apply_sgd(shards, g, touched, 0.05)
    got_all = (sparse_dense_matmul_grad_with_sgd.tpu_sparse_dense_matmul_grad_with_sgd_primitive.bind(
        *st["flat"], np.int32(1), dev(shards), grad, np.float32(0.05), **kw),)
  elif opt == "adagrad":
    want_all = lo.apply_adagrad(shards, acc, g, touched, 0.05)
    got_all = sparse_dense_matmul_grad_with_adagrad.tpu_sparse_dense_matmul_grad_with_adagrad_primitive.bind(
        *st["flat"], np.int32(1), dev(shards), dev(acc), grad, np.float32(0.05), **kw)
  else:
    hyp = lo.adam_hyperparameters(1e-3, 0.9, 0.999, 1e-8, 2)
    want_all = lo.apply_adam(shards, acc, vel, g, touched, *hyp)
    got_all = sparse_dense_matmul_grad_with_adam.tpu_sparse_dense_matmul_grad_with_adam_primitive.bind(
        *st["flat"], np.int32(1), dev(shards), dev(acc), dev(vel), grad, *hyp, **kw)
  for a, b in zip(got_all, want_all):
    assert_close(a.cpu().numpy(), b)


def test_forward_long_bags():
  """Samples with hundreds of ids in one table take the long-row path of the forward plan."""
  import torch

  case = cases.make_case("long", seed=5, batch=64, num_sc_per_device=2, combiner="sum", tables=[
      dict(vocab=5000, dim=32, features=[dict(kind="ragged", min_len=0, max_len=600)])])
  st = _setup(case)["table_0"]
  assert max(len(np.unique(r)) for r in case.features[0]) > 300
  want = np.concatenate(lo.forward(st["csr"], st["shards"], num_sc_per_device=2, device_batch_size=st["bdev"]))
  table = torch.from_numpy(st["shards"].reshape(-1, st["shards"].shape[-1])).cuda()
  for _ in range(2):
    got = sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.bind(
        *st["flat"], np.int32(1), table, device_batch_size=st["bdev"], **_kw(case, st["spec"]))
    np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_hot_rows_over_several_sparsecores():
  """Rows hit by thousands of entries spread over four SparseCore slices: the entry list is ordered by the
  counting sort (long-row path included) and must equal the radix-sorted order bit for bit."""
  import os
  import subprocess
  import sys
  import torch

  case = cases.make_case("hot4", seed=12, num_sc_per_device=4, optimizer="adagrad", batch=8192, tables=[
      dict(vocab=64, dim=128, features=[dict(kind="dense", valency=1, dist="zipf", a=2.0)])])
  st = _setup(case)["table_0"]
  shards = st["shards"]
  g, touched = lo.table_gradient(st["csr"], st["grads"], shards.shape, num_sc_per_device=4)
  acc = np.full(shards.shape, 0.1, np.float32)
  want = lo.apply_adagrad(shards, acc, g, touched, 0.01)
  dev = lambda a: torch.from_numpy(a.reshape(-1, a.shape[-1]).copy()).cuda()
  outs = []
  for _ in range(2):
    outs.append(sparse_dense_matmul_grad_with_adagrad.tpu_sparse_dense_matmul_grad_with_adagrad_primitive.bind(
        *st["flat"], np.int32(1), dev(shards), dev(acc), torch.from_numpy(np.concatenate(st["grads"])).cuda(),
        np.float32(0.01), **_kw(case, st["spec"])))
  assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
  assert_close(outs[0][0].cpu().numpy(), want[0])
  assert_close(outs[0][1].cpu().numpy(), want[1])
  np.save("/tmp/sc_hot4_table.npy", outs[0][0].cpu().numpy())
  # The same update with the radix sort (chosen per process) in a child process.
  code = (
      "import sys, numpy as np, torch; sys.path[:0] = %r\n"
      "import cases, test_gpu_lookup as t\n"
      "from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_grad_with_adagrad as m\n"
      "case = cases.make_case('hot4', seed=12, num_sc_per_device=4, optimizer='adagrad', batch=8192, tables=["
      "dict(vocab=64, dim=128, features=[dict(kind='dense', valency=1, dist='zipf', a=2.0)])])\n"
      "st = t._setup(case)['table_0']; sh = st['shards']; acc = np.full(sh.shape, 0.1, np.float32)\n"
      "dev = lambda a: torch.from_numpy(a.reshape(-1, a.shape[-1]).copy()).cuda()\n"
      "out = m.tpu_sparse_dense_matmul_grad_with_adagrad_primitive.bind(*st['flat'], np.int32(1), dev(sh), dev(acc), "
      "torch.from_numpy(np.concatenate(st['grads'])).cuda(), np.float32(0.01), **t._kw(case, st['spec']))\n"
      "assert np.array_equal(out[0].cpu().numpy(), np.load('/tmp/sc_hot4_table.npy'))\n" % (sys.path,))
  run = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, SC_BWD_SORT="radix"), capture_output=True, text=True)
  assert run.returncode == 0, run.stderr[-2000:]


def test_rank1_table():
  """Tables of rank 1 (dim 1), as in the reference's dim-1 forward test."""
  import torch

  case = cases.make_case("r1", seed=3, tables=[dict(vocab=64, dim=8, features=[dict(kind="dense", valency=2)])], batch=32)
  st = _setup(case)["table_0"]
  table = (np.arange(st["shards"].shape[1], dtype=np.float32) + 1.0)
  want = lo.forward(st["csr"], table.reshape(1, -1), num_sc_per_device=1, device_batch_size=st["bdev"])[0]
  got = sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.bind(
      *st["flat"], np.int32(1), torch.from_numpy(table).cuda(), device_batch_size=st["bdev"], **_kw(case, st["spec"]))
  assert got.shape == (st["bdev"],)
  np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_operand_validation():
  import torch

  case = CASES[0]
  st = _setup(case)["table_0"]
  table = torch.from_numpy(st["shards"][0]).cuda()
  bind = sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.bind
  kw = dict(device_batch_size=st["bdev"], **_kw(case, st["spec"]))
  with pytest.raises(ValueError, match="lhs_gains must have type"):
    bind(st["flat"][0], st["flat"][1], st["flat"][2], st["flat"][3].double(), np.int32(1), table, **kw)
  with pytest.raises(ValueError, match="sharding_strategy must be MOD"):
    bind(*st["flat"], np.int32(1), table, sharding_strategy=2, **kw)
  with pytest.raises(ValueError, match="max_ids_per_partition must be positive"):
    bind(*st["flat"], np.int32(1), table, **dict(kw, max_ids_per_partition=0))
  with pytest.raises(ValueError, match="equal rank 1 shapes"):
    bind(st["flat"][0], st["flat"][1][:-8], st["flat"][2], st["flat"][3], np.int32(1), table, **kw)


@pytest.mark.parametrize("dims", [(128, 96), (16, 8), (96, 128), (64, 40)])
@pytest.mark.parametrize("opt", ["sgd", "adagrad", "adam"])
def test_mixed_dims_in_one_group(dims, opt):
  """Two tables of different dims in the same row-length class share ONE grouped launch; hot rows of
  both span several 32-entry chunks, so both use the partial-sum scratch at the same time."""
  import torch
  from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops

  prim = {"sgd": sparse_dense_matmul_grad_with_sgd.tpu_sparse_dense_matmul_grad_with_sgd_primitive,
          "adagrad": sparse_dense_matmul_grad_with_adagrad.tpu_sparse_dense_matmul_grad_with_adagrad_primitive,
          "adam": sparse_dense_matmul_grad_with_adam.tpu_sparse_dense_matmul_grad_with_adam_primitive}[opt]
  assert _ops.shape_class(dims[0]) == _ops.shape_class(dims[1])
  requests, wants, fwd_requests, fwd_wants = [], [], [], []
  for ti, dim in enumerate(dims):
    case = cases.make_case(f"mixed{ti}", seed=31 + ti, batch=4096, optimizer="adagrad", tables=[
        dict(vocab=40, dim=8, features=[dict(kind="dense", valency=1, dist="zipf", a=1.3)])], max_ids=4096, max_unique=4096)
    st = _setup(case, seed=ti, dim_override=dim)["table_0"]
    shards = st["shards"]
    g, touched = lo.table_gradient(st["csr"], st["grads"], shards.shape, num_sc_per_device=1)
    acc = np.full(shards.shape, 0.1, np.float32)
    vel = np.full(shards.shape, 1e-4, np.float32)
    dev = lambda a: torch.from_numpy(a.reshape(-1, a.shape[-1]).copy()).cuda()
    grad = torch.from_numpy(np.concatenate(st["grads"])).cuda()
    kw = _kw(case, st["spec"])
    fwd_requests.append(sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.prepare(
        *st["flat"], np.int32(1), dev(shards), device_batch_size=st["bdev"], **kw))
    fwd_wants.append(np.concatenate(lo.forward(st["csr"], shards, num_sc_per_device=1, device_batch_size=st["bdev"])))
    if opt == "sgd":
      wants.append(lo.apply_sgd(shards, g, touched, 0.05))
      requests.append(prim.prepare(*st["flat"], np.int32(1), dev(shards), grad, np.float32(0.05), **kw))
    elif opt == "adagrad":
      wants.append(lo.apply_adagrad(shards, acc, g, touched, 0.05))
      requests.append(prim.prepare(*st["flat"], np.int32(1), dev(shards), dev(acc), grad, np.float32(0.05), **kw))
    else:
      hyp = lo.adam_hyperparameters(1e-3, 0.9, 0.999, 1e-8, 2)
      wants.append(lo.apply_adam(shards, acc, vel, g, touched, *hyp))
      requests.append(prim.prepare(*st["flat"], np.int32(1), dev(shards), dev(acc), dev(vel), grad, *hyp, **kw))
  call = _ops.GradGroupCall(requests)
  assert len(call.groups) == 1, "both tables must travel in one grouped launch"
  for got_all, want_all in zip(call.run(), wants):
    for a, b in zip(got_all, want_all):
      assert_close(a.cpu().numpy(), b)
  for got, want in zip(_ops.run_forward_group(fwd_requests), fwd_wants):
    np.testing.assert_array_equal(got.cpu().numpy(), want)
