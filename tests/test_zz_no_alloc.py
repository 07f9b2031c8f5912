"""The allocation-free update entry point (`sc_sparse_dense_matmul_grad_static`).

Some callers of this library cannot call cudaMalloc: a server whose device memory was handed out
completely at start-up, a plugin running inside another runtime's callback, a loop that must not
block on the driver's allocator.  For them the library carries its scratch in a fixed array inside
its own image.  This test drives that entry point through the C ABI and checks it against the
ordinary entry point (caller-provided workspace) and against the numpy oracle on identical inputs,
twice in a row, because the built-in scratch keeps whatever the previous call left in it.

The file name sorts last on purpose: it runs after every other test.
"""

import ctypes

import numpy as np
import pytest

import cases
import oracle_backend as ob
from oracle import lookup_oracle as lo
from jax_tpu_embedding.sparsecore import _native

pytestmark = pytest.mark.gpu


def _inputs(seed, batch, vocab, dim, a=1.2):
  """Single-hot Zipf batch (hot rows span several 32-entry chunks) preprocessed by the oracle."""
  case = cases.make_case("static", seed=seed, tables=[dict(vocab=vocab, dim=dim, features=[dict(kind="dense", valency=1, dist="zipf", a=a)])],
                         batch=batch, optimizer="adagrad", max_ids=batch, max_unique=batch)
  out = ob.oracle_preprocess(case.features, None, case.feature_specs, 1, 1, num_sc_per_device=1)
  spec = case.feature_specs[0].table_spec.stacked_table_spec
  return [out[i]["table_0"] for i in range(4)], spec


def _run(entry, csr_arrays, spec, table, acc, mom, grad, kind, hyper):
  """Calls either entry point on device copies and returns the updated arrays."""
  import torch

  lib = _native.lib()
  rp, ids, sids, gains = [torch.from_numpy(a).cuda() for a in csr_arrays]
  t, a, m, g = (torch.from_numpy(x.copy()).cuda() for x in (table, acc, mom, grad))
  csr = _native.Csr(rp.data_ptr(), ids.data_ptr(), sids.data_ptr(), gains.data_ptr(), ids.numel(), 1, 1,
                    grad.shape[0], table.shape[1], 0, table.shape[0])
  opt = _native.Optimizer()
  opt.optimizer = kind
  for i, h in enumerate(hyper):
    opt.hyper[i] = h
  opt.clip_min = opt.clip_max = float("nan")
  ptr = lambda x: (_native.c_vp * 1)(x.data_ptr())
  stream = _native.current_stream_ptr()
  if entry == "static":
    status = lib.sc_sparse_dense_matmul_grad_static(ctypes.byref(csr), g.data_ptr(), ptr(t), ptr(a), ptr(m),
                                                    ctypes.byref(opt), stream)
  else:
    nbytes = lib.sc_sparse_dense_matmul_grad_workspace_bytes(ctypes.byref(csr))
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    status = lib.sc_sparse_dense_matmul_grad(ctypes.byref(csr), g.data_ptr(), ptr(t), ptr(a), ptr(m),
                                             ctypes.byref(opt), ws.data_ptr(), nbytes, stream)
  _native.check(status)
  torch.cuda.synchronize()
  return t.cpu().numpy(), a.cpu().numpy(), m.cpu().numpy()


def _oracle(csr_arrays, table, acc, mom, grad, kind, hyper):
  """The same update by the numpy oracle (one shard, one SparseCore)."""
  g, touched = lo.table_gradient([tuple(csr_arrays)], [grad], (1,) + table.shape, num_sc_per_device=1)
  if kind == 0:
    return [x[0] for x in lo.apply_sgd(table[None], g, touched, *hyper)] + [acc, mom]
  if kind == 1:
    return [x[0] for x in lo.apply_adagrad(table[None], acc[None], g, touched, *hyper)] + [mom]
  return [x[0] for x in lo.apply_adam(table[None], acc[None], mom[None], g, touched, *hyper)]


# (seed, batch, vocab, dim, optimizer kind, hyper-parameters).  Dim 6 takes the kernel for rows that are
# not whole 16-byte vectors; the last problem fills the built-in scratch to the documented limit
# (65536 slots at dim 128).
_PROBLEMS = [(1, 8192, 3000, 128, 1, (0.01,)),
             (2, 4096, 50, 64, 2, (1e-3, 0.9, 0.999, 1e-8)),
             (3, 2048, 500, 6, 0, (0.05,)),
             (4, 65536, 100000, 128, 1, (0.01,))]


def test_static_scratch_update_matches_workspace_update_twice():
  rng = np.random.default_rng(0)
  # Different problems back to back: every call starts from the previous call's scratch.
  for seed, batch, vocab, dim, kind, hyper in _PROBLEMS:
    csr_arrays, spec = _inputs(seed, batch, vocab, dim)
    rows = spec.stack_vocab_size
    table = rng.normal(0, 0.01, size=(rows, dim)).astype(np.float32)
    acc = rng.uniform(0.05, 0.2, size=(rows, dim)).astype(np.float32)
    mom = rng.uniform(0.0, 1e-4, size=(rows, dim)).astype(np.float32)
    grad = (rng.normal(size=(batch, dim)) * 1e-2).astype(np.float32)
    want = _run("workspace", csr_arrays, spec, table, acc, mom, grad, kind, hyper)
    oracle = _oracle(csr_arrays, table, acc, mom, grad, kind, hyper)
    for _ in range(2):
      got = _run("static", csr_arrays, spec, table, acc, mom, grad, kind, hyper)
      for g, w, o in zip(got, want, oracle):
        # The hottest rows of the largest problem sum ~10^4 gradient rows; the kernels add them in
        # 32-entry chunks, the oracle one after the other, hence the absolute floor.
        np.testing.assert_allclose(g, o, rtol=1e-5, atol=4e-6 * float(np.abs(o).max()) + 1e-12)
        # Same kernels and the same summation order as the workspace entry point: identical results.
        np.testing.assert_array_equal(g, w)
    assert not np.array_equal(want[0], table), "the update must have changed the table"


def test_static_scratch_limit_is_the_documented_one():
  """768 + chunks * (8 dim + 1) + ceil(chunks / 32) * (4 dim + 1) bytes, chunks = ceil(slots / 32)."""
  import torch

  lib = _native.lib()
  scratch = 2 * 1024 * 1024 + 64 * 1024
  ceil_div = lambda a, b: (a + b - 1) // b
  need = lambda slots, dim: (768 + ceil_div(slots, 32) * (8 * dim + 1) + ceil_div(ceil_div(slots, 32), 32) * (4 * dim + 1))
  dim = 128
  slots = 65536
  while need(slots + 32, dim) <= scratch:
    slots += 32
  assert need(slots, dim) <= scratch < need(slots + 32, dim)
  # A buffer of exactly `slots` slots whose row pointer says "no entries": accepted; one chunk more: rejected.
  rp = torch.zeros(8, dtype=torch.int32, device="cuda")
  ints = torch.full((slots + 32,), 2**31 - 1, dtype=torch.int32, device="cuda")
  gains = torch.full((slots + 32,), float("nan"), dtype=torch.float32, device="cuda")
  table = torch.zeros((16, dim), device="cuda")
  grad = torch.zeros((8, dim), device="cuda")
  opt = _native.Optimizer()
  opt.optimizer = 0
  opt.hyper[0] = 0.1
  opt.clip_min = opt.clip_max = float("nan")
  ptr = (_native.c_vp * 1)(table.data_ptr())
  for n, status in ((slots, _native.SC_OK), (slots + 32, _native.SC_WORKSPACE_TOO_SMALL)):
    csr = _native.Csr(rp.data_ptr(), ints.data_ptr(), ints.data_ptr(), gains.data_ptr(), n, 1, 1, 8, dim, 0, 16)
    assert lib.sc_sparse_dense_matmul_grad_static(ctypes.byref(csr), grad.data_ptr(), ptr, None, None,
                                                  ctypes.byref(opt), _native.current_stream_ptr()) == status
  torch.cuda.synchronize()
  assert float(table.abs().sum()) == 0.0


def test_static_scratch_rejects_oversized_and_sharded_inputs():
  import torch

  lib = _native.lib()
  dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
  f = torch.zeros(8, dtype=torch.float32, device="cuda")
  opt = _native.Optimizer()
  opt.clip_min = opt.clip_max = float("nan")
  ptr = (_native.c_vp * 1)(f.data_ptr())
  big = _native.Csr(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), f.data_ptr(), 1 << 20, 1, 1, 1024, 128, 0, 1 << 20)
  assert lib.sc_sparse_dense_matmul_grad_static(ctypes.byref(big), f.data_ptr(), ptr, None, None, ctypes.byref(opt),
                                                None) == _native.SC_WORKSPACE_TOO_SMALL
  assert "built-in scratch" in _native.last_error()
  sharded = _native.Csr(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), f.data_ptr(), 1024, 2, 2, 1024, 128, 0, 64)
  assert lib.sc_sparse_dense_matmul_grad_static(ctypes.byref(sharded), f.data_ptr(), ptr, None, None,
                                                ctypes.byref(opt), None) == _native.SC_UNSUPPORTED
