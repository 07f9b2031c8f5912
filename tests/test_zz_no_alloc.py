"""The allocation-free update entry point (`sc_sparse_dense_matmul_grad_static`).

Some callers of this library cannot call cudaMalloc: a server whose device memory was handed out
completely at start-up, a plugin running inside another runtime's callback, a loop that must not
block on the driver's allocator.  For them the library carries its scratch in a fixed array inside
its own image.  This test drives that entry point through the C ABI and checks it against the
ordinary entry point (caller-provided workspace) on identical inputs, twice in a row, because the
built-in scratch keeps whatever the previous call left in it.

The file name sorts last on purpose: it runs after every other test.
"""

import ctypes

import numpy as np
import pytest

import cases
import oracle_backend as ob
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


def test_static_scratch_update_matches_workspace_update_twice():
  rng = np.random.default_rng(0)
  # Two different problems back to back: the second call starts from the first call's scratch.
  for seed, batch, vocab, dim, kind, hyper in [(1, 8192, 3000, 128, 1, (0.01,)),
                                               (2, 4096, 50, 64, 2, (1e-3, 0.9, 0.999, 1e-8))]:
    csr_arrays, spec = _inputs(seed, batch, vocab, dim)
    rows = spec.stack_vocab_size
    table = rng.normal(0, 0.01, size=(rows, dim)).astype(np.float32)
    acc = rng.uniform(0.05, 0.2, size=(rows, dim)).astype(np.float32)
    mom = rng.uniform(0.0, 1e-4, size=(rows, dim)).astype(np.float32)
    grad = (rng.normal(size=(batch, dim)) * 1e-2).astype(np.float32)
    want = _run("workspace", csr_arrays, spec, table, acc, mom, grad, kind, hyper)
    for _ in range(2):
      got = _run("static", csr_arrays, spec, table, acc, mom, grad, kind, hyper)
      for g, w in zip(got, want):
        np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-6 * float(np.abs(w).max()) + 1e-12)
        # Same kernels and the same summation order: the results are in fact identical.
        np.testing.assert_array_equal(g, w)
    assert not np.array_equal(want[0], table), "the update must have changed the table"


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
