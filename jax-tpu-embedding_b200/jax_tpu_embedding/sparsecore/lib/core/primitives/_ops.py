"""Launch glue between the operator objects and the C ABI of libsc_b200.so.

An operator mirrors a `jax.extend.core.Primitive` of the reference: `bind(*operands,
**attributes)` validates exactly like the reference's abstract evaluation and then runs
the CUDA kernels on the current stream.  Three keyword attributes exist only here,
because the reference gets them from the TPU topology instead of from operands:

  num_sc_per_device    table shards per device (default: 1 on B200),
  global_device_count  devices that share the stacked table (default: the size of the
                       torch.distributed world, or 1),
  local_device_count   devices whose buffers are concatenated in the operands
                       (default 1).  With local == global the call computes every
                       device's slice on this GPU ("virtual devices"), which is how
                       multi-device layouts are replayed on one GPU.

Tables and slot variables are updated IN PLACE by the gradient operators and returned.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np

from jax_tpu_embedding.sparsecore import _native
from jax_tpu_embedding.sparsecore.utils import utils as sc_utils


class Primitive:
  """Named operator with a `bind` entry point."""

  def __init__(self, name: str, impl, multiple_results: bool = False):
    self.name = name
    self._impl = impl
    self.multiple_results = multiple_results

  def bind(self, *operands, **attributes):
    return self._impl(*operands, **attributes)

  def __repr__(self):
    return self.name


def _world_size() -> int:
  torch = _native.torch_mod()
  if torch.distributed.is_available() and torch.distributed.is_initialized():
    return torch.distributed.get_world_size()
  return 1


class Geometry:
  """Sizes derived from operand shapes plus the three topology attributes."""

  def __init__(self, row_pointers, embedding_ids, table, device_batch_size, num_sc_per_device, global_device_count,
               local_device_count):
    s = int(num_sc_per_device) if num_sc_per_device else sc_utils.num_sparsecores_per_device()
    c = int(global_device_count) if global_device_count else _world_size()
    l = int(local_device_count) if local_device_count else 1
    if s <= 0 or c <= 0 or l <= 0 or l > c:
      raise ValueError(f"invalid topology: num_sc_per_device={s}, global_device_count={c}, local_device_count={l}")
    p = s * c
    if p & (p - 1):
      raise ValueError(f"Total number of SparseCores ({p}) must be a power of 2.")
    r = max(p, 8)
    if row_pointers.shape[0] != l * s * r:
      raise ValueError(
          f"lhs_row_pointers has {row_pointers.shape[0]} entries, expected {l * s * r} "
          f"(local devices {l} x SparseCores {s} x {r})")
    coo = embedding_ids.shape[0]
    if coo == 0 or coo % (l * s):
      raise ValueError(f"COO buffer size {coo} must be a positive multiple of {l * s}")
    rows = table.shape[0]
    if rows % (l * s):
      raise ValueError(f"embedding_table has {rows} rows, not divisible by {l * s} local shards")
    self.s, self.c, self.l, self.p = s, c, l, p
    self.s_eff = l * s
    self.coo = coo
    self.rows_per_shard = rows // (l * s)
    self.dim = table.shape[1] if table.dim() > 1 else 1
    self.batch = int(device_batch_size) * l
    if device_batch_size <= 0 or device_batch_size % s:
      raise ValueError(f"device_batch_size ({device_batch_size}) must be a positive multiple of num_sc_per_device ({s})")

  def csr(self, rp, ids, sids, gains, max_ids_per_sample=0) -> _native.Csr:
    return _native.Csr(rp.data_ptr(), ids.data_ptr(), sids.data_ptr(), gains.data_ptr(), self.coo, self.s_eff, self.p,
                       self.batch, self.dim, int(max_ids_per_sample), self.rows_per_shard)

  def shard_pointers(self, tensor):
    """Device pointers of all P shards of `tensor` ([local shards * rows_per_shard, dim])."""
    if self.l != self.c:
      from jax_tpu_embedding.sparsecore import distributed  # pylint: disable=g-import-not-at-top

      return distributed.shard_pointers(tensor, self)
    stride = self.rows_per_shard * self.dim * 4
    arr = (_native.c_vp * self.p)()
    base = tensor.data_ptr()
    for g in range(self.p):
      arr[g] = base + g * stride
    return arr


def _device_operands(rp, ids, sids, gains):
  torch = _native.require_cuda()
  return (_native.as_device(rp, torch.int32, "lhs_row_pointers"),
          _native.as_device(ids, torch.int32, "lhs_local_embedding_ids"),
          _native.as_device(sids, torch.int32, "lhs_local_sample_ids"),
          _native.as_device(gains, torch.float32, "lhs_gains"))


def run_forward(rp, ids, sids, gains, table, *, device_batch_size, num_sc_per_device=None, global_device_count=None,
                local_device_count=None, max_ids_per_sample=0):
  torch = _native.require_cuda()
  lib = _native.lib()
  rp, ids, sids, gains = _device_operands(rp, ids, sids, gains)
  table = _native.as_device(table, torch.float32, "embedding_table")
  geo = Geometry(rp, ids, table, device_batch_size, num_sc_per_device, global_device_count, local_device_count)
  csr = geo.csr(rp, ids, sids, gains, max_ids_per_sample)
  out_shape = (geo.batch, geo.dim) if table.dim() > 1 else (geo.batch,)
  act = torch.empty(out_shape, dtype=torch.float32, device=table.device)
  nbytes = lib.sc_sparse_dense_matmul_fwd_workspace_bytes(ctypes.byref(csr))
  ws = _native.workspace(nbytes, "lookup")
  ptrs = geo.shard_pointers(table)
  _native.check(lib.sc_sparse_dense_matmul_fwd(ctypes.byref(csr), ptrs, act.data_ptr(), ws.data_ptr(), ws.numel(),
                                               _native.current_stream_ptr()))
  return act


_OPT_KIND = {"sgd": 0, "adagrad": 1, "adam": 2}


def run_grad(kind, rp, ids, sids, gains, table, slots, act_grad, hyper, *, min_value=None, max_value=None,
             num_sc_per_device=None, global_device_count=None, local_device_count=None):
  """Fused gradient + optimizer update; returns (table, *slots), updated in place."""
  torch = _native.require_cuda()
  lib = _native.lib()
  rp, ids, sids, gains = _device_operands(rp, ids, sids, gains)
  table = _native.as_device(table, torch.float32, "embedding_table")
  slots = [_native.as_device(s, torch.float32, "slot variable") for s in slots]
  act_grad = _native.as_device(act_grad, torch.float32, "activations_grad")
  batch = act_grad.shape[0]
  geo_l = int(local_device_count) if local_device_count else 1
  geo = Geometry(rp, ids, table, batch // geo_l, num_sc_per_device, global_device_count, local_device_count)
  csr = geo.csr(rp, ids, sids, gains)
  opt = _native.Optimizer()
  opt.optimizer = _OPT_KIND[kind]
  for i in range(4):
    opt.hyper[i] = float(hyper[i]) if i < len(hyper) else 0.0
  opt.clip_min = float("nan") if min_value is None else float(min_value)
  opt.clip_max = float("nan") if max_value is None else float(max_value)
  nbytes = lib.sc_sparse_dense_matmul_grad_workspace_bytes(ctypes.byref(csr))
  ws = _native.workspace(nbytes, "lookup")
  t_ptrs = geo.shard_pointers(table)
  s_ptrs = [geo.shard_pointers(s) for s in slots] + [None, None]
  _native.check(lib.sc_sparse_dense_matmul_grad(ctypes.byref(csr), act_grad.data_ptr(), t_ptrs, s_ptrs[0], s_ptrs[1],
                                                ctypes.byref(opt), ws.data_ptr(), ws.numel(),
                                                _native.current_stream_ptr()))
  return (table, *slots)


def scalar_f32(x) -> float:
  """Hyper-parameter operand (python float, numpy or torch scalar) -> python float of its f32 value."""
  if hasattr(x, "item"):
    x = x.item()
  return float(np.float32(x))


def is_finite_or_none(x) -> bool:
  return x is None or not math.isnan(float(x))
