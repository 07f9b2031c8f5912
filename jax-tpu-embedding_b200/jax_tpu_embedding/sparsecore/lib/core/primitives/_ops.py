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
  """Named operator.  `prepare` validates operands and returns a request; `bind` runs it.

  Requests of several operators can be executed together with `run_forward_group` /
  `run_grad_group`, which is how the embedding API serves all stacked tables in one launch.
  """

  def __init__(self, name: str, prepare, runner, multiple_results: bool = False, unwrap=None):
    self.name = name
    self.prepare = prepare
    self._runner = runner
    self._unwrap = unwrap or (lambda r: r)
    self.multiple_results = multiple_results

  def bind(self, *operands, **attributes):
    return self._unwrap(self._runner([self.prepare(*operands, **attributes)])[0])

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
    if l != c:
      from jax_tpu_embedding.sparsecore import distributed  # pylint: disable=g-import-not-at-top

      if l != 1 or not distributed.is_active() or distributed.world_size() != c:
        raise ValueError(
            f"operands carry {l} of {c} devices: either pass the buffers of all devices (virtual devices on one "
            "GPU) or run one process per GPU with sparsecore.distributed.init()")
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


def shape_class(dim: int) -> tuple[int, int, int]:
  """(vector width, vectors per lane, lanes per row) the kernels use for a row of `dim` floats.

  Tables of one grouped call must agree on it; mirrors pick_group_shape in csrc/sc_lookup.cu.
  """
  w = 4 if dim % 4 == 0 else 1
  vecs = dim // w
  for limit, k, g in ((4, 1, 4), (8, 1, 8), (16, 2, 8), (32, 4, 8), (64, 4, 16), (128, 4, 32), (256, 8, 32)):
    if vecs <= limit:
      return w, k, g
  raise ValueError(f"embedding dimension {dim} is too large")


class ForwardRequest:
  """One stacked table of a grouped forward call (operands already validated)."""

  def __init__(self, rp, ids, sids, gains, table, *, device_batch_size, num_sc_per_device=None,
               global_device_count=None, local_device_count=None, max_ids_per_sample=0, forward_plan=None):
    torch = _native.require_cuda()
    self.rp, self.ids, self.sids, self.gains = _device_operands(rp, ids, sids, gains)
    self.table = _native.as_device(table, torch.float32, "embedding_table")
    self.geo = Geometry(self.rp, self.ids, self.table, device_batch_size, num_sc_per_device, global_device_count,
                        local_device_count)
    out_shape = (self.geo.batch, self.geo.dim) if self.table.dim() > 1 else (self.geo.batch,)
    self.act = torch.empty(out_shape, dtype=torch.float32, device=self.table.device)
    self.csr = self.geo.csr(self.rp, self.ids, self.sids, self.gains, max_ids_per_sample)
    self.ptrs = self.geo.shard_pointers(self.table)
    # (plan_slots, plan_bags) emitted by this package's preprocessing for exactly these buffers.
    self.plan = None
    if forward_plan is not None and self.geo.l == 1:
      slots, bags = forward_plan
      if (slots.dtype != torch.int32 or bags.dtype != torch.int32 or not slots.is_cuda or not bags.is_cuda
          or bags.numel() != 2 * self.geo.batch):
        raise ValueError("forward_plan does not belong to these buffers")
      self.plan = (slots, bags)
    self.local_shard = -1
    if self.geo.l != self.geo.c:  # one process per GPU: the other shards are peer mappings
      from jax_tpu_embedding.sparsecore import distributed  # pylint: disable=g-import-not-at-top

      self.local_shard = distributed.rank() * self.geo.s_eff


class _CsrFields:
  """The CSR (and forward plan) pointer fields of a descriptor array as strided numpy views, with their offsets from
  the two buffers of the preprocessing output the descriptors were built from: moving the descriptors to another
  output of the same layout is a handful of vector additions."""

  def __init__(self, items, item_type, count: int, bases, with_plan: bool):
    size = ctypes.sizeof(item_type)
    field = lambda offset: np.ndarray((count,), dtype=np.uint64, buffer=items, offset=offset, strides=(size,))
    c = item_type.csr.offset
    self.int_fields = [field(c + _native.Csr.row_pointers.offset), field(c + _native.Csr.embedding_ids.offset),
                       field(c + _native.Csr.sample_ids.offset)]
    if with_plan:
      self.int_fields += [field(item_type.plan_slots.offset), field(item_type.plan_bags.offset)]
    self.float_fields = [field(c + _native.Csr.gains.offset)]
    self.bases = (int(bases[0]), int(bases[1]))
    # A null pointer (a descriptor without a plan) stays null.
    self.int_rel = [(f != 0, f - np.uint64(self.bases[0])) for f in self.int_fields]
    self.float_rel = [(f != 0, f - np.uint64(self.bases[1])) for f in self.float_fields]

  def rebase(self, bases) -> None:
    ibase, fbase = int(bases[0]), int(bases[1])
    if (ibase, fbase) == self.bases:
      return
    for f, (used, rel) in zip(self.int_fields, self.int_rel):
      np.copyto(f, rel + np.uint64(ibase), where=used)
    for f, (used, rel) in zip(self.float_fields, self.float_rel):
      np.copyto(f, rel + np.uint64(fbase), where=used)
    self.bases = (ibase, fbase)


class ForwardGroupCall:
  """Validated requests turned into ready-to-launch descriptor arrays (one per shape class).

  Holds only addresses and sizes, so it can be replayed whenever the same buffers are passed
  again; outputs are allocated per run.
  """

  def __init__(self, requests, bases=None):
    lib = _native.lib()
    self.requests = requests
    self.groups = []
    self.csr_fields = []
    by_class: dict = {}
    for i, r in enumerate(requests):
      by_class.setdefault(shape_class(r.geo.dim), []).append(i)
    for idxs in by_class.values():
      items = (_native.FwdItem * len(idxs))()
      for j, i in enumerate(idxs):
        r = requests[i]
        items[j].csr = r.csr
        items[j].shard_tables = r.ptrs
        items[j].activations = r.act.data_ptr()
        items[j].local_shard = r.local_shard
        if r.plan is not None:
          items[j].plan_slots = r.plan[0].data_ptr()
          items[j].plan_bags = r.plan[1].data_ptr()
      nbytes = lib.sc_sparse_dense_matmul_fwd_grouped_workspace_bytes(items, len(idxs))
      if nbytes == 0:
        _native.check(lib.sc_sparse_dense_matmul_fwd_grouped(items, len(idxs), None, 0, None))
      # The activation pointers of the group's descriptors as one strided numpy view (filled per run).
      act_field = np.ndarray((len(idxs),), dtype=np.uint64, buffer=items, offset=_native.FwdItem.activations.offset,
                             strides=(ctypes.sizeof(_native.FwdItem),))
      self.groups.append((items, idxs, nbytes, act_field))
      if bases is not None:
        self.csr_fields.append(_CsrFields(items, _native.FwdItem, len(idxs), bases, with_plan=True))
    self.shapes = [tuple(r.act.shape) for r in requests]
    self.sizes = [int(np.prod(shape)) for shape in self.shapes]
    self.total_floats = sum(self.sizes)
    dims = {shape[-1] for shape in self.shapes if len(shape) == 2}
    self.common_dim = dims.pop() if len(dims) == 1 and all(len(shape) == 2 for shape in self.shapes) else 0
    self.rows = [shape[0] for shape in self.shapes]
    self.byte_offsets = np.concatenate([[0], np.cumsum(self.sizes)[:-1]]).astype(np.uint64) * np.uint64(4)
    self.first = True
    self.sharded = any(r.geo.l != r.geo.c for r in requests)
    self.keep = [(r.ptrs,) for r in requests]
    # Requests keep tensors alive; a replayable call must not, so drop them after the first run.

  def rebase(self, bases) -> None:
    """Points the descriptors at another preprocessing output of the same layout (its two buffer addresses)."""
    for fields in self.csr_fields:
      fields.rebase(bases)

  def run(self):
    torch = _native.torch_mod()
    lib = _native.lib()
    if self.first:
      outs = [r.act for r in self.requests]
      self.first = False
      self.requests = None
    else:
      # One allocation for all activations of the call.
      if self.common_dim:
        # All activations are [rows, dim] with one dim: the pieces of a 2-D buffer need no reshaping.
        flat = torch.empty((self.total_floats // self.common_dim, self.common_dim), dtype=torch.float32, device="cuda")
        outs = list(torch.split_with_sizes(flat, self.rows))
      else:
        flat = torch.empty(self.total_floats, dtype=torch.float32, device="cuda")
        outs = [t.view(shape) for t, shape in zip(torch.split_with_sizes(flat, self.sizes), self.shapes)]
      addresses = self.byte_offsets + np.uint64(flat.data_ptr())
      for _, idxs, _, act_field in self.groups:
        act_field[:] = addresses[idxs]
    stream = _native.current_stream_ptr()
    if self.sharded:
      # Every peer must have finished updating its shard before remote rows are read.
      from jax_tpu_embedding.sparsecore import distributed  # pylint: disable=g-import-not-at-top

      distributed.barrier_before_lookup()
    for items, idxs, nbytes, _ in self.groups:
      ws = _native.workspace(nbytes, "lookup")
      _native.check(lib.sc_sparse_dense_matmul_fwd_grouped(items, len(idxs), ws.data_ptr(), ws.numel(), stream))
    return outs


def run_forward_group(requests):
  """Runs every request; requests whose rows fall in one shape class share a grouped launch."""
  return ForwardGroupCall(requests).run()


def run_forward(rp, ids, sids, gains, table, **kw):
  return run_forward_group([ForwardRequest(rp, ids, sids, gains, table, **kw)])[0]


_OPT_KIND = {"sgd": 0, "adagrad": 1, "adam": 2, "adagrad_momentum": 3, "ftrl": 4, "laprop": 5, "f2a": 6}


class GradRequest:
  """One stacked table of a grouped backward call."""

  def __init__(self, kind, rp, ids, sids, gains, table, slots, act_grad, hyper, *, min_value=None, max_value=None,
               num_sc_per_device=None, global_device_count=None, local_device_count=None, partition_capacity=None,
               exchange_key=None):
    torch = _native.require_cuda()
    self.rp, self.ids, self.sids, self.gains = _device_operands(rp, ids, sids, gains)
    self.table = _native.as_device(table, torch.float32, "embedding_table")
    self.slots = [_native.as_device(s, torch.float32, "slot variable") for s in slots]
    self.act_grad = _native.as_device(act_grad, torch.float32, "activations_grad")
    l = int(local_device_count) if local_device_count else 1
    self.geo = Geometry(self.rp, self.ids, self.table, self.act_grad.shape[0] // l, num_sc_per_device,
                        global_device_count, local_device_count)
    if self.act_grad.shape[0] != self.geo.batch:
      raise ValueError(f"activations_grad has {self.act_grad.shape[0]} rows, expected {self.geo.batch}")
    self.csr = self.geo.csr(self.rp, self.ids, self.sids, self.gains)
    opt = _native.Optimizer()
    opt.optimizer = _OPT_KIND[kind]
    for i in range(8):
      opt.hyper[i] = float(hyper[i]) if i < len(hyper) else 0.0
    opt.clip_min = float("nan") if min_value is None else float(min_value)
    opt.clip_max = float("nan") if max_value is None else float(max_value)
    self.opt = opt
    self.pull = None
    if self.geo.l != self.geo.c:
      # Row-sharded table, one process per GPU: this process owns one shard and pulls the entries
      # every process holds for it (see sparsecore.distributed).
      from jax_tpu_embedding.sparsecore import distributed  # pylint: disable=g-import-not-at-top

      if self.geo.s != 1:
        raise ValueError("row-sharded tables with one process per GPU need num_sc_per_device == 1")
      self.pull = distributed.exchange_buffers(exchange_key or "default", self.rp.numel(), self.geo.coo,
                                               self.geo.batch, self.geo.dim)
      cap = self.geo.coo if not partition_capacity else min(self.geo.coo, (int(partition_capacity) + 7) // 8 * 8)
      self.partition_capacity = cap
      self.shard = distributed.rank()
      self.t_ptrs = (_native.c_vp * 1)(self.table.data_ptr())
      self.s_ptrs = [(_native.c_vp * 1)(s.data_ptr()) for s in self.slots]
    else:
      self.t_ptrs = self.geo.shard_pointers(self.table)
      self.s_ptrs = [self.geo.shard_pointers(s) for s in self.slots]

  def results(self):
    return (self.table, *self.slots)


class GradGroupCall:
  """Ready-to-launch descriptors of a grouped backward call (addresses and sizes only)."""

  def __init__(self, requests, bases=None):
    lib = _native.lib()
    self.requests = requests
    self.groups = []
    self.csr_fields = []
    self.grad_fields = []
    by_class: dict = {}
    for i, r in enumerate(requests):
      by_class.setdefault((shape_class(r.geo.dim), r.opt.optimizer), []).append(i)
    for idxs in by_class.values():
      items = (_native.GradItem * len(idxs))()
      for j, i in enumerate(idxs):
        r = requests[i]
        items[j].csr = r.csr
        items[j].activation_grad = r.act_grad.data_ptr()
        items[j].shard_tables = r.t_ptrs
        if len(r.s_ptrs) > 0:
          items[j].shard_slot0 = r.s_ptrs[0]
        if len(r.s_ptrs) > 1:
          items[j].shard_slot1 = r.s_ptrs[1]
        items[j].optimizer = r.opt
        if r.pull is not None:
          items[j].sources = r.pull["sources"]
          items[j].num_sources = r.geo.c
          items[j].shard = r.shard
          items[j].partition_capacity = r.partition_capacity
      nbytes = lib.sc_sparse_dense_matmul_grad_grouped_workspace_bytes(items, len(idxs))
      if nbytes == 0:
        _native.check(lib.sc_sparse_dense_matmul_grad_grouped(items, len(idxs), None, 0, None))
      if any(requests[i].pull is not None for i in idxs):
        stage_bytes = lib.sc_sparse_dense_matmul_grad_stage_workspace_bytes(items, len(idxs))
        if stage_bytes == 0:
          _native.check(lib.sc_sparse_dense_matmul_grad_stage(items, len(idxs), None, 0, None))
        nbytes = max(nbytes, stage_bytes)
      self.groups.append((items, idxs, nbytes))
      # The gradient pointers of the group's descriptors as one strided numpy view (see set_gradients).
      self.grad_fields.append(np.ndarray((len(idxs),), dtype=np.uint64, buffer=items,
                                         offset=_native.GradItem.activation_grad.offset,
                                         strides=(ctypes.sizeof(_native.GradItem),)))
      if bases is not None:
        self.csr_fields.append(_CsrFields(items, _native.GradItem, len(idxs), bases, with_plan=False))
    self.keep = [(r.t_ptrs, r.s_ptrs, r.pull) for r in requests]
    self.sharded = any(r.pull is not None for r in requests)
    # Two row-sharded requests of one call must not stage into the same peer buffers (equal `exchange_key` and
    # geometry): the second staging would overwrite the first before the update reads it.
    staged = [id(r.pull) for r in requests if r.pull is not None]
    if len(set(staged)) != len(staged):
      raise ValueError("two requests of one grouped update share their exchange buffers: give each stacked table "
                       "its own computation_name / exchange_key")
    self._results = [r.results() for r in requests]
    self.first = True

  def rebase(self, bases) -> None:
    """Points the descriptors at another preprocessing output of the same layout (its two buffer addresses)."""
    for fields in self.csr_fields:
      fields.rebase(bases)

  def set_gradients(self, addresses) -> None:
    """Points the descriptors at the activation gradients of this call (device addresses in request order; the
    tensors have the shapes and dtype of those the descriptors were built from)."""
    addresses = np.asarray(addresses, dtype=np.uint64)
    for (_, idxs, _), field in zip(self.groups, self.grad_fields):
      field[:] = addresses[idxs]

  def run(self):
    lib = _native.lib()
    stream = _native.current_stream_ptr()
    if self.sharded:
      from jax_tpu_embedding.sparsecore import distributed  # pylint: disable=g-import-not-at-top

      distributed.barrier_before_staging()  # peers are done reading the exchange buffers of the previous call
      for items, idxs, nbytes in self.groups:
        ws = _native.workspace(nbytes, "lookup")
        _native.check(lib.sc_sparse_dense_matmul_grad_stage(items, len(idxs), ws.data_ptr(), ws.numel(), stream))
      distributed.stream_barrier("BarrierAfterStaging")  # every peer's exchange buffers are complete
    for items, idxs, nbytes in self.groups:
      ws = _native.workspace(nbytes, "lookup")
      _native.check(lib.sc_sparse_dense_matmul_grad_grouped(items, len(idxs), ws.data_ptr(), ws.numel(), stream))
    if self.sharded:
      distributed.note_update_launched()
    if self.first:
      self.first = False
      self.requests = None
      res, self._results = self._results, None
      return res
    return None


def run_grad_group(requests):
  return GradGroupCall(requests).run()


def run_grad(kind, rp, ids, sids, gains, table, slots, act_grad, hyper, **kw):
  """Fused gradient + optimizer update; returns (table, *slots), updated in place."""
  return run_grad_group([GradRequest(kind, rp, ids, sids, gains, table, slots, act_grad, hyper, **kw)])[0]


def scalar_f32(x) -> float:
  """Hyper-parameter operand (python float, numpy or torch scalar) -> python float of its f32 value."""
  if hasattr(x, "item"):
    x = x.item()
  return float(np.float32(x))


def is_finite_or_none(x) -> bool:
  return x is None or not math.isnan(float(x))
