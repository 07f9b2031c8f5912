"""Input preprocessing front end: same module name and call signatures as the
reference's pybind11 extension, executed by CUDA kernels on the current device.

Replaces jax_tpu_embedding/sparsecore/lib/core/pybind_input_preprocessing.cc
(`preprocess_sparse_dense_matmul_input` :190-216 / :124-188,
`compute_row_pointers_size_per_device` :218-229,
`compute_theoretical_max_coo_buffer_size` :315, `compute_coo_buffer_size_per_device`
:231-253, `SparseDenseMatmulInputStats` :320-330).  The host side only flattens the
numpy inputs into one CSR per stacked table and local device; sorting, deduplication,
id dropping, statistics and buffer filling run in `sc_preprocess_table`.

Differences from the reference, all deliberate:
  * exceeding `max_ids_per_partition` without `allow_id_dropping` raises ValueError
    instead of aborting the process;
  * slots past the last row pointer of a SparseCore slice hold padding
    (PADDING_VALUE / NaN) instead of uninitialised memory;
  * `device_output=True` keeps the four buffers on the GPU as torch tensors.
Minibatching (and its `all_reduce_interface`) only exists to fit TPU on-chip memory
and is rejected.
"""

from __future__ import annotations

import ctypes
import dataclasses
import enum
import operator
from typing import Any, Sequence

import numpy as np

from jax_tpu_embedding.sparsecore import _native


class ShardingStrategy(enum.IntEnum):
  MOD = 1


MOD = ShardingStrategy.MOD


class AllReduceInterface:  # placeholder type for signature compatibility
  pass


@dataclasses.dataclass
class RaggedInput:
  """A ragged feature already in CSR form (values + row_splits), host or device memory.

  Leaf type accepted wherever a feature array is expected; `weights` is optional.
  Device tensors (torch, CUDA) are used in place without a host round trip.
  """

  values: Any  # int32 [nnz]
  row_splits: Any  # int32/int64 [rows + 1]
  weights: Any = None  # float32 [nnz]

  @property
  def shape(self):
    return (len(self.row_splits) - 1,)


class SparseDenseMatmulInputStats:
  """Per stacked table: ids / unique ids per partition, required buffer sizes, drops."""

  def __init__(self):
    self.max_ids_per_partition: dict[str, np.ndarray] = {}
    self.max_unique_ids_per_partition: dict[str, np.ndarray] = {}
    self.required_buffer_sizes: dict[str, np.ndarray] = {}
    self.dropped_id_count: dict[str, int] = {}


def compute_row_pointers_size_per_device(global_device_count: int, num_sc_per_device: int,
                                         enable_minibatching: bool = False) -> int:
  _reject_minibatching(enable_minibatching)
  return int(_native.lib().sc_compute_row_pointers_size_per_device(global_device_count, num_sc_per_device))


def compute_theoretical_max_coo_buffer_size(max_ids_per_partition: int, global_device_count: int,
                                            num_sc_per_device: int, enable_minibatching: bool = False) -> int:
  _reject_minibatching(enable_minibatching)
  return int(_native.lib().sc_compute_theoretical_max_coo_buffer_size(
      max_ids_per_partition, global_device_count, num_sc_per_device))


def _coo_buffer_size(max_ids: int, global_device_count: int, num_sc_per_device: int, suggested) -> int:
  v = _native.lib().sc_compute_coo_buffer_size_per_device(
      int(max_ids), int(global_device_count), int(num_sc_per_device), -1 if suggested is None else int(suggested))
  if v < 0:
    raise ValueError(_native.last_error())
  return int(v)


def compute_coo_buffer_size_per_device(feature_specs: Sequence[Any], global_device_count: int,
                                       num_sc_per_device: int, enable_minibatching: bool = False) -> dict[str, int]:
  _reject_minibatching(enable_minibatching)
  out = {}
  for name, members in _group_by_stack(feature_specs).items():
    stacked = members[0][1].table_spec.stacked_table_spec
    out[name] = _coo_buffer_size(stacked.max_ids_per_partition, global_device_count, num_sc_per_device,
                                 stacked.suggested_coo_buffer_size_per_device)
  return out


def _reject_minibatching(enable_minibatching: bool) -> None:
  if enable_minibatching:
    raise NotImplementedError(
        "enable_minibatching=True is not supported: minibatching splits a batch to fit TPU SparseCore "
        "on-chip memory, a limit that does not exist on B200.")


def _group_by_stack(feature_specs):
  """{stack name: [(feature index, spec), ...] ordered by row_offset} (pybind...cc:55-122)."""
  stacks: dict[str, list] = {}
  for i, spec in enumerate(feature_specs):
    name = spec.table_spec.setting_in_stack.stack_name
    stacks.setdefault(name, []).append((i, spec))
  for members in stacks.values():
    members.sort(key=lambda m: _transform(m[1])[0])
  return stacks


def _transform(spec):
  t = spec._id_transformation  # pylint: disable=protected-access
  return (0, 0, 0) if t is None else (int(t.row_offset), int(t.col_offset), int(t.col_shift))


# ------------------------------------------------------------------------------ host flattening


def _is_torch(x) -> bool:
  return type(x).__module__.startswith("torch")


def _feature_rows(feature) -> int:
  if isinstance(feature, RaggedInput):
    return len(feature.row_splits) - 1
  return feature.shape[0]


def _to_cuda(x, tdt):
  torch = _native.torch_mod()
  if _is_torch(x):
    if x.is_cuda and x.dtype == tdt and x.is_contiguous():
      return x
    return x.to(device="cuda", dtype=tdt, non_blocking=True).contiguous()
  npdt = {torch.int32: np.int32, torch.float32: np.float32}[tdt]
  return torch.from_numpy(np.ascontiguousarray(x, dtype=npdt)).to(device="cuda", non_blocking=True)


def _cat(parts, tdt):
  torch = _native.torch_mod()
  parts = [_to_cuda(p, tdt) for p in parts]
  return parts[0] if len(parts) == 1 else torch.cat(parts)


class _DeviceBatch:
  """The rows of one stacked table that one device processes, as device arrays + descriptors."""

  def __init__(self, members, features, feature_weights, device_index: int, local_device_count: int):
    torch = _native.torch_mod()
    ids_parts, off_parts, w_parts, descs = [], [], [], []
    id_base, row_base = 0, 0
    any_ragged, any_weights = False, False
    for idx, spec in members:
      feature = features[idx]
      weights = None if feature_weights is None else feature_weights[idx]
      rows_total = _feature_rows(feature)
      per_dev = rows_total // local_device_count
      lo, hi = device_index * per_dev, (device_index + 1) * per_dev
      transform = _transform(spec)
      if isinstance(feature, RaggedInput):
        splits = feature.row_splits
        b, e = int(splits[lo]), int(splits[hi])
        ids_parts.append(feature.values[b:e])
        off = splits[lo:hi] - splits[lo] + id_base
        off_parts.append(off)
        w = feature.weights if feature.weights is not None else weights
        w_parts.append(None if w is None else w[b:e])
        descs.append(_native.FeatureDesc(row_base, per_dev, *transform, 0, 0))
        n_ids = e - b
        any_ragged = True
      elif _is_torch(feature) or (isinstance(feature, np.ndarray) and feature.dtype != object):
        if feature.ndim != 2:
          raise ValueError("Only 1D and 2D numpy arrays supported as inputs.")
        valency = int(feature.shape[1])
        ids_parts.append(feature[lo:hi].reshape(-1))
        off_parts.append(("dense", per_dev, valency, id_base))
        w_parts.append(None if weights is None else weights[lo:hi].reshape(-1))
        descs.append(_native.FeatureDesc(row_base, per_dev, *transform, valency, id_base))
        n_ids = per_dev * valency
        if valency == 0:
          any_ragged = True
      else:
        arr = np.asarray(feature)
        if arr.ndim != 1:
          raise ValueError("Only 1D and 2D numpy arrays supported as inputs.")
        rows = [np.asarray(r, dtype=np.int32).reshape(-1) for r in arr[lo:hi]]
        lens = np.fromiter((len(r) for r in rows), dtype=np.int64, count=len(rows))
        off = np.zeros(len(rows), dtype=np.int64)
        if len(rows) > 1:
          np.cumsum(lens[:-1], out=off[1:])
        n_ids = int(lens.sum())
        ids_parts.append(np.concatenate(rows) if n_ids else np.zeros(0, np.int32))
        off_parts.append(off + id_base)
        if weights is None:
          w_parts.append(None)
        else:
          wr = [np.asarray(r, dtype=np.float32).reshape(-1) for r in np.asarray(weights, dtype=object)[lo:hi]]
          w = np.concatenate(wr) if wr else np.zeros(0, np.float32)
          if len(w) != n_ids:
            raise ValueError("Dimension mismatch for features and weights")
          w_parts.append(w)
        descs.append(_native.FeatureDesc(row_base, per_dev, *transform, 0, 0))
        any_ragged = True
      any_weights = any_weights or w_parts[-1] is not None
      id_base += n_ids
      row_base += per_dev
    self.nnz, self.total_rows = id_base, row_base
    self.descs = (_native.FeatureDesc * len(descs))(*descs)
    self.ids = _cat(ids_parts, torch.int32) if id_base else torch.zeros(1, dtype=torch.int32, device="cuda")
    self.offsets = None
    if any_ragged:
      full = []
      for o in off_parts:
        if isinstance(o, tuple):
          _, rows, valency, base = o
          full.append(np.arange(rows, dtype=np.int64) * valency + base)
        else:
          full.append(o)
      full.append(np.asarray([id_base], np.int64))
      self.offsets = _cat(full, torch.int32)
    self.weights = None
    if any_weights:
      ws = [w if w is not None else np.ones(int(p.numel() if _is_torch(p) else np.size(p)), np.float32)
            for w, p in zip(w_parts, ids_parts)]
      self.weights = _cat(ws, torch.float32)


# ------------------------------------------------------------------------------ device call


def preprocess_stack_on_device(ids, row_offsets, weights, feature_descs, *, global_device_count: int,
                               num_sc_per_device: int, combiner: str, max_ids_per_partition: int,
                               max_unique_ids_per_partition: int, allow_id_dropping: bool,
                               coo_buffer_size_per_device: int, stack_vocab_size: int, outputs=None):
  """Runs `sc_preprocess_table` for one stacked table and one device, asynchronously.

  Args:
    ids, row_offsets, weights: CUDA int32 / int32 / float32 (or None) tensors, the CSR of the
      device's rows with the features of the stack back to back in row_offset order.
    feature_descs: list of (rows, row_offset, col_offset, col_shift) per feature.
    outputs: optional (row_pointers, embedding_ids, sample_ids, gains) tensors to fill.

  Returns:
    (row_pointers, embedding_ids, sample_ids, gains, stats) CUDA tensors; `stats` is the
    int32 block described in include/sc_b200.h.  Nothing is synchronised.
  """
  torch = _native.require_cuda()
  lib = _native.lib()
  nfeat = len(feature_descs)
  descs = (_native.FeatureDesc * nfeat)()
  row = 0
  for i, (rows, row_offset, col_offset, col_shift) in enumerate(feature_descs):
    descs[i] = _native.FeatureDesc(row, int(rows), int(row_offset), int(col_offset), int(col_shift), 0, 0)
    row += int(rows)
  total_rows = row
  nnz = int(ids.numel())
  if row_offsets.numel() != total_rows + 1:
    raise ValueError("row_offsets must have one entry per row plus one")
  opt = _native.PreprocessOptions(int(global_device_count), int(num_sc_per_device), _native.COMBINERS.get(combiner, 0),
                                  int(max_ids_per_partition), int(max_unique_ids_per_partition),
                                  int(bool(allow_id_dropping)), int(coo_buffer_size_per_device), int(stack_vocab_size))
  p = global_device_count * num_sc_per_device
  rp_size = max(p, 8) * num_sc_per_device
  if outputs is None:
    dev = ids.device
    outputs = (torch.empty(rp_size, dtype=torch.int32, device=dev),
               torch.empty(coo_buffer_size_per_device, dtype=torch.int32, device=dev),
               torch.empty(coo_buffer_size_per_device, dtype=torch.int32, device=dev),
               torch.empty(coo_buffer_size_per_device, dtype=torch.float32, device=dev))
  rp, eids, sids, gains = outputs
  stats = torch.empty(2 * p + num_sc_per_device + 3, dtype=torch.int32, device=ids.device)
  nbytes = lib.sc_preprocess_workspace_bytes(nnz, total_rows, ctypes.byref(opt))
  if nbytes == 0:
    _native.check(_native.SC_INVALID_ARGUMENT)
  ws = _native.workspace(nbytes, "preprocess")
  status = lib.sc_preprocess_table(
      ids.data_ptr() if nnz else None, row_offsets.data_ptr(), None if weights is None else weights.data_ptr(), nnz,
      total_rows, descs, nfeat, ctypes.byref(opt), rp.data_ptr(), eids.data_ptr(), sids.data_ptr(), gains.data_ptr(),
      stats.data_ptr(), ws.data_ptr(), ws.numel(), _native.current_stream_ptr())
  _native.check(status)
  return rp, eids, sids, gains, stats


def _raise_for_status(stats_host: np.ndarray, p: int, s: int, table: str, max_ids: int, max_unique: int) -> None:
  status = int(stats_host[2 * p + s + 1])
  if status == _native.SC_OK:
    return
  if status == _native.SC_ID_LIMIT_EXCEEDED:
    obs_ids, obs_unique = int(stats_host[:p].max()), int(stats_host[p:2 * p].max())
    if obs_ids > max_ids:
      raise ValueError(
          f"Observed max ids per partition: {obs_ids} for table: {table} is greater than the set max ids per "
          f"partition: {max_ids}. Use `allow_id_dropping` or increase the `max_ids_per_partition`. You could "
          "also try to reduce the batch size.")
    raise ValueError(
        f"Observed max unique ids per partition: {obs_unique} for table: {table} is greater than the set max "
        f"unique ids per partition: {max_unique}. Use `allow_id_dropping` or increase the "
        "`max_ids_per_partition`. You could also try to reduce the batch size.")
  raise ValueError(
      f"Invalid input for table {table}: an embedding id is negative or outside the stacked vocabulary, or the "
      "feature row offsets do not match the batch.")


class _DeferredStats:
  """The statistics block of one call while it travels to the host (pinned buffer + CUDA event).

  `resolve()` waits for the copy, raises the ValueError of a violated limit or invalid input exactly as
  the synchronous path does, and returns the four per-table dicts.  It runs at most once.
  """

  def __init__(self, pinned, event, names, limits, p, s):
    self.pinned, self.event, self.names, self.limits, self.p, self.s = pinned, event, names, limits, p, s
    self.host = None  # the block once it has arrived
    self.fields = None
    self.error = None

  def check(self):
    """Waits for the copy and raises the error of the call, if any (cheap: one vector test of the status column).
    The per-table dicts are built only when somebody reads them."""
    if self.host is None:
      self.event.synchronize()
      self.host = self.pinned.numpy().copy()
      self.pinned = None
      p, s = self.p, self.s
      try:
        status = self.host[:, 2 * p + s + 1]
        if status.any():
          si = int(np.flatnonzero(status)[0])
          _raise_for_status(self.host[si], p, s, self.names[si], *self.limits[si])
      except ValueError as e:
        self.error = e
    if self.error is not None:
      raise self.error

  @property
  def checked(self) -> bool:
    return self.host is not None

  def resolve(self):
    self.check()
    if self.fields is None:
      host, p, s = self.host, self.p, self.s
      fields = ({}, {}, {}, {})
      for si, name in enumerate(self.names):
        fields[0][name] = host[si, :p].copy()
        fields[1][name] = host[si, p:2 * p].copy()
        fields[2][name] = host[si, 2 * p:2 * p + s].copy()
        fields[3][name] = int(host[si, 2 * p + s])
      self.fields = fields
    return self.fields


class LazyStatsDict(dict):
  """One per-table statistics dict that is filled from a _DeferredStats on first use."""

  def __init__(self, *args, deferred=None, field=0, **kw):
    super().__init__(*args, **kw)
    self._deferred, self._field = deferred, field

  def _fill(self):
    if self._deferred is not None:
      deferred, self._deferred = self._deferred, None
      super().update(deferred.resolve()[self._field])

  def __getitem__(self, k):
    self._fill()
    return super().__getitem__(k)

  def __iter__(self):
    self._fill()
    return super().__iter__()

  def __len__(self):
    self._fill()
    return super().__len__()

  def __contains__(self, k):
    self._fill()
    return super().__contains__(k)

  def __repr__(self):
    self._fill()
    return super().__repr__()

  def __eq__(self, other):
    self._fill()
    return super().__eq__(other)

  __hash__ = None

  def keys(self):
    self._fill()
    return super().keys()

  def values(self):
    self._fill()
    return super().values()

  def items(self):
    self._fill()
    return super().items()

  def get(self, k, default=None):
    self._fill()
    return super().get(k, default)

  def __setitem__(self, k, v):
    self._fill()
    super().__setitem__(k, v)

  def copy(self):
    self._fill()
    return dict(self)


class BufferDict(dict):
  """dict of output arrays that remembers which device buffers all its values are views of.

  `token` = (address of the int32 buffer, address of the float32 buffer, layout ..., index of the dict): callers
  that cache launch descriptors use it instead of looking at every array - the layout part keys the cache, the
  two addresses are all that differs between the outputs of two calls with one layout.  Any change of the dict drops
  the token.
  """

  token = None
  forward_plans = None  # on the row-pointer dict: {stack name: (plan_slots, plan_bags)} for the forward

  def _changed(self):
    self.token = None
    self.forward_plans = None

  def __setitem__(self, k, v):
    self._changed()
    super().__setitem__(k, v)

  def __delitem__(self, k):
    self._changed()
    super().__delitem__(k)

  def update(self, *a, **k):
    self._changed()
    super().update(*a, **k)

  def pop(self, *a):
    self._changed()
    return super().pop(*a)

  def clear(self):
    self._changed()
    super().clear()

  def setdefault(self, *a):
    self._changed()
    return super().setdefault(*a)

  def popitem(self):
    self._changed()
    return super().popitem()


class _DensePlan:
  """Everything about a call that depends only on the specs and the input shapes.

  Used when every feature is a dense 2-D int32 CUDA tensor (and every weight a float32 one) and the
  process handles one device: the launch descriptors, buffer layout and workspace size are built
  once; a call then only allocates its output buffers and fills in addresses.
  """

  def __init__(self, feature_specs, shapes, weighted: bool, global_device_count: int, s: int, allow_id_dropping: bool):
    self.keep = list(feature_specs)
    self.stacks = list(_group_by_stack(feature_specs).items())
    self.weighted = weighted
    p = s * global_device_count
    self.p, self.s = p, s
    self.rp_size = max(p, 8) * s
    self.stats_size = 2 * p + s + 3
    n = len(self.stacks)
    self.items = (_native.PreprocessItem * n)()
    self.descs = []
    self.members = []
    self.coos, self.limits, self.names = [], [], []
    for si, (stack_name, members) in enumerate(self.stacks):
      stacked = members[0][1].table_spec.stacked_table_spec
      coo = _coo_buffer_size(stacked.max_ids_per_partition, global_device_count, s,
                             stacked.suggested_coo_buffer_size_per_device)
      self.coos.append(coo)
      self.names.append(stack_name)
      self.limits.append((stacked.max_ids_per_partition, stacked.max_unique_ids_per_partition))
      descs, id_base, row_base = [], 0, 0
      for idx, spec in members:
        rows, valency = shapes[idx]
        descs.append(_native.FeatureDesc(row_base, rows, *_transform(spec), valency, id_base))
        id_base += rows * valency
        row_base += rows
      arr = (_native.FeatureDesc * len(descs))(*descs)
      self.descs.append(arr)
      self.members.append([idx for idx, _ in members])
      it = self.items[si]
      it.row_offsets = None
      it.weights = None
      it.nnz, it.total_rows = id_base, row_base
      it.features = arr
      it.num_features = len(descs)
      it.options = _native.PreprocessOptions(
          int(global_device_count), int(s), _native.COMBINERS.get(stacked.combiner, 0),
          int(stacked.max_ids_per_partition), int(stacked.max_unique_ids_per_partition),
          int(bool(allow_id_dropping)), int(coo), int(stacked.stack_vocab_size))
    # Output layout: one int32 buffer [row pointers | embedding ids | sample ids] per stack, one
    # float32 buffer of gains; byte offsets of every array.
    self.int_sizes, self.int_offsets = [], []
    pos = 0
    for coo in self.coos:
      for size in (self.rp_size, coo, coo):
        self.int_sizes.append(size)
        self.int_offsets.append(pos * 4)
        pos += size
    # ... followed by the forward plan of every stack: [slots (one per input id) | bags (two per row)].
    self.plan_sizes, self.plan_offsets = [], []
    for si in range(n):
      for size in (int(self.items[si].nnz), 2 * int(self.items[si].total_rows)):
        pos = (pos + 3) // 4 * 4  # 16-byte aligned
        self.plan_sizes.append(size)
        self.plan_offsets.append(pos * 4)
        pos += size
    self.int_total = pos
    self.float_offsets = [4 * sum(self.coos[:i]) for i in range(n)]
    self.float_total = sum(self.coos)
    # One split of the int32 buffer yields every output view: pieces in address order, alignment gaps included.
    pieces = sorted([(off // 4, size, ("csr", i)) for i, (off, size) in enumerate(zip(self.int_offsets, self.int_sizes))] +
                    [(off // 4, size, ("plan", i)) for i, (off, size) in enumerate(zip(self.plan_offsets, self.plan_sizes))])
    self.split_sizes, self.csr_piece, self.plan_piece = [], [0] * len(self.int_sizes), [0] * len(self.plan_sizes)
    cursor = 0
    for off, size, (kind, i) in pieces:
      if off > cursor:
        self.split_sizes.append(off - cursor)
      (self.csr_piece if kind == "csr" else self.plan_piece)[i] = len(self.split_sizes)
      self.split_sizes.append(size)
      cursor = off + size
    if cursor < self.int_total:
      self.split_sizes.append(self.int_total - cursor)
    # Pickers of the pieces of one output column (row pointers, ids, sample ids) and of the plan arrays, in stack order.
    def picker(indices):
      indices = list(indices)
      return operator.itemgetter(*indices) if len(indices) > 1 else (lambda seq, i=indices[0]: (seq[i],))
    n_stacks = len(self.int_sizes) // 3
    self.pick_columns = [picker(self.csr_piece[3 * si + k] for si in range(n_stacks)) for k in range(3)]
    self.pick_plan_slots = picker(self.plan_piece[2 * si] for si in range(n_stacks))
    self.pick_plan_bags = picker(self.plan_piece[2 * si + 1] for si in range(n_stacks))
    # The pointer fields of the launch descriptors as strided numpy views: a call fills them with a few
    # vector operations instead of one attribute assignment per field and stack.
    stride = ctypes.sizeof(_native.PreprocessItem)

    def field(name):
      return np.ndarray((n,), dtype=np.uint64, buffer=self.items, offset=getattr(_native.PreprocessItem, name).offset,
                        strides=(stride,))

    self.f_ids, self.f_weights = field("ids"), field("weights")
    self.f_out = [field(k) for k in ("row_pointers", "embedding_ids", "sample_ids", "plan_slots", "plan_bags")]
    self.o_out = [np.asarray(self.int_offsets[0::3], np.uint64), np.asarray(self.int_offsets[1::3], np.uint64),
                  np.asarray(self.int_offsets[2::3], np.uint64), np.asarray(self.plan_offsets[0::2], np.uint64),
                  np.asarray(self.plan_offsets[1::2], np.uint64)]
    self.f_gains, self.o_gains = field("gains"), np.asarray(self.float_offsets, np.uint64)
    self.f_stats, self.o_stats = field("stats"), np.arange(n, dtype=np.uint64) * np.uint64(self.stats_size * 4)
    self.single_member = all(len(m) == 1 for m in self.members)
    self.first_member = [m[0] for m in self.members]
    self.groups = None  # launch groups and workspace sizes, sized on the first run (needs real addresses)
    self.deferred = [None] * 4  # statistics of the last calls made with sync_stats=False (ring)
    self.deferred_next = 0

  def _size_groups(self):
    """Launch groups (bounded by the 32-bit sort key) and their workspace sizes."""
    lib = _native.lib()
    n = len(self.stacks)
    self.groups = []
    start = 0
    while start < n:
      m = n - start
      while True:
        sub = ctypes.cast(ctypes.byref(self.items, start * ctypes.sizeof(_native.PreprocessItem)),
                          ctypes.POINTER(_native.PreprocessItem))
        nbytes = lib.sc_preprocess_grouped_workspace_bytes(sub, m)
        if nbytes or m == 1:
          break
        m = (m + 1) // 2
      self.groups.append((sub, m, nbytes))
      start += m

  def run(self, features, feature_weights, has_leading_dimension: bool, device_output: bool, sync_stats: bool = True):
    torch = _native.torch_mod()
    lib = _native.lib()
    n = len(self.stacks)
    if not sync_stats:
      # The statistics of the previous deferred call have long arrived: a violated limit surfaces here.
      previous = self.deferred[(self.deferred_next - 1) % len(self.deferred)]
      if previous is not None and not previous.checked and previous.event.query():
        previous.check()
    ints = torch.empty(self.int_total, dtype=torch.int32, device="cuda")
    floats = torch.empty(self.float_total, dtype=torch.float32, device="cuda")
    stats_dev = torch.empty((n, self.stats_size), dtype=torch.int32, device="cuda")
    ibase, fbase, sbase = ints.data_ptr(), floats.data_ptr(), stats_dev.data_ptr()
    keep = []
    if self.single_member:
      self.f_ids[:] = [features[i].data_ptr() for i in self.first_member]
      if self.weighted:
        self.f_weights[:] = [feature_weights[i].data_ptr() for i in self.first_member]
    else:
      for si in range(n):
        it = self.items[si]
        idxs = self.members[si]
        if len(idxs) == 1:
          it.ids = features[idxs[0]].data_ptr()
          if self.weighted:
            it.weights = feature_weights[idxs[0]].data_ptr()
        else:
          cat = torch.cat([features[i].reshape(-1) for i in idxs])
          keep.append(cat)
          it.ids = cat.data_ptr()
          if self.weighted:
            wcat = torch.cat([feature_weights[i].reshape(-1) for i in idxs])
            keep.append(wcat)
            it.weights = wcat.data_ptr()
    for view, offsets in zip(self.f_out[:3] if not device_output else self.f_out, self.o_out):
      view[:] = offsets + np.uint64(ibase)
    if not device_output:
      self.f_out[3][:] = 0
      self.f_out[4][:] = 0
    self.f_gains[:] = self.o_gains + np.uint64(fbase)
    self.f_stats[:] = self.o_stats + np.uint64(sbase)
    stream = _native.current_stream_ptr()
    if self.groups is None:
      self._size_groups()
    for sub, m, nbytes in self.groups:
      if nbytes == 0:
        _native.check(lib.sc_preprocess_grouped(sub, m, None, 0, None))
      ws = _native.workspace(nbytes, "preprocess")
      _native.check(lib.sc_preprocess_grouped(sub, m, ws.data_ptr(), ws.numel(), stream))
    p, s = self.p, self.s
    stats = SparseDenseMatmulInputStats()
    host = None
    if sync_stats:
      host = stats_dev.cpu().numpy()  # the only synchronisation of the call
      status = host[:, 2 * p + s + 1]
      if status.any():
        si = int(np.flatnonzero(status)[0])
        _raise_for_status(host[si], p, s, self.names[si], *self.limits[si])
      max_ids, max_unique = host[:, :p].copy(), host[:, p:2 * p].copy()
      required, dropped = host[:, 2 * p:2 * p + s].copy(), host[:, 2 * p + s]
    else:
      # No synchronisation: the block is copied to pinned memory behind the kernels; the dicts of `stats` fetch
      # it (and raise for a violated limit) when they are first read.
      slot = self.deferred_next % len(self.deferred)
      old = self.deferred[slot]
      if old is not None and not old.checked:
        try:
          old.check()  # its pinned buffer is about to be recycled
        except ValueError:
          pass
      pinned = torch.empty((n, self.stats_size), dtype=torch.int32, pin_memory=True)
      pinned.copy_(stats_dev, non_blocking=True)
      event = torch.cuda.Event()
      event.record()
      deferred = _DeferredStats(pinned, event, list(self.names), list(self.limits), p, s)
      self.deferred[slot] = deferred
      self.deferred_next += 1
      stats.max_ids_per_partition = LazyStatsDict(deferred=deferred, field=0)
      stats.max_unique_ids_per_partition = LazyStatsDict(deferred=deferred, field=1)
      stats.required_buffer_sizes = LazyStatsDict(deferred=deferred, field=2)
      stats.dropped_id_count = LazyStatsDict(deferred=deferred, field=3)
    del keep
    pieces = torch.split_with_sizes(ints, self.split_sizes)
    float_views = torch.split_with_sizes(floats, self.coos)
    columns = [list(pick(pieces)) for pick in self.pick_columns] + [list(float_views)]
    if has_leading_dimension:
      columns = [[t.view(1, -1) for t in col] for col in columns]
    if not device_output:
      columns = [[t.cpu().numpy() for t in col] for col in columns]
    # dict.__init__ fills the dicts without the per-item bookkeeping of BufferDict.__setitem__.
    out_rp, out_ids, out_sids, out_gains = (BufferDict(zip(self.names, col)) for col in columns)
    if host is not None:
      for si, name in enumerate(self.names):
        stats.max_ids_per_partition[name] = max_ids[si]
        stats.max_unique_ids_per_partition[name] = max_unique[si]
        stats.required_buffer_sizes[name] = required[si]
        stats.dropped_id_count[name] = int(dropped[si])
    if device_output:
      # The arrays keep the two buffers alive, so the addresses identify the contents' location.
      token = (ibase, fbase, self, bool(has_leading_dimension))  # (addresses of the two buffers, layout ...)
      for i, d in enumerate((out_rp, out_ids, out_sids, out_gains)):
        d.token = token + (i,)
      out_rp.forward_plans = dict(zip(self.names, zip(self.pick_plan_slots(pieces), self.pick_plan_bags(pieces))))
    return out_rp, out_ids, out_sids, out_gains, 1, stats


_DENSE_PLANS: dict = {}


def clear_caches() -> None:
  """Forgets the cached per-spec preprocessing plans."""
  _DENSE_PLANS.clear()


def _dense_plan(features, feature_weights, feature_specs, local_device_count, global_device_count, s, allow_id_dropping):
  """The cached _DensePlan of this call, or None if the inputs do not qualify."""
  torch = _native.torch_mod()
  if local_device_count != 1:
    return None
  shapes = []
  for f in features:
    if not (isinstance(f, torch.Tensor) and f.is_cuda and f.dtype == torch.int32 and f.dim() == 2 and f.shape[1] > 0
            and f.is_contiguous()):
      return None
    shapes.append((int(f.shape[0]), int(f.shape[1])))
  weighted = feature_weights is not None
  if weighted:
    for w, f in zip(feature_weights, features):
      if not (isinstance(w, torch.Tensor) and w.is_cuda and w.dtype == torch.float32 and w.shape == f.shape
              and w.is_contiguous()):
        return None
  key = (tuple((id(f), id(f.table_spec._stacked_table_spec), id(f._id_transformation)) for f in feature_specs),  # pylint: disable=protected-access
         tuple(shapes), weighted, global_device_count, s, bool(allow_id_dropping))
  plan = _DENSE_PLANS.get(key)
  if plan is None:
    if len(_DENSE_PLANS) > 16:
      _DENSE_PLANS.clear()
    plan = _DENSE_PLANS[key] = _DensePlan(feature_specs, shapes, weighted, global_device_count, s, allow_id_dropping)
  return plan


def preprocess_sparse_dense_matmul_input(features, feature_weights, feature_specs, local_device_count: int,
                                         global_device_count: int, *, num_sc_per_device: int,
                                         sharding_strategy: ShardingStrategy = ShardingStrategy.MOD,
                                         has_leading_dimension: bool = False, allow_id_dropping: bool = False,
                                         batch_number: int = 0, enable_minibatching: bool = False,
                                         all_reduce_interface=None, device_output: bool = False,
                                         sync_stats: bool = True):
  """Flat lists of features / weights / specs -> (row_pointers, embedding_ids, sample_ids, gains,
  num_minibatches, stats), the first four being dicts keyed by stacked table name.

  sync_stats=False (dense device inputs only) returns without waiting for the GPU: the statistics arrive when
  they are first read, and a violated id limit raises then, or at the next call, instead of at this one."""
  del batch_number, all_reduce_interface
  _reject_minibatching(enable_minibatching)
  if int(sharding_strategy) != int(ShardingStrategy.MOD):
    raise ValueError("Only mod sharding is supported for now.")
  # PreprocessSparseDenseMatmulInputOptions::Validate (input_preprocessing_util.cc:490-522).
  if local_device_count <= 0:
    raise ValueError(f"local_device_count must be greater than 0, but got {local_device_count}")
  if global_device_count <= 0:
    raise ValueError(f"global_device_count must be greater than 0, but got {global_device_count}")
  if global_device_count < local_device_count:
    raise ValueError(
        "global_device_count must be greater than or equal to local_device_count, but got "
        f"{global_device_count} vs {local_device_count}")
  if num_sc_per_device <= 0:
    raise ValueError(f"num_sc_per_device must be greater than 0, but got {num_sc_per_device}")
  p = num_sc_per_device * global_device_count
  if p & (p - 1):
    raise ValueError(f"Total number of SparseCores ({p}) must be a power of 2.")
  features = list(features)
  if not features:
    raise ValueError("input_batches cannot be empty.")
  feature_specs = list(feature_specs)
  if feature_weights is not None:
    feature_weights = list(feature_weights)
    if len(feature_weights) != len(features):
      raise ValueError("features and feature_weights must have the same length")
  if len(features) != len(feature_specs):
    raise ValueError("features and feature_specs must have the same length")

  torch = _native.require_cuda()
  lib = _native.lib()
  l, s = local_device_count, num_sc_per_device
  plan = _dense_plan(features, feature_weights, feature_specs, l, global_device_count, s, allow_id_dropping)
  if plan is not None:
    return plan.run(features, feature_weights, has_leading_dimension, device_output, sync_stats and True)
  out_rp, out_ids, out_sids, out_gains = BufferDict(), BufferDict(), BufferDict(), BufferDict()
  stats = SparseDenseMatmulInputStats()
  stacks = list(_group_by_stack(feature_specs).items())
  rp_size = max(p, 8) * s
  stats_size = 2 * p + s + 3
  coos = []
  for _, members in stacks:
    stacked = members[0][1].table_spec.stacked_table_spec
    coos.append(_coo_buffer_size(stacked.max_ids_per_partition, global_device_count, s,
                                 stacked.suggested_coo_buffer_size_per_device))
  batches = [[_DeviceBatch(members, features, feature_weights, d, l) for d in range(l)] for _, members in stacks]
  # One int32 buffer holds [row pointers | embedding ids | sample ids] of every stack and device (and, for a
  # single device with device output, the forward plan of every stack), one float32 buffer the gains, one
  # int32 buffer the statistics.
  with_plan = device_output and l == 1
  int_total = sum(l * (rp_size + 2 * c) for c in coos)
  plan_offsets = []
  if with_plan:
    for (batch,) in batches:
      for size in (batch.nnz, 2 * batch.total_rows):
        int_total = (int_total + 3) // 4 * 4
        plan_offsets.append((int_total, size))
        int_total += size
  ints = torch.empty(int_total, dtype=torch.int32, device="cuda")
  floats = torch.empty(sum(l * c for c in coos), dtype=torch.float32, device="cuda")
  stats_dev = torch.empty((len(stacks), l, stats_size), dtype=torch.int32, device="cuda")
  items = (_native.PreprocessItem * (len(stacks) * l))()
  keep, views = batches, []
  ipos = fpos = 0
  for si, ((stack_name, members), coo) in enumerate(zip(stacks, coos)):
    stacked = members[0][1].table_spec.stacked_table_spec
    rp_v = ints[ipos:ipos + l * rp_size].view(l, rp_size); ipos += l * rp_size
    id_v = ints[ipos:ipos + l * coo].view(l, coo); ipos += l * coo
    sid_v = ints[ipos:ipos + l * coo].view(l, coo); ipos += l * coo
    gain_v = floats[fpos:fpos + l * coo].view(l, coo); fpos += l * coo
    views.append((rp_v, id_v, sid_v, gain_v))
    opt = _native.PreprocessOptions(int(global_device_count), int(s), _native.COMBINERS.get(stacked.combiner, 0),
                                    int(stacked.max_ids_per_partition), int(stacked.max_unique_ids_per_partition),
                                    int(bool(allow_id_dropping)), int(coo), int(stacked.stack_vocab_size))
    for d in range(l):
      batch = batches[si][d]
      it = items[si * l + d]
      it.ids = batch.ids.data_ptr()
      it.row_offsets = None if batch.offsets is None else batch.offsets.data_ptr()
      it.weights = None if batch.weights is None else batch.weights.data_ptr()
      it.nnz, it.total_rows = batch.nnz, batch.total_rows
      it.features = batch.descs
      it.num_features = len(batch.descs)
      it.options = opt
      it.row_pointers = rp_v[d].data_ptr()
      it.embedding_ids = id_v[d].data_ptr()
      it.sample_ids = sid_v[d].data_ptr()
      it.gains = gain_v[d].data_ptr()
      it.stats = stats_dev[si, d].data_ptr()
      if with_plan:
        it.plan_slots = ints.data_ptr() + 4 * plan_offsets[2 * si][0]
        it.plan_bags = ints.data_ptr() + 4 * plan_offsets[2 * si + 1][0]
  # Groups are bounded by the 32-bit sort key: split greedily when a group does not fit.
  start, count = 0, len(items)
  stream = _native.current_stream_ptr()
  while start < count:
    n = count - start
    while True:
      sub = ctypes.cast(ctypes.byref(items, start * ctypes.sizeof(_native.PreprocessItem)),
                        ctypes.POINTER(_native.PreprocessItem))
      nbytes = lib.sc_preprocess_grouped_workspace_bytes(sub, n)
      if nbytes or n == 1:
        break
      n = (n + 1) // 2
    if nbytes == 0:
      _native.check(lib.sc_preprocess_grouped(sub, n, None, 0, None))
    ws = _native.workspace(nbytes, "preprocess")
    _native.check(lib.sc_preprocess_grouped(sub, n, ws.data_ptr(), ws.numel(), stream))
    start += n

  host = stats_dev.cpu().numpy()  # the only synchronisation of the call
  del keep
  for si, ((stack_name, members), dev_out) in enumerate(zip(stacks, views)):
    stacked = members[0][1].table_spec.stacked_table_spec
    for d in range(l):
      _raise_for_status(host[si, d], p, s, stack_name, stacked.max_ids_per_partition,
                        stacked.max_unique_ids_per_partition)
    stats.max_ids_per_partition[stack_name] = host[si, :, :p].reshape(-1).copy()
    stats.max_unique_ids_per_partition[stack_name] = host[si, :, p:2 * p].reshape(-1).copy()
    stats.required_buffer_sizes[stack_name] = host[si, :, 2 * p:2 * p + s].reshape(-1).copy()
    stats.dropped_id_count[stack_name] = int(host[si, :, 2 * p + s].sum())
    arrays = dev_out if has_leading_dimension else tuple(t.reshape(-1) for t in dev_out)
    if not device_output:
      arrays = tuple(t.cpu().numpy() for t in arrays)
    out_rp[stack_name], out_ids[stack_name], out_sids[stack_name], out_gains[stack_name] = arrays
  if with_plan:
    # The arrays keep the buffers alive; addresses plus layout identify every array of the call.
    token = (ints.data_ptr(), floats.data_ptr(), tuple(coos), tuple(plan_offsets), rp_size, bool(has_leading_dimension))
    for i, d in enumerate((out_rp, out_ids, out_sids, out_gains)):
      d.token = token + (i,)
    out_rp.forward_plans = {
        name: tuple(ints[off:off + size] for off, size in plan_offsets[2 * si:2 * si + 2])
        for si, (name, _) in enumerate(stacks)}
  return out_rp, out_ids, out_sids, out_gains, 1, stats


def preprocess_sparse_dense_matmul_sparse_coo_input(indices, values, dense_shapes, feature_specs, local_device_count: int,
                                                    global_device_count: int, *, num_sc_per_device: int,
                                                    sharding_strategy: ShardingStrategy = ShardingStrategy.MOD,
                                                    has_leading_dimension: bool = False,
                                                    allow_id_dropping: bool = False, batch_number: int = 0,
                                                    enable_minibatching: bool = False, all_reduce_interface=None,
                                                    device_output: bool = False):
  """Same as preprocess_sparse_dense_matmul_input for features given as sparse COO tensors.

  Per feature: `indices` int [N, 2] of (sample, position) in row-major order, `values` int32 [N]
  of embedding ids, `dense_shape` (batch, max positions).  Every id has weight 1.  Mirrors
  `preprocess_sparse_dense_matmul_sparse_coo_input` of the reference's pybind module
  (jax_tpu_embedding/sparsecore/lib/core/pybind_input_preprocessing.cc:301-310; the row pointers
  of sparse_coo_input_batch.cc:35-79 are the row splits built here).
  """
  indices, values, dense_shapes = list(indices), list(values), list(dense_shapes)
  if not (len(indices) == len(values) == len(dense_shapes) == len(list(feature_specs))):
    raise ValueError("indices, values, dense_shapes and feature_specs must have the same length")
  features = []
  for idx, val, shape in zip(indices, values, dense_shapes):
    idx = np.asarray(idx.cpu() if _is_torch(idx) else idx)
    val_host = np.asarray(val.cpu() if _is_torch(val) else val)
    shape = np.asarray(shape).reshape(-1)
    if idx.ndim != 2 or idx.shape[1] != 2:
      raise ValueError(f"indices must have shape [N, 2], got {idx.shape}")
    if val_host.ndim != 1 or len(val_host) != len(idx):
      raise ValueError("values must be 1-D with one id per index")
    if len(shape) != 2:
      raise ValueError("dense_shape must have two elements")
    batch = int(shape[0])
    rows = idx[:, 0]
    if len(rows) and (np.any(np.diff(rows) < 0) or rows[0] < 0 or rows[-1] >= batch):
      raise ValueError("indices must be in row-major order with row ids inside the dense shape")
    splits = np.searchsorted(rows, np.arange(batch + 1), side="left").astype(np.int64)
    features.append(RaggedInput(np.ascontiguousarray(val_host, dtype=np.int32), splits, None))
  return preprocess_sparse_dense_matmul_input(
      features, None, feature_specs, local_device_count, global_device_count, num_sc_per_device=num_sc_per_device,
      sharding_strategy=sharding_strategy, has_leading_dimension=has_leading_dimension,
      allow_id_dropping=allow_id_dropping, batch_number=batch_number, enable_minibatching=enable_minibatching,
      all_reduce_interface=all_reduce_interface, device_output=device_output)
