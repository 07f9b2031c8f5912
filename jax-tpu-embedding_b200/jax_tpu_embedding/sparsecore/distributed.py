"""Row-sharded tables across the GPUs of one box: one process per GPU.

The reference runs lookup and update per device inside `jax.shard_map`; the exchange between
chips happens inside the TPU custom call (jax_tpu_embedding/sparsecore/docs/parameters.rst:20-24,
sharding in lib/nn/embedding.py:1092-1112).  Here every process owns shard `rank` of each stacked
table (`num_sc_per_device == 1`) and all shards are mapped into every process through CUDA IPC:

* forward  - the gather kernel reads remote table rows with plain loads over NVLink; no ids are
             exchanged and no second collective follows;
* backward - every process copies its CSR buffers and activation gradients into peer-visible
             exchange buffers; the owner of a shard then pulls, from all processes, the entries
             destined to it, reduces all contributions of a row in a fixed (source, sample) order
             and applies the optimizer once.

Ordering between processes uses stream-ordered barriers (a 4-byte NCCL all-reduce on the compute
stream), never host-side waits inside kernels.
"""

from __future__ import annotations

import ctypes
import dataclasses

import numpy as np

from jax_tpu_embedding.sparsecore import _native


@dataclasses.dataclass
class _PeerAllocation:
  base: int
  nbytes: int
  peer_bases: list  # device pointer of the same allocation in every rank's address space
  tensor: object


class _Context:

  def __init__(self, rank: int, world: int, group):
    self.rank, self.world, self.group = rank, world, group
    self.allocations: list[_PeerAllocation] = []
    self.exchange: dict = {}
    self.token = None
    # What the peers may still be doing with this rank's memory since the last barrier.
    self.peers_may_read_exchange = False  # a pull update was launched: peers read the exchange buffers
    self.peers_may_write_tables = True    # ... and update the shards that the next lookup reads (or still fill them)


_ctx: _Context | None = None


def init(group=None) -> None:
  """Call once per process after torch.distributed.init_process_group and torch.cuda.set_device."""
  global _ctx
  torch = _native.require_cuda()
  dist = torch.distributed
  if not dist.is_initialized():
    raise RuntimeError("torch.distributed must be initialised before sparsecore.distributed.init")
  _ctx = _Context(dist.get_rank(group), dist.get_world_size(group), group)
  _ctx.token = torch.zeros(1, dtype=torch.int32, device="cuda")


def is_active() -> bool:
  return _ctx is not None and _ctx.world > 1


def rank() -> int:
  return _ctx.rank if _ctx else 0


def world_size() -> int:
  return _ctx.world if _ctx else 1


class _RawCudaBuffer:
  """Exposes a raw device allocation through the CUDA array interface."""

  def __init__(self, ptr: int, nbytes: int):
    self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                     "strides": None}


def alloc(shape, dtype=None):
  """Collective: allocates a tensor of `shape` on every rank and maps all of them into every rank.

  Must be called by all ranks in the same order with the same shape.  The memory comes from
  `sc_peer_alloc` (cudaMalloc) so that it can be exported through CUDA IPC.
  """
  torch = _native.require_cuda()
  if _ctx is None:
    raise RuntimeError("sparsecore.distributed.init() was not called")
  dtype = dtype or torch.float32
  lib = _native.lib()
  nbytes = int(np.prod(shape)) * torch.empty(0, dtype=dtype).element_size()
  # Whole 2 MiB pages: a peer mapping of an allocation that is not a multiple of the large page
  # size falls back to small pages, and random row reads over NVLink then run at a quarter of the
  # link bandwidth (measured: 160 GB/s against 700 GB/s).
  page = 2 << 20
  nbytes = max((nbytes + page - 1) // page * page, page)
  ptr = _native.c_vp()
  _native.check(lib.sc_peer_alloc(nbytes, ctypes.byref(ptr)))
  handle = ctypes.create_string_buffer(64)
  _native.check(lib.sc_ipc_export(ptr, handle))
  gathered = [None] * _ctx.world
  torch.distributed.all_gather_object(gathered, bytes(handle.raw), group=_ctx.group)
  bases = []
  for r, h in enumerate(gathered):
    if r == _ctx.rank:
      bases.append(int(ptr.value))
      continue
    peer = _native.c_vp()
    _native.check(lib.sc_ipc_import(ctypes.create_string_buffer(h, 64), ctypes.byref(peer)))
    bases.append(int(peer.value))
  flat = torch.as_tensor(_RawCudaBuffer(int(ptr.value), nbytes), device="cuda")
  tensor = flat[:int(np.prod(shape)) * torch.empty(0, dtype=dtype).element_size()].view(dtype).view(*shape)
  _ctx.allocations.append(_PeerAllocation(int(ptr.value), nbytes, bases, flat))
  _ctx.peers_may_write_tables = True  # the owner is about to fill it: the next lookup starts with a barrier
  return tensor


def peer_pointers(tensor) -> list[int]:
  """Device pointers of `tensor`'s counterpart on every rank (tensor must come from `alloc`)."""
  if _ctx is None:
    raise RuntimeError("sparsecore.distributed.init() was not called")
  p = tensor.data_ptr()
  for a in _ctx.allocations:
    if a.base <= p < a.base + a.nbytes:
      off = p - a.base
      return [b + off for b in a.peer_bases]
  raise ValueError(
      "This tensor is not visible to the other GPUs: with row-sharded tables (global_device_count > devices in "
      "this process) tables and slot variables must be created by embedding.init_embedding_variables or "
      "sparsecore.distributed.alloc.")


def shard_pointers(tensor, geo):
  """Pointers of all `geo.p` shards of a stacked table whose local part is `tensor`."""
  bases = peer_pointers(tensor)
  local_shards = geo.s_eff
  stride = geo.rows_per_shard * geo.dim * 4
  arr = (_native.c_vp * geo.p)()
  for g in range(geo.p):
    arr[g] = bases[g // local_shards] + (g % local_shards) * stride
  return arr


_barrier_events: list | None = None  # (name, begin event, end event) while barrier timing is on


def time_barriers(enable: bool) -> None:
  """Starts (and clears) or stops recording a pair of CUDA events around every stream barrier."""
  global _barrier_events
  _barrier_events = [] if enable else None


def barrier_times() -> dict:
  """{barrier name: total milliseconds} since time_barriers(True); clears the records."""
  out: dict = {}
  if _barrier_events:
    torch = _native.torch_mod()
    torch.cuda.synchronize()
    for name, begin, end in _barrier_events:
      out[name] = out.get(name, 0.0) + begin.elapsed_time(end)
    _barrier_events.clear()
  return out


def stream_barrier(name: str = "Barrier") -> None:
  """All work enqueued so far on every rank's current stream completes before any rank continues."""
  torch = _native.torch_mod()
  if is_active():
    if _barrier_events is not None:
      begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      begin.record()
    torch.distributed.all_reduce(_ctx.token, group=_ctx.group)
    if _barrier_events is not None:
      end.record()
      _barrier_events.append((name, begin, end))
    _ctx.peers_may_read_exchange = False
    _ctx.peers_may_write_tables = False


def barrier_before_lookup() -> None:
  """Remote rows are about to be read: needed only if a peer may still be updating its shard."""
  if is_active() and _ctx.peers_may_write_tables:
    stream_barrier("BarrierBeforeLookup")


def barrier_before_staging() -> None:
  """The exchange buffers are about to be overwritten: needed only if a peer may still read them."""
  if is_active() and _ctx.peers_may_read_exchange:
    stream_barrier("BarrierBeforeStaging")


def note_update_launched() -> None:
  """Every rank launched its pull update (all ranks run the same call sequence)."""
  if _ctx is not None:
    _ctx.peers_may_read_exchange = True
    _ctx.peers_may_write_tables = True


def release_all() -> None:
  """Collective: frees every peer-visible allocation of this process and unmaps the peers' ones.

  Tensors returned by `alloc` (tables, slot variables, exchange buffers) must not be used afterwards.  All
  ranks finish their work and drop their mappings before any rank frees its memory.
  """
  if _ctx is None:
    return
  torch = _native.torch_mod()
  lib = _native.lib()
  torch.cuda.synchronize()
  torch.distributed.barrier(group=_ctx.group)
  for a in _ctx.allocations:
    for r, base in enumerate(a.peer_bases):
      if r != _ctx.rank:
        _native.check(lib.sc_ipc_release(_native.c_vp(base)))
  torch.distributed.barrier(group=_ctx.group)
  for a in _ctx.allocations:
    _native.check(lib.sc_peer_free(_native.c_vp(a.base)))
  _ctx.allocations.clear()
  _ctx.exchange.clear()
  _ctx.peers_may_read_exchange = False
  _ctx.peers_may_write_tables = True


def shutdown() -> None:
  """release_all() and forget the process group (call before destroying it)."""
  global _ctx
  release_all()
  _ctx = None


def exchange_buffers(key, rp_size: int, coo: int, batch: int, dim: int):
  """Peer-visible staging buffers of one stacked table (allocated collectively on first use).

  `grad` holds max(batch, coo) rows: one reduced gradient row per slot when the sources exchange
  reduced runs, the plain activation gradients otherwise.
  """
  torch = _native.torch_mod()
  full_key = (key, rp_size, coo, batch, dim)
  buf = _ctx.exchange.get(full_key)
  if buf is None:
    buf = dict(rp=alloc((rp_size,), torch.int32), ids=alloc((coo,), torch.int32), sids=alloc((coo,), torch.int32),
               gains=alloc((coo,), torch.float32), grad=alloc((max(batch, coo), dim), torch.float32))
    buf["sources"] = (_native.PullSource * _ctx.world)()
    ptrs = {k: peer_pointers(buf[k]) for k in ("rp", "ids", "sids", "gains", "grad")}
    for r in range(_ctx.world):
      buf["sources"][r] = _native.PullSource(ptrs["rp"][r], ptrs["ids"][r], ptrs["sids"][r], ptrs["gains"][r],
                                             ptrs["grad"][r])
    _ctx.exchange[full_key] = buf
  return buf
