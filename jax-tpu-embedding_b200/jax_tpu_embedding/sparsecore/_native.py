"""ctypes binding of libsc_b200.so (the C ABI declared in include/sc_b200.h).

There is no CPU fallback: if the shared library is missing, every operator raises
`RuntimeError`.  PyTorch is used for device memory, streams and host<->device
copies only.
"""

from __future__ import annotations

import ctypes
import os
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# SC_B200_LIBRARY selects another build of the library (kernel tuning experiments).
LIB_PATH = os.environ.get("SC_B200_LIBRARY") or os.path.join(_HERE, "libsc_b200.so")

SC_OK = 0
SC_INVALID_ARGUMENT = 1
SC_WORKSPACE_TOO_SMALL = 2
SC_ID_LIMIT_EXCEEDED = 3
SC_CUDA_ERROR = 4
SC_UNSUPPORTED = 5
SC_MAX_SHARDS = 64

COMBINERS = {"sum": 0, "mean": 1, "sqrtn": 2}

c_i32, c_i64, c_f32, c_vp, c_sz = (ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t)


class FeatureDesc(ctypes.Structure):
  _fields_ = [("row_begin", c_i32), ("rows", c_i32), ("row_offset", c_i32), ("col_offset", c_i32),
              ("col_shift", c_i32), ("valency", c_i32), ("id_begin", c_i32)]


class PreprocessOptions(ctypes.Structure):
  _fields_ = [("global_device_count", c_i32), ("num_sc_per_device", c_i32), ("combiner", c_i32),
              ("max_ids_per_partition", c_i32), ("max_unique_ids_per_partition", c_i32),
              ("allow_id_dropping", c_i32), ("coo_buffer_size_per_device", c_i32), ("stack_vocab_size", c_i32)]


class PreprocessItem(ctypes.Structure):
  _fields_ = [("ids", c_vp), ("row_offsets", c_vp), ("weights", c_vp), ("nnz", c_i64), ("total_rows", c_i64),
              ("features", ctypes.POINTER(FeatureDesc)), ("num_features", c_i32), ("options", PreprocessOptions),
              ("row_pointers", c_vp), ("embedding_ids", c_vp), ("sample_ids", c_vp), ("gains", c_vp), ("stats", c_vp),
              ("plan_slots", c_vp), ("plan_bags", c_vp)]


class Csr(ctypes.Structure):
  _fields_ = [("row_pointers", c_vp), ("embedding_ids", c_vp), ("sample_ids", c_vp), ("gains", c_vp),
              ("coo_buffer_size", c_i32), ("num_sc_per_device", c_i32), ("num_scs", c_i32),
              ("device_batch_size", c_i32), ("dim", c_i32), ("max_ids_per_sample", c_i32),
              ("rows_per_shard", c_i64)]


class Optimizer(ctypes.Structure):
  _fields_ = [("optimizer", c_i32), ("hyper", c_f32 * 8), ("clip_min", c_f32), ("clip_max", c_f32)]


class FwdItem(ctypes.Structure):
  _fields_ = [("csr", Csr), ("shard_tables", ctypes.POINTER(c_vp)), ("activations", c_vp), ("local_shard", ctypes.c_int32),
              ("plan_slots", c_vp), ("plan_bags", c_vp)]


class PullSource(ctypes.Structure):
  _fields_ = [("row_pointers", c_vp), ("embedding_ids", c_vp), ("sample_ids", c_vp), ("gains", c_vp),
              ("activation_grad", c_vp)]


class GradItem(ctypes.Structure):
  _fields_ = [("csr", Csr), ("activation_grad", c_vp), ("shard_tables", ctypes.POINTER(c_vp)),
              ("shard_slot0", ctypes.POINTER(c_vp)), ("shard_slot1", ctypes.POINTER(c_vp)), ("optimizer", Optimizer),
              ("sources", ctypes.POINTER(PullSource)), ("num_sources", c_i32), ("shard", c_i32),
              ("partition_capacity", c_i32)]


_lib = None
_lock = threading.Lock()


def available() -> bool:
  return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
  """Loads the library once; fails loudly when it has not been built."""
  global _lib
  if _lib is not None:
    return _lib
  with _lock:
    if _lib is not None:
      return _lib
    if not os.path.exists(LIB_PATH):
      raise RuntimeError(
          f"{LIB_PATH} is missing: build it with `python jax-tpu-embedding_b200/csrc/build.py`. "
          "The SparseCore operators have no CPU fallback.")
    l = ctypes.CDLL(LIB_PATH)
    l.sc_version.restype = c_i32
    l.sc_launch_count.restype = c_i64
    l.sc_status_name.restype = ctypes.c_char_p
    l.sc_status_name.argtypes = [c_i32]
    l.sc_last_error.restype = c_i32
    l.sc_last_error.argtypes = [ctypes.c_char_p, c_i32]
    l.sc_phase_timing.restype = c_i32
    l.sc_phase_timing.argtypes = [c_i32]
    l.sc_phase_report.restype = c_i32
    l.sc_phase_report.argtypes = [ctypes.c_char_p, c_i32]
    l.sc_compute_theoretical_max_coo_buffer_size.restype = c_i64
    l.sc_compute_theoretical_max_coo_buffer_size.argtypes = [c_i32, c_i32, c_i32]
    l.sc_compute_coo_buffer_size_per_device.restype = c_i64
    l.sc_compute_coo_buffer_size_per_device.argtypes = [c_i32, c_i32, c_i32, c_i64]
    l.sc_compute_row_pointers_size_per_device.restype = c_i32
    l.sc_compute_row_pointers_size_per_device.argtypes = [c_i32, c_i32]
    l.sc_preprocess_stats_size.restype = c_i32
    l.sc_preprocess_stats_size.argtypes = [c_i32, c_i32]
    l.sc_preprocess_workspace_bytes.restype = c_sz
    l.sc_preprocess_workspace_bytes.argtypes = [c_i64, c_i64, ctypes.POINTER(PreprocessOptions)]
    l.sc_preprocess_table.restype = c_i32
    l.sc_preprocess_table.argtypes = [c_vp, c_vp, c_vp, c_i64, c_i64, ctypes.POINTER(FeatureDesc), c_i32,
                                      ctypes.POINTER(PreprocessOptions), c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]
    l.sc_preprocess_grouped_workspace_bytes.restype = c_sz
    l.sc_preprocess_grouped_workspace_bytes.argtypes = [ctypes.POINTER(PreprocessItem), c_i32]
    l.sc_preprocess_grouped.restype = c_i32
    l.sc_preprocess_grouped.argtypes = [ctypes.POINTER(PreprocessItem), c_i32, c_vp, c_sz, c_vp]
    l.sc_sparse_dense_matmul_fwd_workspace_bytes.restype = c_sz
    l.sc_sparse_dense_matmul_fwd_workspace_bytes.argtypes = [ctypes.POINTER(Csr)]
    l.sc_sparse_dense_matmul_fwd.restype = c_i32
    l.sc_sparse_dense_matmul_fwd.argtypes = [ctypes.POINTER(Csr), ctypes.POINTER(c_vp), c_vp, c_vp, c_sz, c_vp]
    l.sc_sparse_dense_matmul_grad_workspace_bytes.restype = c_sz
    l.sc_sparse_dense_matmul_grad_workspace_bytes.argtypes = [ctypes.POINTER(Csr)]
    l.sc_sparse_dense_matmul_grad.restype = c_i32
    l.sc_sparse_dense_matmul_grad.argtypes = [ctypes.POINTER(Csr), c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp),
                                              ctypes.POINTER(c_vp), ctypes.POINTER(Optimizer), c_vp, c_sz, c_vp]
    l.sc_sparse_dense_matmul_fwd_grouped_workspace_bytes.restype = c_sz
    l.sc_sparse_dense_matmul_fwd_grouped_workspace_bytes.argtypes = [ctypes.POINTER(FwdItem), c_i32]
    l.sc_sparse_dense_matmul_fwd_grouped.restype = c_i32
    l.sc_sparse_dense_matmul_fwd_grouped.argtypes = [ctypes.POINTER(FwdItem), c_i32, c_vp, c_sz, c_vp]
    l.sc_sparse_dense_matmul_grad_grouped_workspace_bytes.restype = c_sz
    l.sc_sparse_dense_matmul_grad_grouped_workspace_bytes.argtypes = [ctypes.POINTER(GradItem), c_i32]
    l.sc_sparse_dense_matmul_grad_grouped.restype = c_i32
    l.sc_sparse_dense_matmul_grad_grouped.argtypes = [ctypes.POINTER(GradItem), c_i32, c_vp, c_sz, c_vp]
    l.sc_sparse_dense_matmul_grad_stage_workspace_bytes.restype = c_sz
    l.sc_sparse_dense_matmul_grad_stage_workspace_bytes.argtypes = [ctypes.POINTER(GradItem), c_i32]
    l.sc_sparse_dense_matmul_grad_stage.restype = c_i32
    l.sc_sparse_dense_matmul_grad_stage.argtypes = [ctypes.POINTER(GradItem), c_i32, c_vp, c_sz, c_vp]
    l.sc_peer_alloc.restype = c_i32
    l.sc_peer_alloc.argtypes = [c_sz, ctypes.POINTER(c_vp)]
    l.sc_peer_free.restype = c_i32
    l.sc_peer_free.argtypes = [c_vp]
    l.sc_ipc_export.restype = c_i32
    l.sc_ipc_export.argtypes = [c_vp, ctypes.c_char_p]
    l.sc_ipc_import.restype = c_i32
    l.sc_ipc_import.argtypes = [ctypes.c_char_p, ctypes.POINTER(c_vp)]
    l.sc_ipc_release.restype = c_i32
    l.sc_ipc_release.argtypes = [c_vp]
    l.sc_sparse_dense_matmul_grad_static.restype = c_i32
    l.sc_sparse_dense_matmul_grad_static.argtypes = [ctypes.POINTER(Csr), c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp),
                                                     ctypes.POINTER(c_vp), ctypes.POINTER(Optimizer), c_vp]
    _lib = l
  return _lib


def last_error() -> str:
  buf = ctypes.create_string_buffer(512)
  lib().sc_last_error(buf, 512)
  return buf.value.decode("utf-8", "replace")


def phase_timing(enable: bool) -> None:
  """Starts (and clears) or stops the per-stage CUDA-event timing of the library."""
  lib().sc_phase_timing(1 if enable else 0)


def phase_report() -> dict:
  """{stage name: (total milliseconds, count)} since phase_timing(True); clears the records."""
  buf = ctypes.create_string_buffer(8192)
  check(lib().sc_phase_report(buf, 8192))
  out = {}
  for item in buf.value.decode().split(";"):
    if "=" in item:
      name, rest = item.split("=")
      ms, count = rest.split("/")
      out[name] = (float(ms), int(count))
  return out


def check(status: int) -> None:
  """Raises ValueError for invalid arguments / id-limit violations, RuntimeError otherwise."""
  if status == SC_OK:
    return
  msg = last_error() or lib().sc_status_name(status).decode()
  if status in (SC_INVALID_ARGUMENT, SC_ID_LIMIT_EXCEEDED):
    raise ValueError(msg)
  raise RuntimeError(f"sc_b200 {lib().sc_status_name(status).decode()}: {msg}")


# ---------------------------------------------------------------------------- torch plumbing


def torch_mod():
  import torch  # pylint: disable=g-import-not-at-top

  return torch


def require_cuda():
  torch = torch_mod()
  if not torch.cuda.is_available():
    raise RuntimeError("The SparseCore operators need a CUDA device (NVIDIA B200); there is no CPU fallback.")
  return torch


def current_stream_ptr() -> int:
  return int(torch_mod().cuda.current_stream().cuda_stream)


_workspaces: dict = {}


def workspace(nbytes: int, tag: str = "default"):
  """A cached uint8 device buffer of at least `nbytes` for (device, stream, tag)."""
  torch = torch_mod()
  key = (torch.cuda.current_device(), current_stream_ptr(), tag)
  buf = _workspaces.get(key)
  if buf is None or buf.numel() < nbytes:
    buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device="cuda")
    _workspaces[key] = buf
  return buf


def clear_workspaces() -> None:
  """Drops the cached workspace buffers (they are re-created on demand)."""
  _workspaces.clear()


def as_device(x, dtype, name: str):
  """numpy / torch input -> contiguous CUDA tensor of `dtype` on the current device."""
  torch = torch_mod()
  if isinstance(x, torch.Tensor):
    if x.dtype != dtype:
      raise ValueError(f"{name} must have type {dtype}, got {x.dtype}")
    if not x.is_cuda:
      x = x.cuda(non_blocking=True)
    return x.contiguous()
  arr = np.asarray(x)
  want = {torch.int32: np.int32, torch.float32: np.float32}[dtype]
  if arr.dtype != want:
    raise ValueError(f"{name} must have type {np.dtype(want)!r}, got {arr.dtype!r}")
  return torch.from_numpy(np.ascontiguousarray(arr)).cuda(non_blocking=True)


def ptr_array(tensors):
  """Host array of device pointers for the shards of a table (or of a slot variable)."""
  arr = (c_vp * len(tensors))()
  for i, t in enumerate(tensors):
    arr[i] = t.data_ptr()
  return arr
