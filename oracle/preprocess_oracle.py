"""ctypes front end of the C preprocessing oracle (test infrastructure).

TEST INFRASTRUCTURE - NOT THE PRODUCT.  Only tests, the smoke test and the CPU
baseline leg of the benchmark may import this module.  Parity status: pinned
(see the header of ``sc_oracle.c``).
"""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Sequence

import numpy as np

from . import build as _build

PADDING_VALUE = 2**31 - 1
COMBINERS = {"sum": 0, "mean": 1, "sqrtn": 2}

OK = 0
INVALID_ARGUMENT = 1
ID_LIMIT_EXCEEDED = 3


class _Feature(ctypes.Structure):
  _fields_ = [
      ("ids", ctypes.c_void_p),
      ("offsets", ctypes.c_void_p),
      ("weights", ctypes.c_void_p),
      ("rows", ctypes.c_int64),
      ("row_offset", ctypes.c_int32),
      ("col_offset", ctypes.c_int32),
      ("col_shift", ctypes.c_int32),
  ]


class _Options(ctypes.Structure):
  _fields_ = [
      ("local_device_count", ctypes.c_int32),
      ("global_device_count", ctypes.c_int32),
      ("num_sc_per_device", ctypes.c_int32),
      ("combiner", ctypes.c_int32),
      ("has_weights", ctypes.c_int32),
      ("max_ids_per_partition", ctypes.c_int32),
      ("max_unique_ids_per_partition", ctypes.c_int32),
      ("allow_id_dropping", ctypes.c_int32),
      ("coo_buffer_size_per_device", ctypes.c_int32),
      ("num_threads", ctypes.c_int32),
  ]


_lib = None


def lib() -> ctypes.CDLL:
  global _lib
  if _lib is None:
    _lib = ctypes.CDLL(_build.build())
    _lib.sc_oracle_coo_buffer_size.restype = ctypes.c_int64
    _lib.sc_oracle_coo_buffer_size.argtypes = [
        ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64]
    _lib.sc_oracle_preprocess_table.restype = ctypes.c_int
  return _lib


@dataclasses.dataclass
class FeatureInput:
  """One feature of a stack as a CSR view of the rows this process holds."""

  ids: np.ndarray  # int32 [nnz]
  offsets: np.ndarray  # int64 [rows + 1]
  weights: np.ndarray | None  # float32 [nnz] or None
  row_offset: int = 0
  col_offset: int = 0
  col_shift: int = 0

  @property
  def rows(self) -> int:
    return len(self.offsets) - 1


def flatten_feature(feature, weights=None):
  """Dense [B, v] or ragged (object array / list of 1-D arrays) -> (ids, offsets, weights)."""
  if isinstance(feature, np.ndarray) and feature.dtype != object and feature.ndim == 2:
    b, v = feature.shape
    ids = np.ascontiguousarray(feature, dtype=np.int32).reshape(-1)
    offsets = np.arange(b + 1, dtype=np.int64) * v
    w = None
    if weights is not None:
      w = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
    return ids, offsets, w
  rows = [np.asarray(r, dtype=np.int32).reshape(-1) for r in feature]
  lens = np.fromiter((len(r) for r in rows), dtype=np.int64, count=len(rows))
  offsets = np.zeros(len(rows) + 1, dtype=np.int64)
  np.cumsum(lens, out=offsets[1:])
  ids = np.concatenate(rows) if rows else np.zeros(0, np.int32)
  ids = np.ascontiguousarray(ids, dtype=np.int32)
  w = None
  if weights is not None:
    wr = [np.asarray(r, dtype=np.float32).reshape(-1) for r in weights]
    w = np.concatenate(wr) if wr else np.zeros(0, np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
  return ids, offsets, w


def coo_buffer_size(max_ids_per_partition, global_device_count, num_sc_per_device, suggested=None) -> int:
  v = lib().sc_oracle_coo_buffer_size(
      int(max_ids_per_partition), int(global_device_count), int(num_sc_per_device),
      -1 if suggested is None else int(suggested))
  if v < 0:
    raise ValueError("coo buffer size out of range or above the theoretical maximum")
  return int(v)


def row_pointers_size(global_device_count, num_sc_per_device) -> int:
  return max(global_device_count * num_sc_per_device, 8) * num_sc_per_device


def preprocess_table(
    features: Sequence[FeatureInput],
    *,
    local_device_count: int,
    global_device_count: int,
    num_sc_per_device: int,
    combiner: str = "sum",
    max_ids_per_partition: int = 256,
    max_unique_ids_per_partition: int = 256,
    allow_id_dropping: bool = False,
    suggested_coo_buffer_size_per_device: int | None = None,
    num_threads: int = 1,
):
  """Runs the oracle for one stacked table; returns a dict of numpy arrays.

  ``features`` must be ordered by ``row_offset``.  Slots the reference never
  writes keep the prefill (PADDING_VALUE / NaN).
  """
  feats = sorted(features, key=lambda f: f.row_offset)
  has_weights = any(f.weights is not None for f in feats)
  coo = coo_buffer_size(max_ids_per_partition, global_device_count, num_sc_per_device,
                        suggested_coo_buffer_size_per_device)
  L, S = local_device_count, num_sc_per_device
  P = S * global_device_count
  R = max(P, 8)
  arr = (_Feature * len(feats))()
  keep = []
  for i, f in enumerate(feats):
    ids = np.ascontiguousarray(f.ids, dtype=np.int32)
    off = np.ascontiguousarray(f.offsets, dtype=np.int64)
    w = None if f.weights is None else np.ascontiguousarray(f.weights, dtype=np.float32)
    if has_weights and w is None:
      w = np.ones(len(ids), np.float32)
    keep += [ids, off, w]
    arr[i].ids = ids.ctypes.data
    arr[i].offsets = off.ctypes.data
    arr[i].weights = None if w is None else w.ctypes.data
    arr[i].rows = len(off) - 1
    arr[i].row_offset = int(f.row_offset)
    arr[i].col_offset = int(f.col_offset)
    arr[i].col_shift = int(f.col_shift)
  opt = _Options(L, global_device_count, S, COMBINERS.get(combiner, 0), int(has_weights),
                 int(max_ids_per_partition), int(max_unique_ids_per_partition),
                 int(allow_id_dropping), coo, int(num_threads))
  row_pointers = np.zeros((L, R * S), np.int32)
  embedding_ids = np.full((L, coo), PADDING_VALUE, np.int32)
  sample_ids = np.full((L, coo), PADDING_VALUE, np.int32)
  gains = np.full((L, coo), np.nan, np.float32)
  max_ids = np.zeros(L * P, np.int32)
  max_unique = np.zeros(L * P, np.int32)
  required = np.zeros(L * S, np.int32)
  dropped = ctypes.c_int64(0)
  status = lib().sc_oracle_preprocess_table(
      arr, ctypes.c_int(len(feats)), ctypes.byref(opt),
      ctypes.c_void_p(row_pointers.ctypes.data), ctypes.c_void_p(embedding_ids.ctypes.data),
      ctypes.c_void_p(sample_ids.ctypes.data), ctypes.c_void_p(gains.ctypes.data),
      ctypes.c_void_p(max_ids.ctypes.data), ctypes.c_void_p(max_unique.ctypes.data),
      ctypes.c_void_p(required.ctypes.data), ctypes.byref(dropped))
  del keep
  return dict(
      status=int(status), row_pointers=row_pointers, embedding_ids=embedding_ids,
      sample_ids=sample_ids, gains=gains, max_ids_per_partition=max_ids,
      max_unique_ids_per_partition=max_unique, required_buffer_sizes=required,
      dropped_id_count=int(dropped.value), coo_buffer_size_per_device=coo)
