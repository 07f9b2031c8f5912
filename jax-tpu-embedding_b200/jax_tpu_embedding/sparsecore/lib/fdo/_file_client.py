"""Shared logic of the file-backed FDO clients; the storage format is the only difference.

Files are named `fdo_stats_<process>_<nanosecond timestamp>.<extension>`.  A file holds one array
per (table, statistic) under the key `<table><suffix>`, the suffix being the one declared on the
field of `embedding.SparseDenseMatmulInputStats`.  Recording twice stacks the observations as rows;
loading takes, per process, the newest file only and merges processes with an element-wise maximum
(jax_tpu_embedding/sparsecore/lib/fdo/file_fdo_client.py:65-213 of the reference).
"""

from __future__ import annotations

import dataclasses
import glob
import os
import re
import time

import numpy as np

from jax_tpu_embedding.sparsecore.lib.fdo import fdo_client
from jax_tpu_embedding.sparsecore.lib.nn import embedding

FILE_STEM = "fdo_stats"
FIELDS = dataclasses.fields(embedding.SparseDenseMatmulInputStats)
SUFFIXES = [f.metadata["suffix"] for f in FIELDS]


def process_index() -> int:
  """Rank of this process: torch.distributed if initialised, else $RANK, else 0."""
  try:
    import torch.distributed as dist  # pylint: disable=g-import-not-at-top

    if dist.is_available() and dist.is_initialized():
      return dist.get_rank()
  except ImportError:
    pass
  return int(os.environ.get("RANK", "0"))


class FileFDOClient(fdo_client.FDOClient):
  """Keeps {statistic: {table: array}} in memory; subclasses read and write one file."""

  extension = ""

  def __init__(self, base_dir, retain_history: bool = True):
    self._base_dir = os.fspath(base_dir)
    self._retain_history = retain_history
    self._params: dict[str, dict[str, np.ndarray]] = {f.name: {} for f in FIELDS}

  # -- storage format, provided by the subclass
  def _write(self, path: str, arrays: dict[str, np.ndarray]) -> None:
    raise NotImplementedError

  def _read(self, path: str) -> dict[str, np.ndarray]:
    raise NotImplementedError

  # -- FDOClient
  def record(self, data: embedding.SparseDenseMatmulInputStats) -> None:
    for name, per_table in dataclasses.asdict(data).items():
      store = self._params.get(name)
      if store is None:
        continue
      for table, value in per_table.items():
        value = np.asarray(value, dtype=np.int64)
        if table not in store:
          store[table] = value
        elif self._retain_history:
          store[table] = np.vstack((store[table], value))
        else:
          store[table] = np.maximum(store[table], value)

  def _generate_file_name(self) -> str:
    return os.path.join(self._base_dir, f"{FILE_STEM}_{process_index()}_{time.time_ns()}.{self.extension}")

  def _get_latest_files_by_process(self, files: list[str]) -> list[str]:
    """Newest file of every process, processes in descending order of their index string."""
    pattern = re.compile(rf"{FILE_STEM}_(\d+)_(\d+)\.{self.extension}$")
    newest: dict[str, tuple[int, str]] = {}
    for path in files:
      m = pattern.search(os.path.basename(path))
      if not m:
        continue
      proc, stamp = m.group(1), int(m.group(2))
      if proc not in newest or (stamp, path) > newest[proc]:
        newest[proc] = (stamp, path)
    return [newest[proc][1] for proc in sorted(newest, reverse=True)]

  def publish(self) -> None:
    arrays = {}
    for field in FIELDS:
      for table, value in self._params[field.name].items():
        arrays[f"{table}{field.metadata['suffix']}"] = np.asarray(value)
    os.makedirs(self._base_dir, exist_ok=True)
    self._write(self._generate_file_name(), arrays)

  def load(self) -> embedding.SparseDenseMatmulInputStats:
    pattern = os.path.join(self._base_dir, f"{FILE_STEM}*.{self.extension}")
    files = self._get_latest_files_by_process(glob.glob(pattern))
    if not files:
      raise FileNotFoundError(f"No stats files found in {pattern}")
    merged: dict[str, np.ndarray] = {}
    for path in files:
      for key, value in self._read(path).items():
        merged[key] = value if key not in merged else np.max(np.vstack((merged[key], value)), axis=0)
    result: dict[str, dict[str, np.ndarray]] = {f.name: {} for f in FIELDS}
    for key, value in merged.items():
      for field in FIELDS:
        suffix = field.metadata["suffix"]
        if key.endswith(suffix):
          result[field.name][key[:-len(suffix)]] = value
          break
      else:
        raise ValueError(f"Unexpected key: {key}, expected to end with {SUFFIXES}")
    self._params = result
    return embedding.SparseDenseMatmulInputStats(**result)
