"""FDO client that stores statistics as .npz files (reference: lib/fdo/file_fdo_client.py:37-213)."""

from __future__ import annotations

import numpy as np

from jax_tpu_embedding.sparsecore.lib.fdo import _file_client


class NPZFileFDOClient(_file_client.FileFDOClient):
  """`fdo_stats_<process>_<time>.npz`, one array per key.  Every `record` adds a row."""

  extension = "npz"

  def __init__(self, base_dir):
    super().__init__(base_dir, retain_history=True)

  def _write(self, path, arrays):
    np.savez(path, **arrays)

  def _read(self, path):
    with np.load(path) as data:
      return {key: data[key] for key in data.files}
