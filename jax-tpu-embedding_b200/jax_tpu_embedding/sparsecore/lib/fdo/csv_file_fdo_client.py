"""FDO client that stores statistics as .csv files (reference: lib/fdo/csv_file_fdo_client.py:38-216).

A file has the header `key,values` and one line per recorded observation: the key and the values
separated by blanks.  With `retain_history=False` the client keeps only the running maximum.
"""

from __future__ import annotations

import collections
import csv

import numpy as np

from jax_tpu_embedding.sparsecore.lib.fdo import _file_client


class CSVFileFDOClient(_file_client.FileFDOClient):
  extension = "csv"

  def __init__(self, base_dir, retain_history: bool = True):
    super().__init__(base_dir, retain_history=retain_history)

  def _write(self, path, arrays):
    with open(path, "w", newline="") as f:
      writer = csv.writer(f)
      writer.writerow(["key", "values"])
      for key, array in arrays.items():
        for row in np.atleast_2d(array.astype(np.int64)):
          writer.writerow([key, " ".join(str(int(v)) for v in row)])

  def _read(self, path):
    rows = collections.defaultdict(list)
    with open(path, "r", newline="") as f:
      reader = csv.reader(f)
      next(reader, None)
      for line in reader:
        if not line:
          continue
        key, values = line
        rows[key].append(np.array(values.split(), dtype=np.int64))
    return {key: (np.vstack(v) if len(v) > 1 else v[0]) for key, v in rows.items()}
