"""Interface of an FDO (feedback-directed optimisation) client.

One client per process.  `record` keeps the statistics of a preprocessing call in memory,
`publish` writes what was recorded to shared storage, `load` reads what every process published
and returns the element-wise maximum.  Mirrors `FDOClient` of the reference
(jax_tpu_embedding/sparsecore/lib/fdo/fdo_client.py:21-83).
"""

from __future__ import annotations

import abc

from jax_tpu_embedding.sparsecore.lib.nn import embedding


class FDOClient(abc.ABC):
  """record() -> (train a few steps) -> publish() -> load() -> embedding.update_preprocessing_parameters()."""

  @abc.abstractmethod
  def record(self, data: embedding.SparseDenseMatmulInputStats) -> None:
    """Keeps the statistics of one preprocessing call in process-local memory."""
    raise NotImplementedError

  @abc.abstractmethod
  def publish(self) -> None:
    """Writes everything recorded so far to the storage location."""
    raise NotImplementedError

  @abc.abstractmethod
  def load(self) -> embedding.SparseDenseMatmulInputStats:
    """Reads the latest publication of every process and aggregates them (maximum per element)."""
    raise NotImplementedError
