"""Table and slot-variable initializers that fill device memory in place.

The reference takes `jax.nn.initializers` callables `(key, shape) -> array`
(jax_tpu_embedding/sparsecore/lib/nn/embedding_spec.py:45-51).  Here an
initializer is any callable `(rng, shape, device=None) -> torch.Tensor`, with
`rng` a `torch.Generator` (or None for the global generator).  Tables can be tens
of GB, so the built-in ones generate directly on the target device.
"""

from __future__ import annotations

import torch


def _gen(rng, device):
  if rng is None or isinstance(rng, torch.Generator):
    return rng
  g = torch.Generator(device=device if device is not None else "cpu")
  g.manual_seed(int(rng))
  return g


def constant(value: float):
  def init(rng, shape, device=None):
    del rng
    return torch.full(tuple(shape), float(value), dtype=torch.float32, device=device)

  return init


def zeros():
  return constant(0.0)


def normal(stddev: float = 1e-2, mean: float = 0.0):
  def init(rng, shape, device=None):
    out = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    return out.normal_(mean, stddev, generator=_gen(rng, out.device))

  return init


def uniform(low: float = 0.0, high: float = 1.0):
  def init(rng, shape, device=None):
    out = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    return out.uniform_(low, high, generator=_gen(rng, out.device))

  return init


def truncated_normal(stddev: float = 1e-2, lower: float = -2.0, upper: float = 2.0):
  def init(rng, shape, device=None):
    out = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    torch.nn.init.trunc_normal_(out, 0.0, stddev, lower * stddev, upper * stddev,
                                generator=_gen(rng, out.device))
    return out

  return init
