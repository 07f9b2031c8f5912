"""Table sharding helpers and the shards-per-device map.

Mirrors jax_tpu_embedding/sparsecore/utils/utils.py of the reference
(`NUM_SC_PER_DEVICE_MAP` :30-36, `num_sparsecores_per_device` :48-77,
`shard_emb_table` :90-113, `unshard_emb_table` :116-136).  On B200 one GPU owns
exactly one table shard, so the map gains the entry ``'NVIDIA B200': 1``; 2 and 4
stay legal as *virtual* SparseCores so that buffers laid out for TPUs can be
replayed.  The TPU tiled-layout helpers (`embedding_table_format*`) have no GPU
counterpart: tables are plain row-major float32 in HBM.
"""

from __future__ import annotations

import typing

import numpy as np

NUM_SC_PER_DEVICE_MAP = {
    "TPU v5": 4,
    "TPU v5p": 4,
    "TPU v6e": 2,
    "TPU v6 lite": 2,
    "TPU7x": 2,
    "NVIDIA B200": 1,
}


class DeviceLike(typing.Protocol):

  @property
  def device_kind(self) -> str:
    ...


def num_sparsecores_per_device(device: DeviceLike | None = None) -> int:
  """Number of table shards served by one device (1 on B200)."""
  if device is None:
    import torch  # pylint: disable=g-import-not-at-top

    if not torch.cuda.is_available():
      # No accelerator visible: host-side spec work defaults to the B200 value.
      return NUM_SC_PER_DEVICE_MAP["NVIDIA B200"]
    kind = torch.cuda.get_device_name(torch.cuda.current_device())
  else:
    if not hasattr(device, "device_kind"):
      raise ValueError(f"Cannot determine device kind for device: {device}")
    kind = device.device_kind
  if kind not in NUM_SC_PER_DEVICE_MAP:
    raise ValueError(
        f"Unknown sparsecore count for device kind: {kind}. Known"
        f" device kinds: {NUM_SC_PER_DEVICE_MAP.keys()}")
  return NUM_SC_PER_DEVICE_MAP[kind]


def _is_torch(x) -> bool:
  return type(x).__module__.startswith("torch")


def shard_emb_table(table, *, num_devices: int, num_sc_per_device: int, sharding_strategy: str = "MOD"):
  """[V, ...] -> [num_devices, num_sc_per_device * V / num_scs, ...] ('(v c s) -> c (s v)')."""
  if sharding_strategy != "MOD":
    raise ValueError("Currently only MOD sharding strategy is supported")
  c, s = num_devices, num_sc_per_device
  if not _is_torch(table):
    table = np.asarray(table)
  rest = tuple(table.shape[1:])
  v = table.shape[0] // (c * s)
  x = table.reshape((v, c, s) + rest)
  if _is_torch(x):
    x = x.permute(1, 2, 0, *range(3, x.dim())).contiguous()
  else:
    x = np.ascontiguousarray(np.moveaxis(x, 0, 2))
  return x.reshape((c, s * v) + rest)


def unshard_emb_table(sharded_table, num_sc_per_device: int, sharding_strategy: str = "MOD"):
  """Inverse of `shard_emb_table` ('c (s v) -> (v c s)')."""
  if sharding_strategy != "MOD":
    raise ValueError("Currently only MOD sharding strategy is supported")
  s = num_sc_per_device
  if not _is_torch(sharded_table):
    sharded_table = np.asarray(sharded_table)
  c = sharded_table.shape[0]
  rest = tuple(sharded_table.shape[2:])
  v = sharded_table.shape[1] // s
  x = sharded_table.reshape((c, s, v) + rest)
  if _is_torch(x):
    x = x.permute(2, 0, 1, *range(3, x.dim())).contiguous()
  else:
    x = np.ascontiguousarray(np.moveaxis(x, 2, 0))
  return x.reshape((v * c * s,) + rest)
