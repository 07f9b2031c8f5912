"""Stacking of several tables into one mod-sharded lookup unit.

Spec arithmetic and value layout follow the reference's
jax_tpu_embedding/sparsecore/lib/nn/table_stacking.py: padding rules
(`round_up_dim_and_vocab_size` :355-378), grouping for automatic stacking
(:381-498), per-table placement (`compute_table_to_setting_in_stack` :570-613),
feature transformations (`_stack_feature_specs` :648-754), `stack_tables` :792,
`auto_stack_tables` :897, value stacking (`stack_and_shard_tables` :144-221,
`unshard_and_unstack_tables` :288-310) and `compute_physical_row_ids` :1229-1255.
The proto-driven variants of the reference (checkpoint tooling) are not part of
the lookup path and are not provided.

A stacked table is stored as [num_shards, rows_per_shard, dim]: shard `g` holds,
for every member table, the rows `i` with `(i % num_shards + rotation) % num_shards
== g`, at local row `row_offset_in_shard + i // num_shards`.
"""

from __future__ import annotations

import collections
import hashlib
import logging
from typing import Callable, Mapping, Sequence

import numpy as np

from jax_tpu_embedding.sparsecore import _tree
from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec

TableSpec = embedding_spec.TableSpec
StackedTableSpec = embedding_spec.StackedTableSpec
LimitsCallable = Callable[[str, int], int]
DEFAULT_ACTIVATION_MEM_BYTES_LIMIT = embedding_spec.DEFAULT_ACTIVATION_MEM_BYTES_LIMIT

_log = logging.getLogger(__name__)


def _ceil_to(value: int, multiple: int) -> int:
  return -(-value // multiple) * multiple


def _is_torch(x) -> bool:
  return type(x).__module__.startswith("torch")


def get_default_limits(name: str, batch_size: int) -> int:
  del name, batch_size
  return 256


def round_up_dim_and_vocab_size(tables: Mapping[str, TableSpec], num_sc: int):
  """dim -> multiple of 8, vocabulary -> multiple of 8 * num_sc."""
  dims = {n: _ceil_to(t.embedding_dim, 8) for n, t in tables.items()}
  vocabs = {n: _ceil_to(t.vocabulary_size, 8 * num_sc) for n, t in tables.items()}
  return dims, vocabs


# --------------------------------------------------------------------------- values


def _stack_spec_of(table_spec: TableSpec, num_shards: int) -> StackedTableSpec:
  if table_spec.is_stacked():
    return table_spec.stacked_table_spec
  return StackedTableSpec(
      stack_name=table_spec.name,
      stack_vocab_size=_ceil_to(table_spec.vocabulary_size, 8 * num_shards),
      stack_embedding_dim=_ceil_to(table_spec.embedding_dim, 8),
      optimizer=table_spec.optimizer,
      combiner=table_spec.combiner,
      total_sample_count=0,
      max_ids_per_partition=table_spec.max_ids_per_partition,
      max_unique_ids_per_partition=table_spec.max_unique_ids_per_partition,
      quantization_config=table_spec.quantization_config,
  )


def _place_table(stacked, table_spec: TableSpec, values, num_shards: int, pad_value: float):
  """Writes one table into its slot of `stacked` ([shards, rows, dim], in place)."""
  xp_torch = _is_torch(stacked)
  dim = stacked.shape[-1]
  vocab, emb = table_spec.vocabulary_size, table_spec.embedding_dim
  padded_vocab = _ceil_to(vocab, 8 * num_shards)
  rows = padded_vocab // num_shards
  setting = table_spec.setting_in_stack
  if xp_torch:
    import torch  # pylint: disable=g-import-not-at-top

    padded = torch.full((padded_vocab, dim), float(pad_value), dtype=torch.float32, device=stacked.device)
    padded[:vocab, :emb] = torch.as_tensor(values, dtype=torch.float32, device=stacked.device)
    sharded = padded.reshape(rows, num_shards, dim).transpose(0, 1)
    sharded = torch.roll(sharded, setting.shard_rotation, dims=0)
  else:
    padded = np.full((padded_vocab, dim), pad_value, dtype=np.float32)
    padded[:vocab, :emb] = np.asarray(values, dtype=np.float32)
    sharded = np.roll(padded.reshape(rows, num_shards, dim).swapaxes(0, 1), setting.shard_rotation, axis=0)
  r0 = setting.row_offset_in_shard
  stacked[:, r0:r0 + rows, :] = sharded


def stack_and_shard_tables(table_specs, tables, num_shards: int, pad_value: float = float("nan")):
  """Unstacked table values -> {stack name: [num_shards, rows_per_shard, dim]}.

  `tables` mirrors `table_specs`; a leaf may itself be a tuple of arrays (table
  plus slot variables), in which case every member is stacked the same way.
  """
  spec_leaves = _tree.leaves(table_specs)
  value_leaves = _flatten_up_to(table_specs, tables)
  groups: dict[str, tuple[StackedTableSpec, list[tuple[TableSpec, object]]]] = {}
  for spec, value in zip(spec_leaves, value_leaves):
    stack = _stack_spec_of(spec, num_shards)
    groups.setdefault(stack.stack_name, (stack, []))[1].append((spec, value))

  out = {}
  for stack, members in groups.values():
    rows = stack.stack_vocab_size // num_shards
    dim = stack.stack_embedding_dim
    first_value = members[0][1]

    def new_buffer(like):
      if _is_torch(like):
        import torch  # pylint: disable=g-import-not-at-top

        return torch.zeros((num_shards, rows, dim), dtype=torch.float32, device=like.device)
      return np.zeros((num_shards, rows, dim), dtype=np.float32)

    stacked_tree = _tree.tree_map(new_buffer, first_value)
    for spec, value in members:
      _tree.tree_map(
          lambda buf, v, spec=spec: _place_table(buf, spec, v, num_shards, pad_value), stacked_tree, value)
    out[stack.stack_name] = stacked_tree
  return out


def _flatten_up_to(spec_tree, value_tree):
  """Values aligned with the TableSpec leaves; a value may be a nested container."""
  out = []

  def go(s, v):
    if isinstance(s, TableSpec):
      out.append(v)
      return
    if isinstance(s, dict):
      for k in sorted(s):
        go(s[k], v[k])
    elif isinstance(s, (list, tuple)):
      for a, b in zip(s, v):
        go(a, b)
    elif s is None:
      return
    else:
      raise ValueError(f"unexpected node in table spec tree: {type(s)}")

  go(spec_tree, value_tree)
  return out


def _extract_table(stacked, table_spec: TableSpec, num_shards: int):
  stacked = stacked.reshape(num_shards, -1, stacked.shape[-1])
  dim = stacked.shape[-1]
  rows = _ceil_to(table_spec.vocabulary_size, 8 * num_shards) // num_shards
  setting = table_spec.setting_in_stack
  block = stacked[:, setting.row_offset_in_shard:setting.row_offset_in_shard + rows, :]
  if _is_torch(block):
    import torch  # pylint: disable=g-import-not-at-top

    block = torch.roll(block, -setting.shard_rotation, dims=0).transpose(0, 1).reshape(-1, dim)
  else:
    block = np.roll(block, -setting.shard_rotation, axis=0).swapaxes(0, 1).reshape(-1, dim)
  return block[:table_spec.vocabulary_size, :table_spec.embedding_dim]


def unshard_and_unstack_tables(table_specs, stacked_tables: Mapping[str, object], num_shards: int):
  """Inverse of `stack_and_shard_tables`; returns a tree shaped like `table_specs`."""

  def one(spec: TableSpec):
    name = spec.stacked_table_spec.stack_name if spec.is_stacked() else spec.name
    return _tree.tree_map(lambda s: _extract_table(s, spec, num_shards), stacked_tables[name])

  return _tree.tree_map(one, table_specs)


def get_table_stacks(table_specs) -> dict[str, list[TableSpec]]:
  stacks: dict[str, list[TableSpec]] = collections.defaultdict(list)
  for spec in _tree.leaves(table_specs):
    name = spec.stacked_table_spec.stack_name if spec.is_stacked() else spec.name
    stacks[name].append(spec)
  return stacks


def compute_physical_row_ids(num_sparse_cores: int, stack_vocab_size: int, shard_rotation: int,
                             row_offset_in_shard: int, row_ids):
  """Row index inside the flattened [num_shards * rows_per_shard] stack buffer."""
  shard_size = stack_vocab_size // num_sparse_cores
  shard = (row_ids % num_sparse_cores + shard_rotation) % num_sparse_cores
  return shard * shard_size + row_ids // num_sparse_cores + row_offset_in_shard


# --------------------------------------------------------------------------- specs


def compute_table_to_setting_in_stack(stack_name: str, table_names: Sequence[str], padded_embedding_dim: int,
                                      table_to_padded_vocab_size: Mapping[str, int], num_shards: int,
                                      rotation: int) -> Mapping[str, embedding_spec.TableSettingInStack]:
  """Cumulative row offsets per shard; rotation advances by `rotation` per table."""
  settings = {}
  row_offset, shard_rotation = 0, 0
  for name in table_names:
    if name not in table_to_padded_vocab_size:
      raise ValueError(f"Padded vocab size for Table {name} is missing.")
    settings[name] = embedding_spec.TableSettingInStack(
        stack_name=stack_name,
        padded_vocab_size=table_to_padded_vocab_size[name],
        padded_embedding_dim=padded_embedding_dim,
        row_offset_in_shard=row_offset,
        shard_rotation=shard_rotation,
    )
    row_offset += table_to_padded_vocab_size[name] // num_shards
    shard_rotation = (shard_rotation + rotation) % num_shards
  return settings


def _get_stack_name(table_names: Sequence[str], use_short_stack_names: bool = True,
                    max_original_display_length: int = 50, hash_length: int = 12) -> str:
  full = "_".join(table_names)
  if not use_short_stack_names or len(full) <= max_original_display_length:
    return full
  digest = hashlib.sha256(full.encode("utf-8")).hexdigest()[:hash_length]
  return full[:max_original_display_length] + "..." + digest


def _already_stacked_elsewhere(table: TableSpec) -> bool:
  return table.setting_in_stack is not None and table.setting_in_stack.stack_name != table.name


def _verify_stack_tables(stack_name, table_names, features, tables):
  for name in table_names:
    if _already_stacked_elsewhere(tables[name]):
      raise ValueError(
          f"Table {name} is already stacked in group {tables[name].setting_in_stack.stack_name}.")
  for feature in features:
    t = feature.table_spec
    if _already_stacked_elsewhere(t) and t.setting_in_stack.stack_name == stack_name:
      raise ValueError(f"Cannot use stack name {stack_name} since it's already used.")
  for name, count in collections.Counter(table_names).items():
    if count > 1:
      raise ValueError(f"Table {name} is repeated in group {stack_name}.")
  first = tables[table_names[0]]
  if any(tables[n].optimizer != first.optimizer for n in table_names):
    raise ValueError(f"Tables {table_names} in group {stack_name} have different optimizers.")
  if any(tables[n].combiner != first.combiner for n in table_names):
    raise ValueError(f"Tables {table_names} in group {stack_name} have different combiners.")
  if any(tables[n].quantization_config != first.quantization_config for n in table_names):
    raise ValueError(f"Tables {table_names} in group {stack_name} have different quantization configs.")


def stack_tables(features, table_names: Sequence[str], global_device_count: int, num_sc_per_device: int,
                 rotation: int | None = None,
                 stack_to_max_ids_per_partition: LimitsCallable = get_default_limits,
                 stack_to_max_unique_ids_per_partition: LimitsCallable = get_default_limits,
                 stack_name: str | None = None, fail_on_excess_padding: bool = False, *,
                 activation_mem_bytes_limit: int = DEFAULT_ACTIVATION_MEM_BYTES_LIMIT) -> None:
  """Stacks the named tables; updates the feature specs in place."""
  stack_name = stack_name or _get_stack_name(table_names)
  flat = _tree.leaves(features)
  num_shards = num_sc_per_device * global_device_count
  in_group = {f.table_spec.name: f.table_spec for f in flat if f.table_spec.name in table_names}
  dims, vocabs = round_up_dim_and_vocab_size(in_group, num_shards)
  stack_dim = max(dims.values())
  if any(dims[t] != stack_dim for t in table_names):
    excess = sum((stack_dim - dims[t]) * vocabs[t] for t in table_names)
    msg = (f"Excess padding detected for stacked table {stack_name}.\n  Tables: {table_names},\n"
           f"  Padded sizes: {dims.values()},\n  Excess padding: {excess} values.\n"
           "To reduce the memory footprint, stack tables that have consistent embedding dimensions "
           "when rounded up to the nearest multiple of 8 values.")
    if fail_on_excess_padding:
      raise ValueError(msg)
    _log.warning("WARNING during stack_tables:\n%s", msg)
  _verify_stack_tables(stack_name, table_names, flat, in_group)

  rotation = num_sc_per_device if rotation is None else rotation
  settings = compute_table_to_setting_in_stack(stack_name, table_names, stack_dim, vocabs, num_shards, rotation)

  members = [f for f in flat if f.table_spec.name in table_names]
  row_offsets, samples = {}, 0
  for f in members:
    row_offsets[f.name] = samples
    samples += int(np.prod(f.output_shape[:-1]))

  if len(table_names) == 1:
    only = in_group[table_names[0]]
    max_ids, max_unique = only.max_ids_per_partition, only.max_unique_ids_per_partition
  else:
    max_ids = stack_to_max_ids_per_partition(stack_name, samples)
    max_unique = stack_to_max_unique_ids_per_partition(stack_name, samples)
    _log.warning(
        "Stacking multiple tables together: %s. Per-table max_ids_per_partition / "
        "max_unique_ids_per_partition are ignored; the stack uses max_ids=%d, max_unique_ids=%d. "
        "Use embedding.update_preprocessing_parameters to change them after stacking.",
        table_names, max_ids, max_unique)

  head = members[0].table_spec
  stacked = StackedTableSpec(
      stack_name=stack_name,
      stack_vocab_size=sum(vocabs[t] for t in table_names),
      stack_embedding_dim=stack_dim,
      optimizer=head.optimizer,
      combiner=head.combiner,
      total_sample_count=samples,
      max_ids_per_partition=max_ids,
      max_unique_ids_per_partition=max_unique,
      activation_mem_bytes_limit=activation_mem_bytes_limit,
      quantization_config=head.quantization_config,
  )
  for f in members:
    setting = settings[f.table_spec.name]
    f.table_spec.stacked_table_spec = stacked
    f.table_spec.setting_in_stack = setting
    f.id_transformation = embedding_spec.FeatureIdTransformation(
        row_offset=row_offsets[f.name],
        col_offset=setting.row_offset_in_shard * num_shards,
        col_shift=setting.shard_rotation,
    )


def _stack_groups(num_sc: int, tables: Mapping[str, TableSpec], features, limit: int) -> list[list[str]]:
  """Groups by (padded dim, optimizer, combiner, quantization), then first-fit by activation bytes."""
  dims, _ = round_up_dim_and_vocab_size(tables, num_sc)
  by_key: dict[tuple, list[str]] = collections.defaultdict(list)
  for name, dim in dims.items():
    t = tables[name]
    by_key[(dim, t.optimizer, t.combiner, t.quantization_config)].append(name)

  samples: dict[str, int] = collections.defaultdict(int)
  for f in features:
    samples[f.table_spec.name] += int(np.prod(f.output_shape[:-1]) // num_sc)
  act_bytes = {n: dims[n] * samples[n] * 4 for n in tables}

  groups: list[list[str]] = []
  for names in by_key.values():
    bins: list[list[str]] = []
    for name in names:
      for b in bins:
        if sum(act_bytes[m] for m in b) + act_bytes[name] <= limit:
          b.append(name)
          break
      else:
        bins.append([name])
    groups.extend(bins)
  if {n for g in groups for n in g} != set(tables):
    raise ValueError("Table names are not grouped correctly.")
  return groups


def auto_stack_tables(features, global_device_count: int, num_sc_per_device: int, rotation: int | None = None,
                      stack_to_max_ids_per_partition: LimitsCallable = get_default_limits,
                      stack_to_max_unique_ids_per_partition: LimitsCallable = get_default_limits, *,
                      use_short_stack_names: bool = True,
                      activation_mem_bytes_limit: int | None = DEFAULT_ACTIVATION_MEM_BYTES_LIMIT) -> None:
  """Stacks every group of compatible tables that fits the activation budget."""
  if activation_mem_bytes_limit is None:
    activation_mem_bytes_limit = DEFAULT_ACTIVATION_MEM_BYTES_LIMIT
  flat = _tree.leaves(features)
  tables = {f.table_spec.name: f.table_spec for f in flat}
  groups = _stack_groups(num_sc_per_device * global_device_count, tables, flat, activation_mem_bytes_limit)
  for group in groups:
    stack_tables(
        features, group, global_device_count, num_sc_per_device, rotation,
        stack_to_max_ids_per_partition, stack_to_max_unique_ids_per_partition,
        stack_name=_get_stack_name(group, use_short_stack_names), fail_on_excess_padding=False,
        activation_mem_bytes_limit=activation_mem_bytes_limit)
