"""Embedding lookup and update API of the SparseCore path on B200.

Function names, argument order, keyword names and error behaviour follow the reference's
jax_tpu_embedding/sparsecore/lib/nn/embedding.py (`preprocess_sparse_dense_matmul_input`
:608, `tpu_sparse_dense_matmul` :1048, `tpu_sparse_dense_matmul_grad` :1298,
`prepare_feature_specs_for_training` :342, `auto_stack_tables` :456,
`unstack_embedding_activations` :1029, `stack_embedding_gradients` :1220,
`init_embedding_variables` :1648, `update_preprocessing_parameters` :1768,
`SparseDenseMatmulInputStats` :97, `PreprocessedInput` :191).  Arrays are torch CUDA tensors
(numpy inputs are copied to the GPU); tables and slot variables are updated in place.

Device topology.  The reference runs these functions per device inside
`jax.jit(jax.shard_map(...))`.  Here a process drives one GPU; `global_device_count` is the
number of devices sharing each stacked table and the number of devices whose buffers a call
carries is read from the operand shapes: all of them ("virtual devices" on one GPU - the
whole job computed by one process) or one (one process per GPU, see `distributed`).
"""

from __future__ import annotations

import collections
import dataclasses
from typing import Any, Mapping, NamedTuple, Sequence
import sys
import warnings

import numpy as np

from jax_tpu_embedding.sparsecore import _native
from jax_tpu_embedding.sparsecore import _tree
from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing
from jax_tpu_embedding.sparsecore.lib.core.primitives import _ops
from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_csr
from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec
from jax_tpu_embedding.sparsecore.lib.nn import table_stacking
from jax_tpu_embedding.sparsecore.utils import utils

LimitsCallable = table_stacking.LimitsCallable
get_default_limits = table_stacking.get_default_limits
RaggedInput = pybind_input_preprocessing.RaggedInput


_LEAF_TYPES: tuple = ()


def _leaf_types() -> tuple:
  """The classes whose instances are leaves of a feature tree (torch.Tensor joins once torch is loaded)."""
  global _LEAF_TYPES
  if len(_LEAF_TYPES) < 5:
    types = (embedding_spec.FeatureSpec, embedding_spec.TableSpec, RaggedInput, np.ndarray)
    torch = sys.modules.get("torch")
    if torch is not None:
      types += (torch.Tensor,)
    _LEAF_TYPES = types
  return _LEAF_TYPES


def _is_feature_leaf(x) -> bool:
  return isinstance(x, _leaf_types()) or _is_array(x)


def _is_array(x) -> bool:
  return isinstance(x, np.ndarray) or type(x).__module__.startswith("torch")


def _flat_leaves(tree) -> bool:
  """True for the common case: a plain list or tuple whose elements are all leaves."""
  if type(tree) is not list and type(tree) is not tuple:
    return False
  types = _leaf_types()
  for x in tree:
    if not isinstance(x, types) and not _is_array(x):
      return False
  return True


def _leaves(tree):
  if _flat_leaves(tree):
    return list(tree)
  return _tree.leaves(tree, is_leaf=_is_feature_leaf)


def _assert_same_structure(a, b, a_name: str = "a", b_name: str = "b"):
  if _flat_leaves(a) and _flat_leaves(b) and type(a) is type(b) and len(a) == len(b):
    return
  a_paths = [p for p, _ in _tree.leaves_with_path(a, is_leaf=_is_feature_leaf)]
  b_paths = [p for p, _ in _tree.leaves_with_path(b, is_leaf=_is_feature_leaf)]
  if a_paths != b_paths:
    raise ValueError(
        f"Pytree structures of {a_name} and {b_name} do not match.\n"
        f"{a_name}: {_tree.structure(a, _is_feature_leaf)}\n{b_name}: {_tree.structure(b, _is_feature_leaf)}")


class EmbeddingVariablesInitializer(NamedTuple):
  table: embedding_spec.CallableTableInitializer
  slot: tuple[embedding_spec.CallableTableInitializer, ...]


class EmbeddingVariables(NamedTuple):
  table: Any
  slot: tuple[Any, ...]


class SparseDenseMatmulInput(NamedTuple):
  """The four CSR-wrapped COO buffers, each a dict keyed by stacked table name."""

  lhs_row_pointers: Mapping[str, Any]
  lhs_embedding_ids: Mapping[str, Any]
  lhs_sample_ids: Mapping[str, Any]
  lhs_gains: Mapping[str, Any]


@dataclasses.dataclass
class SparseDenseMatmulInputStats:
  """Statistics of one preprocessing call.

  max_ids_per_partition[table][device * P + g]: ids the device sends to shard g (max over its
  SparseCores); max_unique_ids_per_partition likewise for distinct rows;
  required_buffer_size_per_sc[table][device * S + s]: sum over shards of the id counts rounded
  up to 8; id_drop_counters[table]: ids dropped by the limits or by a full buffer.
  """

  # The suffix names the field in the files of the FDO clients (lib/fdo): "<table><suffix>".
  max_ids_per_partition: dict[str, np.ndarray] = dataclasses.field(metadata={"suffix": "_max_ids"})
  max_unique_ids_per_partition: dict[str, np.ndarray] = dataclasses.field(metadata={"suffix": "_max_unique_ids"})
  required_buffer_size_per_sc: dict[str, np.ndarray] = dataclasses.field(
      metadata={"suffix": "_required_buffer_size"}, default_factory=dict)
  id_drop_counters: dict[str, int] = dataclasses.field(metadata={"suffix": "_id_drop_counters"}, default_factory=dict)

  @classmethod
  def from_cc(cls, stats) -> "SparseDenseMatmulInputStats":
    return cls(
        max_ids_per_partition=stats.max_ids_per_partition,
        max_unique_ids_per_partition=stats.max_unique_ids_per_partition,
        required_buffer_size_per_sc=stats.required_buffer_sizes,
        id_drop_counters=stats.dropped_id_count,
    )

  def get_required_buffer_size_per_device(self, table_name: str, num_sc_per_device: int | None = None) -> int | None:
    if table_name not in self.required_buffer_size_per_sc:
      return None
    val = self.required_buffer_size_per_sc[table_name]
    return int(np.max(val) * (num_sc_per_device or np.size(val)))

  def set_required_buffer_size_per_device(self, table_name: str, required_buffer_size_per_device: int,
                                          num_sc_per_device: int | None = None) -> None:
    val = self.required_buffer_size_per_sc.get(table_name)
    num_sc = num_sc_per_device or (np.size(val) if val is not None else 0)
    if not num_sc:
      raise ValueError("num_sc_per_device must be provided if the table is not present.")
    self.required_buffer_size_per_sc[table_name] = np.full(num_sc, required_buffer_size_per_device / num_sc)


@dataclasses.dataclass
class PreprocessedInput:
  """Result of preprocessing: the CSR buffers and the (always 1) number of minibatches."""

  sparse_dense_matmul_input: SparseDenseMatmulInput
  num_minibatches: Any = dataclasses.field(default_factory=lambda: np.array(1))

  @property
  def lhs_row_pointers(self):
    return self.sparse_dense_matmul_input.lhs_row_pointers

  @property
  def lhs_embedding_ids(self):
    return self.sparse_dense_matmul_input.lhs_embedding_ids

  @property
  def lhs_sample_ids(self):
    return self.sparse_dense_matmul_input.lhs_sample_ids

  @property
  def lhs_gains(self):
    return self.sparse_dense_matmul_input.lhs_gains

  def __iter__(self):
    warnings.warn("Please use attributed lookup on sparse_dense_matmul_input attribute.", DeprecationWarning)
    return iter(self.sparse_dense_matmul_input)


def _verify_unique(names, kind: str) -> None:
  seen = set()
  for n in names:
    if n in seen:
      raise ValueError(f"{kind} spec {n} is already defined.")
    seen.add(n)


def _get_num_sc_per_device(num_sc_per_device: int | None) -> int:
  if num_sc_per_device is None:
    return utils.num_sparsecores_per_device()
  if num_sc_per_device not in utils.NUM_SC_PER_DEVICE_MAP.values():
    raise ValueError(f"Invalid num_sc_per_device: {num_sc_per_device}")
  return num_sc_per_device


def get_table_specs(feature_specs) -> Mapping[str, embedding_spec.TableSpec]:
  flat = _leaves(feature_specs)
  _verify_unique([f.name for f in flat], "Feature")
  tables = {}
  for f in flat:
    prior = tables.get(f.table_spec.name)
    if prior is not None and prior is not f.table_spec and prior != f.table_spec:
      raise ValueError(f"Table spec {f.table_spec.name} is already defined.")
    tables[f.table_spec.name] = f.table_spec
  return tables


def get_stacked_table_specs(feature_specs) -> Mapping[str, embedding_spec.StackedTableSpec]:
  flat = _leaves(feature_specs)
  _verify_unique([f.name for f in flat], "Feature")
  if any(not f.table_spec.is_stacked() for f in flat):
    raise ValueError("embedding.prepare_feature_specs_for_training was not called")
  return {f.table_spec.stacked_table_spec.stack_name: f.table_spec.stacked_table_spec for f in flat}


def prepare_feature_specs_for_training(feature_specs, global_device_count: int,
                                       num_sc_per_device: int | None = None) -> None:
  """Gives every unstacked table a one-table stack; features of one table are stacked by name order."""
  num_sc_per_device = _get_num_sc_per_device(num_sc_per_device)
  flat = _leaves(feature_specs)
  pending = [f for f in flat if not f.table_spec.is_stacked()]
  by_table: dict[str, list] = collections.defaultdict(list)
  for f in pending:
    by_table[f.table_spec.name].append(f)
  row_offsets, sample_counts = {}, {}
  for name, feats in by_table.items():
    feats.sort(key=lambda f: f.name)
    acc = 0
    for f in feats:
      row_offsets[f.name] = acc
      acc += int(np.prod(f.output_shape[:-1]))
    sample_counts[name] = acc
  num_shards = num_sc_per_device * global_device_count
  for f in pending:
    t = f.table_spec
    if t.is_stacked():  # a sibling feature of the same table already populated it
      f.id_transformation = embedding_spec.FeatureIdTransformation(row_offset=row_offsets.get(f.name, 0))
      continue
    if t.setting_in_stack is not None and t.setting_in_stack.stack_name != t.name:
      raise ValueError(
          f"Invalid stacking. Table {t.name} does not have StackedTableSpec populated, but"
          f" feature.table_spec.setting_in_stack.stack_name ({t.setting_in_stack.stack_name}) is not {t.name}.")
    dims, vocabs = table_stacking.round_up_dim_and_vocab_size({t.name: t}, num_shards)
    t.setting_in_stack = embedding_spec.TableSettingInStack(
        stack_name=t.name, padded_embedding_dim=dims[t.name], padded_vocab_size=vocabs[t.name],
        row_offset_in_shard=0, shard_rotation=0)
    t.stacked_table_spec = embedding_spec.StackedTableSpec(
        stack_name=t.name,
        stack_vocab_size=vocabs[t.name],
        stack_embedding_dim=dims[t.name],
        optimizer=t.optimizer,
        combiner=t.combiner,
        total_sample_count=sample_counts[t.name],
        max_ids_per_partition=t.max_ids_per_partition,
        max_unique_ids_per_partition=t.max_unique_ids_per_partition,
        suggested_coo_buffer_size_per_device=t.suggested_coo_buffer_size_per_device,
        quantization_config=t.quantization_config,
    )
    f.id_transformation = embedding_spec.FeatureIdTransformation(row_offset=row_offsets.get(f.name, 0))


def auto_stack_tables(feature_specs, global_device_count: int, num_sc_per_device: int | None = None,
                      stack_to_max_ids_per_partition: LimitsCallable = get_default_limits,
                      stack_to_max_unique_ids_per_partition: LimitsCallable = get_default_limits,
                      use_short_stack_names: bool = True, *, activation_mem_bytes_limit: int | None = None) -> None:
  table_stacking.auto_stack_tables(
      feature_specs, global_device_count=global_device_count,
      num_sc_per_device=_get_num_sc_per_device(num_sc_per_device),
      stack_to_max_ids_per_partition=stack_to_max_ids_per_partition,
      stack_to_max_unique_ids_per_partition=stack_to_max_unique_ids_per_partition,
      use_short_stack_names=use_short_stack_names, activation_mem_bytes_limit=activation_mem_bytes_limit)


def compute_row_pointers_size_per_device(*, global_device_count: int, num_sc_per_device: int | None = None,
                                         enable_minibatching: bool = False) -> int:
  return pybind_input_preprocessing.compute_row_pointers_size_per_device(
      global_device_count=global_device_count, num_sc_per_device=_get_num_sc_per_device(num_sc_per_device),
      enable_minibatching=enable_minibatching)


def compute_theoretical_max_coo_buffer_size(max_ids_per_partition: int, global_device_count: int,
                                            num_sc_per_device: int | None = None,
                                            enable_minibatching: bool = False) -> int:
  return pybind_input_preprocessing.compute_theoretical_max_coo_buffer_size(
      max_ids_per_partition=max_ids_per_partition, global_device_count=global_device_count,
      num_sc_per_device=_get_num_sc_per_device(num_sc_per_device), enable_minibatching=enable_minibatching)


def compute_coo_buffer_size_per_device(feature_specs, global_device_count: int, num_sc_per_device: int | None = None,
                                       enable_minibatching: bool = False) -> dict[str, int]:
  return pybind_input_preprocessing.compute_coo_buffer_size_per_device(
      feature_specs=_leaves(feature_specs), global_device_count=global_device_count,
      num_sc_per_device=_get_num_sc_per_device(num_sc_per_device), enable_minibatching=enable_minibatching)


def sharding_strategy_to_enum(sharding_strategy: str) -> pybind_input_preprocessing.ShardingStrategy:
  if sharding_strategy.upper() == "MOD":
    return pybind_input_preprocessing.ShardingStrategy.MOD
  raise ValueError(f"Unsupported sharding strategy: {sharding_strategy}. Only MOD is supported.")


def preprocess_sparse_dense_matmul_input(features, features_weights, feature_specs, local_device_count: int,
                                         global_device_count: int, *, num_sc_per_device: int | None = None,
                                         sharding_strategy: str = "MOD", has_leading_dimension: bool = False,
                                         allow_id_dropping: bool = False, batch_number: int = 0,
                                         enable_minibatching: bool = False, all_reduce_interface=None,
                                         device_output: bool = True, sync_stats: bool = True
                                         ) -> tuple[PreprocessedInput, SparseDenseMatmulInputStats]:
  """Turns raw feature ids (and weights) into the CSR-wrapped COO buffers the lookup consumes.

  Each feature leaf is a 2-D int array [batch, valency], a 1-D object array of id arrays
  (ragged), or a `RaggedInput`.  With `device_output` (default) the buffers stay on the GPU as
  torch tensors; with False they are numpy arrays like the reference's.  `sync_stats=False` (honoured
  for dense int32 device inputs) does not wait for the GPU: the statistics are fetched when first
  read, and a violated id limit raises then or at the next call.
  """
  num_sc_per_device = _get_num_sc_per_device(num_sc_per_device)
  _assert_same_structure(features, feature_specs, "features", "feature_specs")
  if features_weights is not None:
    _assert_same_structure(features_weights, feature_specs, "features_weights", "feature_specs")
  if enable_minibatching and all_reduce_interface is None and local_device_count < global_device_count:
    raise ValueError("all_reduce_interface must be provided when minibatching is enabled for multi-host.")
  *csr, num_minibatches, stats = pybind_input_preprocessing.preprocess_sparse_dense_matmul_input(
      _leaves(features),
      _leaves(features_weights) if features_weights else None,
      _leaves(feature_specs),
      local_device_count,
      global_device_count,
      num_sc_per_device=num_sc_per_device,
      sharding_strategy=sharding_strategy_to_enum(sharding_strategy),
      has_leading_dimension=has_leading_dimension,
      allow_id_dropping=allow_id_dropping,
      batch_number=batch_number,
      enable_minibatching=enable_minibatching,
      all_reduce_interface=all_reduce_interface,
      device_output=device_output,
      sync_stats=sync_stats,
  )
  minibatches = np.full(local_device_count, num_minibatches)
  if has_leading_dimension:
    minibatches = minibatches.reshape(local_device_count, 1)
  return (PreprocessedInput(SparseDenseMatmulInput(*csr), minibatches), SparseDenseMatmulInputStats.from_cc(stats))


def preprocess_sparse_dense_matmul_input_from_sparse_tensor(indices, values, dense_shapes, feature_specs,
                                                            local_device_count: int, global_device_count: int, *,
                                                            num_sc_per_device: int | None = None,
                                                            sharding_strategy: str = "MOD",
                                                            has_leading_dimension: bool = False,
                                                            allow_id_dropping: bool = False, batch_number: int = 0,
                                                            enable_minibatching: bool = False,
                                                            all_reduce_interface=None, device_output: bool = True
                                                            ) -> tuple[PreprocessedInput, SparseDenseMatmulInputStats]:
  """preprocess_sparse_dense_matmul_input for features given as sparse tensors (unit weights).

  `indices`: per feature an int [N, 2] array of (sample, position), row-major; `values`: int32 [N]
  embedding ids; `dense_shapes`: (batch, max positions).  All three have the structure of
  `feature_specs` (reference: lib/nn/embedding.py:708-819).
  """
  num_sc_per_device = _get_num_sc_per_device(num_sc_per_device)
  _assert_same_structure(indices, feature_specs, "indices", "feature_specs")
  _assert_same_structure(values, feature_specs, "values", "feature_specs")
  _assert_same_structure(dense_shapes, feature_specs, "dense_shapes", "feature_specs")
  if enable_minibatching and all_reduce_interface is None and local_device_count < global_device_count:
    raise ValueError("all_reduce_interface must be provided when minibatching is enabled for multi-host.")
  *csr, num_minibatches, stats = pybind_input_preprocessing.preprocess_sparse_dense_matmul_sparse_coo_input(
      _leaves(indices), _leaves(values), _leaves(dense_shapes), _leaves(feature_specs), local_device_count,
      global_device_count, num_sc_per_device=num_sc_per_device,
      sharding_strategy=sharding_strategy_to_enum(sharding_strategy), has_leading_dimension=has_leading_dimension,
      allow_id_dropping=allow_id_dropping, batch_number=batch_number, enable_minibatching=enable_minibatching,
      all_reduce_interface=all_reduce_interface, device_output=device_output)
  minibatches = np.full(local_device_count, num_minibatches, dtype=np.int32)
  if has_leading_dimension:
    minibatches = minibatches.reshape(local_device_count, 1)
  return (PreprocessedInput(SparseDenseMatmulInput(*csr), minibatches), SparseDenseMatmulInputStats.from_cc(stats))


@dataclasses.dataclass(frozen=True)
class ShapeDtype:
  shape: tuple[int, ...]
  dtype: Any


def eval_preprocess_sparse_dense_matmul_input_shape(feature_specs, local_device_count: int, global_device_count: int,
                                                    *, num_sc_per_device: int | None = None,
                                                    has_leading_dimension: bool = False,
                                                    enable_minibatching: bool = False) -> PreprocessedInput:
  """Shapes and dtypes of the preprocessing output, computed from the specs alone."""
  coo = compute_coo_buffer_size_per_device(feature_specs, global_device_count, num_sc_per_device=num_sc_per_device,
                                           enable_minibatching=enable_minibatching)
  rp = compute_row_pointers_size_per_device(global_device_count=global_device_count,
                                            num_sc_per_device=num_sc_per_device,
                                            enable_minibatching=enable_minibatching)
  mk = lambda size, dt: ShapeDtype((local_device_count * size,), dt)
  num_mb = ShapeDtype((local_device_count, 1) if has_leading_dimension else (local_device_count,), np.int32)
  return PreprocessedInput(
      SparseDenseMatmulInput(
          lhs_row_pointers={n: mk(rp, np.int32) for n in coo},
          lhs_embedding_ids={n: mk(s, np.int32) for n, s in coo.items()},
          lhs_sample_ids={n: mk(s, np.int32) for n, s in coo.items()},
          lhs_gains={n: mk(s, np.float32) for n, s in coo.items()},
      ), num_mb)


# ------------------------------------------------------------------------------------ forward


def _verify_input_batch_size(shape, slices: int, name: str) -> None:
  if shape[0] % slices:
    raise ValueError(
        "The input batch size must be divisible by the number of feature slices per device. Got input shape"
        f" {tuple(shape)} and {slices} feature slices per device for feature {name}.")


def _local_devices(row_pointers, global_device_count: int, num_sc_per_device: int) -> int:
  """Number of devices whose buffers are concatenated in `row_pointers`."""
  per_device = max(global_device_count * num_sc_per_device, 8) * num_sc_per_device
  n = int(np.prod(tuple(row_pointers.shape)))
  if n % per_device:
    raise ValueError(f"lhs_row_pointers has {n} entries, not a multiple of {per_device}")
  return n // per_device


def _get_activation_for_feature(feature, activations, global_device_count: int, num_feature_slices_per_device: int,
                                local_device_count: int = 1):
  """Rows of the stacked activation that belong to `feature` (all local devices)."""
  if feature.output_shape[-1] > feature.table_spec.embedding_dim:
    raise ValueError(
        f"Feature {feature.name} has output shape {feature.output_shape} and embedding dim"
        f" {feature.table_spec.embedding_dim}. The embedding dim in output shape cannot be more than the"
        " (original, unpadded) embedding dim in the FeatureSpec.")
  act = activations[feature.table_spec.stacked_table_spec.stack_name]
  f = num_feature_slices_per_device
  l = local_device_count
  per_slice_offset = feature.id_transformation.row_offset // (global_device_count * f)
  per_slice_batch = feature.output_shape[0] // (global_device_count * f)
  _verify_input_batch_size((act.shape[0] // l,), f, feature.name)
  # [devices, slices, per-slice stacked batch, ...]
  view = act.reshape((l, f, act.shape[0] // (l * f)) + tuple(act.shape[1:]))
  view = view[:, :, per_slice_offset:per_slice_offset + per_slice_batch]
  if act.dim() > 1:
    view = view[..., :feature.output_shape[-1]]
  return view.reshape((l * f * per_slice_batch,) + tuple(view.shape[3:]))


def unstack_embedding_activations(activations, feature_specs, global_device_count: int, num_sc_per_device: int,
                                  use_activation_unstack_primitive: bool = False, local_device_count: int = 1):
  """Stacked activations per table -> activations per feature (same tree as feature_specs)."""
  del use_activation_unstack_primitive  # one implementation: strided views of the stacked buffer
  return _tree.tree_map(
      lambda feat: _get_activation_for_feature(feat, activations, global_device_count, num_sc_per_device,
                                               local_device_count),
      feature_specs, is_leaf=_is_feature_leaf)


def _max_ids_per_sample(feature_specs, stack_name: str) -> int:
  """1 when every feature of the stack is declared single-valent, else 0 (unknown)."""
  for f in _leaves(feature_specs):
    if f.table_spec.stacked_table_spec.stack_name != stack_name:
      continue
    shape = tuple(f.input_shape)
    if len(shape) < 2 or shape[-1] != 1:
      return 0
  return 1


class _SpecInfo:
  """Per feature-spec-tree facts that do not change between steps (cached by object identity)."""

  def __init__(self, feature_specs):
    self.flat = _leaves(feature_specs)
    self.stacked = get_stacked_table_specs(feature_specs)
    self.members: dict[str, list] = collections.defaultdict(list)
    for f in self.flat:
      self.members[f.table_spec.stacked_table_spec.stack_name].append(f)
    self.max_ids_per_sample = {}
    self.trivial = {}  # stack holds one feature that is the whole stacked activation
    for name, feats in self.members.items():
      single_valent = all(len(tuple(f.input_shape)) >= 2 and tuple(f.input_shape)[-1] == 1 for f in feats)
      self.max_ids_per_sample[name] = 1 if single_valent else 0
      f = feats[0]
      self.trivial[name] = (
          len(feats) == 1 and f.id_transformation.row_offset == 0 and len(f.output_shape) == 2
          and f.output_shape[-1] == f.table_spec.embedding_dim
          and f.table_spec.embedding_dim == self.stacked[name].stack_embedding_dim
          and f.output_shape[0] == self.stacked[name].total_sample_count)
    self.all_trivial = all(self.trivial.values())
    self.hypers: dict = {}  # step -> {stack: optimizer hyper-parameters as floats}
    self.flat_stack_names = [f.table_spec.stacked_table_spec.stack_name for f in self.flat]
    self.first_stacked = self.flat[0].table_spec._stacked_table_spec if self.flat else None  # pylint: disable=protected-access
    self.keep = feature_specs  # keeps the ids in the cache key alive


_SPEC_INFO: dict = {}
_LAST_SPEC_INFO: list = [None, None]  # the tree object of the previous call and its facts


def _spec_info(feature_specs) -> _SpecInfo:
  # The same tree object as in the previous call (a training loop): no walk over the tree.  A tree that was
  # changed in place, or whose tables were stacked again, is noticed by its length and its first stacked spec.
  last_tree, last = _LAST_SPEC_INFO
  if (last_tree is feature_specs and type(feature_specs) in (list, tuple) and len(feature_specs) == len(last.flat)
      and last.flat and feature_specs[0] is last.flat[0]
      and last.flat[0].table_spec._stacked_table_spec is last.first_stacked):  # pylint: disable=protected-access
    return last
  flat = _leaves(feature_specs)
  key = tuple((id(f), id(f.table_spec._stacked_table_spec), id(f._id_transformation)) for f in flat)  # pylint: disable=protected-access
  info = _SPEC_INFO.get(key)
  if info is None:
    if len(_SPEC_INFO) > 64:
      _SPEC_INFO.clear()
    info = _SPEC_INFO[key] = _SpecInfo(feature_specs)
  _LAST_SPEC_INFO[0], _LAST_SPEC_INFO[1] = feature_specs, info
  return info


def _is_cuda_tensor(x) -> bool:
  return type(x).__module__.startswith("torch") and x.is_cuda and x.is_contiguous()


_CALL_CACHE: dict = {}
# Replays and rebuilds of launch descriptors since import (a training loop should show replays only).
CALL_CACHE_STATS = {"replayed": 0, "built": 0}


def _csr_key(rps, eids, sids, gains, names):
  """(key, bases): identity of the four CSR array dicts for the launch-descriptor cache (None: not cacheable).

  Dicts that come from this package's preprocessing carry a token naming the two device buffers they are views of
  and their layout.  The key then holds the layout only and `bases` the two addresses: cached descriptors are
  replayed for every output of that layout, their CSR pointers moved to the new buffers (`rebase`).  Otherwise every
  array is described by (address, shape, dtype) and `bases` is None.
  """
  tokens = tuple(getattr(d, "token", None) for d in (rps, eids, sids, gains))
  if all(t is not None for t in tokens) and len(rps) == len(names):
    bases = tokens[0][:2]
    if all(t[:2] == bases for t in tokens):
      return tuple(t[2:] for t in tokens), bases
    return tokens, None
  arrays = [d[n] for n in names for d in (rps, eids, sids, gains)]
  if not all(_is_cuda_tensor(x) for x in arrays):
    return None, None
  return tuple((x.data_ptr(), tuple(x.shape), x.dtype) for x in arrays), None


def _forward_plans(rps, eids, sids, gains):
  """{stack name: (plan_slots, plan_bags)} if the four dicts are the untouched output of ONE call of this
  package's preprocessing (which emits the forward's sample-major plan with the buffers), else None."""
  tokens = [getattr(d, "token", None) for d in (rps, eids, sids, gains)]
  if any(t is None for t in tokens) or len({t[:-1] for t in tokens}) != 1:
    return None
  return getattr(rps, "forward_plans", None)


def _tensor_key(tensors):
  """((address, shape), ...) of contiguous CUDA tensors, or None if any element is something else."""
  try:
    key = tuple((x.data_ptr(), x.shape) for x in tensors if x.is_cuda and x.is_contiguous())
  except AttributeError:
    return None
  return key if len(key) == len(tensors) else None


def _address_key(tensors):
  """Addresses of torch tensors, or None if any element is something else.  For operands that live as long as the
  cached descriptors are useful (tables and slot variables): whatever else there is to check about them was checked
  when the descriptors were built, and a host tensor or a new allocation has another address."""
  try:
    return tuple([x.data_ptr() for x in tensors])
  except AttributeError:
    return None


def clear_caches() -> None:
  """Forgets the cached launch descriptors and spec facts (they hold addresses of tables and buffers).

  Call it after freeing or replacing embedding variables whose addresses may be reused by new ones, and after
  changing a feature-spec tree in place.
  """
  _CALL_CACHE.clear()
  _SPEC_INFO.clear()
  _LAST_SPEC_INFO[0] = _LAST_SPEC_INFO[1] = None
  pybind_input_preprocessing.clear_caches()


def _cache_put(key, value):
  if len(_CALL_CACHE) > 32:
    _CALL_CACHE.clear()
  _CALL_CACHE[key] = value


def tpu_sparse_dense_matmul(preprocessed_inputs, embedding_variables, feature_specs, *, global_device_count: int,
                            sharding_strategy: str = "MOD", num_sc_per_device: int | None = None,
                            enable_minibatching: bool = False, perform_unstacking: bool = True,
                            use_activation_unstack_primitive: bool = False):
  """Embedding lookup: one gather-combine per stacked table, then per-feature views.

  All stacked tables are served by one grouped launch sequence.  When the same device buffers
  are passed again (same addresses, sizes and specs) the validated launch descriptors of the
  previous call are reused, so a training loop pays the per-table Python work once.
  """
  if isinstance(preprocessed_inputs, SparseDenseMatmulInput):
    warnings.warn("SparseDenseMatmulInput is deprecated. Please use PreprocessedInput instead.", DeprecationWarning)
    preprocessed_inputs = PreprocessedInput(preprocessed_inputs)
  rps, eids, sids, gains = preprocessed_inputs.sparse_dense_matmul_input
  num_sc_per_device = _get_num_sc_per_device(num_sc_per_device)
  assert rps.keys() == embedding_variables.keys()
  info = _spec_info(feature_specs)
  stacked_table_specs = info.stacked
  assert rps.keys() == stacked_table_specs.keys()
  strategy = int(sharding_strategy_to_enum(sharding_strategy))

  key = None
  csr_key, bases = _csr_key(rps, eids, sids, gains, stacked_table_specs)
  table_key = _address_key([embedding_variables[n].table for n in stacked_table_specs])
  if csr_key is not None and table_key is not None:
    key = ("fwd", id(info), global_device_count, num_sc_per_device, strategy, enable_minibatching, csr_key, table_key)
  cached = _CALL_CACHE.get(key) if key is not None else None
  CALL_CACHE_STATS["built" if cached is None else "replayed"] += 1
  if cached is None:
    requests, local = [], 1
    # Sample-major plans that this package's preprocessing emitted together with these buffers.
    plans = _forward_plans(rps, eids, sids, gains)
    for name, stacked in stacked_table_specs.items():
      local = _local_devices(rps[name], global_device_count, num_sc_per_device)
      q = stacked.quantization_config
      requests.append(sparse_dense_matmul_csr.tpu_sparse_dense_matmul_csr_primitive.prepare(
          _flat(rps[name]), _flat(eids[name]), _flat(sids[name]), _flat(gains[name]), np.int32(1),
          embedding_variables[name].table,
          device_batch_size=stacked.total_sample_count // global_device_count,
          max_ids_per_partition=stacked.max_ids_per_partition,
          max_unique_ids_per_partition=stacked.max_unique_ids_per_partition,
          sharding_strategy=strategy,
          quantization_config=q.as_tuple() if q else None,
          enable_minibatching=enable_minibatching,
          num_sc_per_device=num_sc_per_device,
          global_device_count=global_device_count,
          local_device_count=local,
          max_ids_per_sample=info.max_ids_per_sample[name],
          forward_plan=plans.get(name) if plans else None,
      ))
    cached = (_ops.ForwardGroupCall(requests, bases), local)
    # (The key holds bare addresses of the tables: only descriptors built from device tensors may be replayed.)
    if key is not None and all(_is_cuda_tensor(embedding_variables[n].table) for n in stacked_table_specs):
      _cache_put(key, cached)
  call, local = cached
  if bases is not None:
    call.rebase(bases)
  # One grouped launch sequence for all stacked tables (the reference issues one call per table).
  activations = dict(zip(stacked_table_specs.keys(), call.run()))
  if perform_unstacking:
    if info.all_trivial and local == 1:
      leaves = [activations[name] for name in info.flat_stack_names]
      if type(feature_specs) is list and len(feature_specs) == len(leaves) and _flat_leaves(feature_specs):
        return leaves
      return _tree.unflatten(feature_specs, leaves, is_leaf=_is_feature_leaf)
    activations = unstack_embedding_activations(
        activations, feature_specs, global_device_count, num_sc_per_device,
        use_activation_unstack_primitive=use_activation_unstack_primitive, local_device_count=local)
  return activations


def _flat(x):
  return x.reshape(-1)


# ------------------------------------------------------------------------------------ backward


def _prepare_gradient_for_stacking(gradient, feature, num_sc_per_device: int):
  torch = _native.torch_mod()
  if not isinstance(gradient, torch.Tensor):
    gradient = torch.from_numpy(np.ascontiguousarray(gradient, dtype=np.float32))
  if torch.cuda.is_available() and not gradient.is_cuda:
    gradient = gradient.cuda(non_blocking=True)
  gradient = gradient.reshape(-1, feature.table_spec.embedding_dim)
  extra = feature.table_spec.setting_in_stack.padded_embedding_dim - feature.table_spec.embedding_dim
  if extra:
    gradient = torch.nn.functional.pad(gradient, (0, extra))
  _verify_input_batch_size(gradient.shape, num_sc_per_device, feature.name)
  return gradient


def stack_embedding_gradients(activation_gradients, feature_specs, num_sc_per_device: int,
                              global_device_count: int | None = None, use_gradient_stacking_primitive: bool = False,
                              local_device_count: int = 1) -> Mapping[str, Any]:
  """Per-feature activation gradients -> one [stacked batch, padded dim] tensor per stacked table."""
  del global_device_count, use_gradient_stacking_primitive
  torch = _native.torch_mod()
  by_stack: dict[str, list] = collections.defaultdict(list)
  for grad, feat in zip(_leaves(activation_gradients), _leaves(feature_specs)):
    if feat._id_transformation is None:  # pylint: disable=protected-access
      raise ValueError(f"FeatureIdTransformation cannot be None here. It is None for {feat.name}")
    by_stack[feat.table_spec.stacked_table_spec.stack_name].append((feat, grad))
  out = {}
  slices = local_device_count * num_sc_per_device
  for name, members in by_stack.items():
    members.sort(key=lambda m: m[0].id_transformation.row_offset)
    parts = []
    for feat, grad in members:
      g = _prepare_gradient_for_stacking(grad, feat, num_sc_per_device)
      parts.append(g.reshape(slices, g.shape[0] // slices, g.shape[1]))
    stacked = parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)
    out[name] = stacked.reshape(-1, stacked.shape[-1]).contiguous()
  return out


def tpu_sparse_dense_matmul_grad(activation_gradients, preprocessed_inputs, embedding_variables, feature_specs, *,
                                 global_device_count: int | None = None, sharding_strategy: str = "MOD",
                                 label: str = "", step=None, num_sc_per_device: int | None = None,
                                 enable_minibatching: bool = False, perform_stacking: bool = True,
                                 use_gradient_stacking_primitive: bool = False, embedding_var_limits=None
                                 ) -> Mapping[str, EmbeddingVariables]:
  """Applies the activation gradients to the tables with each stack's optimizer (in place)."""
  if isinstance(preprocessed_inputs, SparseDenseMatmulInput):
    warnings.warn("SparseDenseMatmulInput is deprecated. Please use PreprocessedInput instead.", DeprecationWarning)
    preprocessed_inputs = PreprocessedInput(preprocessed_inputs)
  rps, eids, sids, gains = preprocessed_inputs.sparse_dense_matmul_input
  assert rps.keys() == embedding_variables.keys()
  info = _spec_info(feature_specs)
  stacked_table_specs = info.stacked
  assert rps.keys() == stacked_table_specs.keys()
  num_sc_per_device = _get_num_sc_per_device(num_sc_per_device)
  if global_device_count is None:
    global_device_count = _ops._world_size()  # pylint: disable=protected-access
  first = next(iter(rps))
  local = _local_devices(rps[first], global_device_count, num_sc_per_device)

  if perform_stacking:
    _assert_same_structure(feature_specs, activation_gradients, "feature_specs", "activation_gradients")
    grad_leaves = _leaves(activation_gradients)
    if info.all_trivial and local == 1 and all(_is_cuda_tensor(g) and g.dim() == 2 for g in grad_leaves):
      gradients = dict(zip(info.flat_stack_names, grad_leaves))
    else:
      gradients = stack_embedding_gradients(activation_gradients, feature_specs, num_sc_per_device,
                                            global_device_count, use_gradient_stacking_primitive,
                                            local_device_count=local)
  else:
    assert isinstance(activation_gradients, Mapping)
    gradients = activation_gradients
  assert rps.keys() == gradients.keys()
  strategy = int(sharding_strategy_to_enum(sharding_strategy))

  # Hyper-parameters per stack; they depend on the specs and on `step` only.
  step_key = step if step is None or isinstance(step, int) else None
  hypers = info.hypers.get(step_key) if (step is None or step_key is not None) else None
  if hypers is None:
    hypers = {n: tuple(float(h) for h in st.optimizer.get_hyperparameters(step)) for n, st in stacked_table_specs.items()}
    if step is None or step_key is not None:
      if len(info.hypers) > 8:
        info.hypers.clear()
      info.hypers[step_key] = hypers
  limits = None if embedding_var_limits is None else tuple(
      tuple(embedding_var_limits[n]) for n in stacked_table_specs)
  key = None
  csr_key, bases = _csr_key(rps, eids, sids, gains, stacked_table_specs)
  names = tuple(stacked_table_specs)
  variable_key = _address_key([x for n in names for x in (embedding_variables[n].table, *embedding_variables[n].slot)])
  # Gradients arrive at other addresses every step (they are outputs of the dense model's backward pass): the key
  # holds their shapes and dtype, the descriptors get the addresses of this call (`set_gradients`).
  grad_list = [gradients[n] for n in names]
  tensor_key = None
  if variable_key is not None and all(_is_cuda_tensor(g) for g in grad_list):
    f32 = _native.torch_mod().float32  # (any other dtype is converted into a copy when the descriptors are built)
    if all(g.dtype == f32 for g in grad_list):
      tensor_key = (variable_key, tuple([g.shape for g in grad_list]))
  if csr_key is not None and tensor_key is not None:
    key = ("bwd", id(info), global_device_count, num_sc_per_device, strategy, enable_minibatching, label, limits,
           tuple(hypers.values()), csr_key, tensor_key)
  call = _CALL_CACHE.get(key) if key is not None else None
  CALL_CACHE_STATS["built" if call is None else "replayed"] += 1
  if call is None:
    requests = []
    for name, stacked in stacked_table_specs.items():
      variables = embedding_variables[name]
      hyper = stacked.optimizer.get_hyperparameters(step)
      symbol = "{}-{}{}".format(stacked.optimizer.short_name(), stacked.stack_name, label)
      extra = {}
      if embedding_var_limits is not None:
        extra["min_value"], extra["max_value"] = embedding_var_limits[name]
      if isinstance(stacked.optimizer, embedding_spec.FTRLOptimizerSpec):
        extra["multiply_linear_by_learning_rate"] = stacked.optimizer.multiply_linear_by_learning_rate
      requests.append(stacked.optimizer.get_optimizer_primitive().prepare(
          _flat(rps[name]), _flat(eids[name]), _flat(sids[name]), _flat(gains[name]), np.int32(1), variables.table,
          *variables.slot, gradients[name], *hyper,
          max_ids_per_partition=stacked.max_ids_per_partition,
          max_unique_ids_per_partition=stacked.max_unique_ids_per_partition,
          computation_name=symbol, sharding_strategy=strategy, enable_minibatching=enable_minibatching,
          num_sc_per_device=num_sc_per_device, global_device_count=global_device_count, local_device_count=local,
          **extra))
    call = _ops.GradGroupCall(requests, bases)
    # (The key holds bare addresses of tables and slot variables: only descriptors built from device tensors may be
    # replayed.)
    if key is not None and all(_is_cuda_tensor(x) for n in names
                               for x in (embedding_variables[n].table, *embedding_variables[n].slot)):
      _cache_put(key, call)
  if bases is not None:
    call.rebase(bases)
  if key is not None:
    call.set_gradients([g.data_ptr() for g in grad_list])
  first_results = call.run()
  # Tables and slot variables were updated in place; hand the same tensors back.
  if first_results is None:  # replayed descriptors: every operand is a device tensor that was updated in place
    return {name: embedding_variables[name] for name in names}
  updated = {}
  for index, name in enumerate(stacked_table_specs):
    variables = embedding_variables[name]
    if _is_cuda_tensor(variables.table) and all(_is_cuda_tensor(x) for x in variables.slot):
      updated[name] = variables
    else:
      results = first_results[index]
      slot_type = type(variables.slot)
      slots = slot_type(*results[1:]) if hasattr(slot_type, "_fields") else tuple(results[1:])
      updated[name] = EmbeddingVariables(table=results[0], slot=slots)
  return updated


# ------------------------------------------------------------------------------------ variables


@dataclasses.dataclass(frozen=True)
class DeviceLayout:
  """Which devices' shards a process materialises (stands in for jax NamedSharding).

  global_device_count devices share every stacked table; this process holds the shards of
  `local_device_count` of them starting at device `first_device`.  On one GPU without
  torch.distributed the default is "all of them" (virtual devices).
  """

  global_device_count: int
  local_device_count: int | None = None
  first_device: int = 0

  def resolved_local(self) -> int:
    return self.global_device_count if self.local_device_count is None else self.local_device_count


def init_embedding_variables(rng, table_specs, global_sharding: DeviceLayout | int | None = None,
                             num_sparsecore_per_device: int | None = None, bypass_mesh_check: bool = False,
                             device: str | None = None, allocator=None) -> Mapping[str, EmbeddingVariables]:
  """Creates every stacked table (and its slot variables) in the device layout the lookup expects.

  Layout of one device: for each of its SparseCores in turn, the per-shard blocks of the stack's
  tables in `row_offset_in_shard` order, i.e. [num_sc_per_device * rows_per_shard, padded_dim].
  `rng` is an int seed or a torch.Generator; every (stack, device, SparseCore, table) block gets
  its own stream of random numbers, as every shard does in the reference.
  """
  del bypass_mesh_check
  torch = _native.torch_mod()
  s = _get_num_sc_per_device(num_sparsecore_per_device)
  if global_sharding is None:
    world = _ops._world_size()  # pylint: disable=protected-access
    layout = DeviceLayout(world, 1 if world > 1 else None,
                          torch.distributed.get_rank() if world > 1 else 0)
  elif isinstance(global_sharding, int):
    layout = DeviceLayout(global_sharding)
  else:
    layout = global_sharding
  c, l = layout.global_device_count, layout.resolved_local()
  if allocator is None and l != c:
    from jax_tpu_embedding.sparsecore import distributed  # pylint: disable=g-import-not-at-top

    if distributed.is_active():
      allocator = distributed.alloc  # shards must be visible to the other GPUs
  if device is None:
    device = "cuda" if torch.cuda.is_available() else "cpu"
  seed = int(rng.initial_seed()) if isinstance(rng, torch.Generator) else int(rng)

  flat = [t for t in _tree.leaves(table_specs, is_leaf=_is_feature_leaf)]
  _verify_unique([t.name for t in flat], "Table")
  stacks: dict[str, list] = collections.defaultdict(list)
  for t in flat:
    stacks[t.setting_in_stack.stack_name].append(t)
  out = {}
  p = s * c
  for stack_index, (stack_name, members) in enumerate(stacks.items()):
    members.sort(key=lambda t: t.setting_in_stack.row_offset_in_shard)
    dim = members[0].setting_in_stack.padded_embedding_dim
    assert all(t.setting_in_stack.padded_embedding_dim == dim for t in members)
    rows_per_shard = sum(t.setting_in_stack.padded_vocab_size // p for t in members)
    inits = EmbeddingVariablesInitializer(table=None, slot=members[0].optimizer.slot_variables_initializers())
    shape = (l * s * rows_per_shard, dim)
    alloc = allocator or (lambda shp: torch.empty(shp, dtype=torch.float32, device=device))
    table = alloc(shape)
    slots = [alloc(shape) for _ in inits.slot]
    for d in range(l):
      for i in range(s):
        shard = (layout.first_device + d) * s + i
        row = (d * s + i) * rows_per_shard
        for t in members:
          n = t.setting_in_stack.padded_vocab_size // p
          gen = torch.Generator(device=device)
          gen.manual_seed((seed * 1000003 + stack_index * 7919 + shard * 104729 + t.setting_in_stack.row_offset_in_shard)
                          % (2**63 - 1))
          table[row:row + n] = _call_init(t.initializer, gen, (n, dim), device)
          for slot, init in zip(slots, inits.slot):
            slot[row:row + n] = _call_init(init, gen, (n, dim), device)
          row += n
    slot_type = type(inits.slot)
    slot_tuple = slot_type(*slots) if hasattr(slot_type, "_fields") else tuple(slots)
    out[stack_name] = EmbeddingVariables(table=table, slot=slot_tuple)
  return out


def _call_init(init, gen, shape, device):
  torch = _native.torch_mod()
  try:
    value = init(gen, shape, device=device)
  except TypeError:
    value = init(gen, shape)
  if not isinstance(value, torch.Tensor):
    value = torch.as_tensor(np.asarray(value, dtype=np.float32))
  return value.to(device=device, dtype=torch.float32)


def update_preprocessing_parameters(feature_specs, updated_params: SparseDenseMatmulInputStats,
                                    num_sc_per_device: int) -> None:
  """Copies observed limits and buffer sizes from `updated_params` into every StackedTableSpec."""
  for feature in _leaves(feature_specs):
    stacked = feature.table_spec.stacked_table_spec
    name = stacked.stack_name
    max_ids = updated_params.max_ids_per_partition.get(name, stacked.max_ids_per_partition)
    max_unique = updated_params.max_unique_ids_per_partition.get(name, stacked.max_unique_ids_per_partition)
    size = updated_params.get_required_buffer_size_per_device(name, num_sc_per_device)
    if size is None:
      size = stacked.suggested_coo_buffer_size_per_device
    feature.table_spec.stacked_table_spec = dataclasses.replace(
        stacked,
        max_ids_per_partition=int(np.max(max_ids)),
        max_unique_ids_per_partition=int(np.max(max_unique)),
        suggested_coo_buffer_size_per_device=size,
    )
