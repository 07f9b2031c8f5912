"""Table, feature and optimizer specifications of the SparseCore embedding path.

Same public names and meaning as the reference's
jax_tpu_embedding/sparsecore/lib/nn/embedding_spec.py: optimizer specs
(`OptimizerSpec` :123-247, `SGDOptimizerSpec` :377, `AdagradOptimizerSpec` :415,
`AdamOptimizerSpec` :463), `FeatureIdTransformation` :919, `TableSettingInStack`
:941, `TableSpec` :980, `FeatureSpec` :1121, `StackedTableSpec` :1169,
`QuantizationConfig` :1208.  Hyper-parameters are float32 numpy scalars; each
optimizer names the fused CUDA backward operator that applies it.
"""

from __future__ import annotations

import abc
import dataclasses
import inspect
from typing import Any, Callable, NamedTuple, Sequence

import numpy as np

from jax_tpu_embedding.sparsecore.lib.nn import initializers

# Default activation memory budget per shard when tables are stacked automatically.
DEFAULT_ACTIVATION_MEM_BYTES_LIMIT: int = 2048 * 1024

CallableTableInitializer = Callable[..., Any]


class SGDSlotVariables(NamedTuple):
  pass


class AdagradSlotVariables(NamedTuple):
  accumulator: Any


class AdamSlotVariables(NamedTuple):
  momentum: Any
  velocity: Any


class AdagradMomentumSlotVariables(NamedTuple):
  accumulator: Any
  momentum: Any


class FTRLSlotVariables(NamedTuple):
  accumulator: Any
  linear: Any


class LaPropSlotVariables(NamedTuple):
  mu: Any
  nu: Any


class F2ASlotVariables(NamedTuple):
  accumulator: Any
  local_step: Any


def _f32(x) -> np.ndarray:
  return np.asarray(x, dtype=np.float32)


class OptimizerSpec(metaclass=abc.ABCMeta):
  """Interface of an embedding optimizer: hyper-parameters, slots, fused operator."""

  def __init__(self, learning_rate=0.001):
    self.learning_rate = learning_rate

  def get_learning_rate(self, step=None) -> np.ndarray:
    """Learning rate as a float32 scalar; callables take no argument or the step."""
    lr = self.learning_rate
    if not callable(lr):
      return _f32(lr)
    params = inspect.getfullargspec(lr).args
    arity = len(params) if inspect.isfunction(lr) else len(params) - 1
    if arity == 0:
      return _f32(lr())
    if arity == 1:
      if step is None:
        raise ValueError(
            f"Specified learning rate callable {lr} requires a `step` argument to be specified.")
      return _f32(lr(step))
    raise ValueError(
        "Learning rate callbacks should either take no parameters, or a single step count argument.")

  def get_hyperparameters(self, step=None) -> tuple[np.ndarray, ...]:
    return (self.get_learning_rate(step),)

  def slot_variables_initializers(self) -> tuple[CallableTableInitializer, ...]:
    return ()

  def slot_variables_count(self) -> int:
    return len(self.slot_variables_initializers())

  @abc.abstractmethod
  def get_optimizer_primitive(self):
    """The fused gradient + update operator (an object with `.bind`)."""

  @abc.abstractmethod
  def short_name(self) -> str:
    """Short tag used in the name of the update computation."""

  @abc.abstractmethod
  def __hash__(self) -> int:
    ...

  def __eq__(self, other: object) -> bool:
    return isinstance(other, OptimizerSpec) and hash(self) == hash(other)

  def __repr__(self) -> str:
    fields = ", ".join(f"{k}={v!r}" for k, v in vars(self).items())
    return f"{type(self).__name__}({fields})"


class SGDOptimizerSpec(OptimizerSpec):
  """theta <- theta - lr * g."""

  def __hash__(self) -> int:
    return hash((self.learning_rate,))

  def short_name(self) -> str:
    return "sgd"

  def slot_variables_initializers(self):
    return SGDSlotVariables()

  def get_optimizer_primitive(self):
    from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_grad_with_sgd as m  # pylint: disable=g-import-not-at-top

    return m.tpu_sparse_dense_matmul_grad_with_sgd_primitive


class AdagradOptimizerSpec(OptimizerSpec):
  """a <- a + g^2; theta <- theta - lr * g / sqrt(a)."""

  def __init__(self, learning_rate=0.001, initial_accumulator_value=0.1):
    super().__init__(learning_rate)
    self.initial_accumulator_value = initial_accumulator_value

  def slot_variables_initializers(self):
    return AdagradSlotVariables(
        accumulator=initializers.constant(float(self.initial_accumulator_value)))

  def __hash__(self) -> int:
    return hash((self.learning_rate, self.initial_accumulator_value))

  def short_name(self) -> str:
    return "adagrad"

  def get_optimizer_primitive(self):
    from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_grad_with_adagrad as m  # pylint: disable=g-import-not-at-top

    return m.tpu_sparse_dense_matmul_grad_with_adagrad_primitive


class AdamOptimizerSpec(OptimizerSpec):
  """Lazy Adam with the bias correction folded into the hyper-parameters."""

  def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.999, epsilon=1e-8):
    super().__init__(learning_rate)
    self.beta_1 = beta_1
    self.beta_2 = beta_2
    self.epsilon = epsilon

  def slot_variables_initializers(self):
    return AdamSlotVariables(momentum=initializers.constant(0.0),
                             velocity=initializers.constant(0.0))

  def get_hyperparameters(self, step=None):
    """(alpha_t, beta_1, beta_2, epsilon_hat) for step t = step + 1, all float32.

    alpha_t = lr * sqrt(1 - beta_2^t) / (1 - beta_1^t),
    epsilon_hat = epsilon * sqrt(1 - beta_2^t).
    """
    if step is None:
      step = 0
    one = np.float32(1.0)
    beta_1, beta_2 = _f32(self.beta_1), _f32(self.beta_2)
    t = np.float32(np.asarray(step) + 1)
    c_2 = np.sqrt(one - np.power(beta_2, t, dtype=np.float32), dtype=np.float32)
    alpha_t = self.get_learning_rate(step) * c_2 / (one - np.power(beta_1, t, dtype=np.float32))
    return (_f32(alpha_t), beta_1, beta_2, _f32(_f32(self.epsilon) * c_2))

  def __hash__(self) -> int:
    return hash((self.learning_rate, self.beta_1, self.beta_2, self.epsilon))

  def short_name(self) -> str:
    return "adam"

  def get_optimizer_primitive(self):
    from jax_tpu_embedding.sparsecore.lib.core.primitives import sparse_dense_matmul_grad_with_adam as m  # pylint: disable=g-import-not-at-top

    return m.tpu_sparse_dense_matmul_grad_with_adam_primitive


def _primitive(module_name: str):
  import importlib  # pylint: disable=g-import-not-at-top

  mod = importlib.import_module(f"jax_tpu_embedding.sparsecore.lib.core.primitives.{module_name}")
  return getattr(mod, f"tpu_{module_name}_primitive")


class AdagradMomentumOptimizerSpec(OptimizerSpec):
  """Adagrad-scaled gradient fed through (optionally Nesterov) momentum.

  a <- a + g^2 (beta2 == 1) or beta2 a + (1 - beta2) g^2; s = (a + epsilon)^(-1/exponent) g;
  m <- momentum m + s; theta <- theta - lr (momentum m + s if use_nesterov else m).
  Mirrors the reference's AdagradMomentumOptimizerSpec (lib/nn/embedding_spec.py:560-650).
  """

  def __init__(self, learning_rate=0.001, momentum: float = 0.9, beta2: float = 1.0, epsilon: float = 1e-10,
               exponent: float = 2.0, use_nesterov: bool = False, initial_accumulator_value: float = 0.1,
               initial_momentum_value: float = 0.0):
    super().__init__(learning_rate)
    self.momentum = momentum
    self.beta2 = beta2
    self.epsilon = epsilon
    self.exponent = exponent
    self.use_nesterov = use_nesterov
    self.initial_accumulator_value = initial_accumulator_value
    self.initial_momentum_value = initial_momentum_value

  def slot_variables_initializers(self):
    return AdagradMomentumSlotVariables(accumulator=initializers.constant(float(self.initial_accumulator_value)),
                                        momentum=initializers.constant(float(self.initial_momentum_value)))

  def get_hyperparameters(self, step=None):
    return (self.get_learning_rate(step), _f32(self.momentum), _f32(self.beta2), _f32(self.epsilon),
            _f32(self.exponent), np.asarray(bool(self.use_nesterov)))

  def __hash__(self) -> int:
    return hash((self.learning_rate, self.momentum, self.beta2, self.epsilon, self.exponent, self.use_nesterov,
                 self.initial_accumulator_value, self.initial_momentum_value))

  def short_name(self) -> str:
    return "adagrad_momentum"

  def get_optimizer_primitive(self):
    return _primitive("sparse_dense_matmul_grad_with_adagrad_momentum")


class FTRLOptimizerSpec(OptimizerSpec):
  """Follow-the-regularized-leader with per-coordinate learning rates.

  Mirrors the reference's FTRLOptimizerSpec (lib/nn/embedding_spec.py:652-742); the update is in
  lib/core/primitives/sparse_dense_matmul_grad_with_ftrl.py:275-334.
  """

  def __init__(self, learning_rate=0.01, learning_rate_power: float = -0.5, l1_regularization_strength: float = 0.0,
               l2_regularization_strength: float = 0.0, beta: float = 0.0, initial_accumulator_value: float = 0.1,
               initial_linear_value: float = 0.0, multiply_linear_by_learning_rate: bool = False):
    super().__init__(learning_rate)
    self.learning_rate_power = learning_rate_power
    self.l1_regularization_strength = l1_regularization_strength
    self.l2_regularization_strength = l2_regularization_strength
    self.beta = beta
    self.initial_accumulator_value = initial_accumulator_value
    self.initial_linear_value = initial_linear_value
    self.multiply_linear_by_learning_rate = multiply_linear_by_learning_rate

  def slot_variables_initializers(self):
    return FTRLSlotVariables(accumulator=initializers.constant(float(self.initial_accumulator_value)),
                             linear=initializers.constant(float(self.initial_linear_value)))

  def get_hyperparameters(self, step=None):
    return (self.get_learning_rate(step), _f32(self.learning_rate_power), _f32(self.l1_regularization_strength),
            _f32(self.l2_regularization_strength), _f32(self.beta))

  def __hash__(self) -> int:
    return hash((self.learning_rate, self.learning_rate_power, self.l1_regularization_strength,
                 self.l2_regularization_strength, self.beta, self.initial_accumulator_value,
                 self.initial_linear_value, self.multiply_linear_by_learning_rate))

  def short_name(self) -> str:
    return "ftrl"

  def get_optimizer_primitive(self):
    return _primitive("sparse_dense_matmul_grad_with_ftrl")


class LaPropOptimizerSpec(OptimizerSpec):
  """LaProp: RMS-normalised gradient, then momentum (https://arxiv.org/abs/2002.04839).

  Mirrors the reference's LaPropOptimizerSpec (lib/nn/embedding_spec.py:744-831): the decay rate of
  the second moment carries the bias correction, b2 (1 - b2^step) / (1 - b2^(step + 1)).
  """

  def __init__(self, learning_rate=0.001, b1: float = 0.9, b2: float = 0.95, eps: float = 1e-30,
               rms_clip_threshold: float | None = None, initial_slot_value: float = 0.0):
    super().__init__(learning_rate)
    self.b1 = b1
    self.b2 = b2
    self.eps = eps
    if rms_clip_threshold is not None:
      raise ValueError("rms_clip_threshold is not yet supported in LaProp optimizer.")
    self.initial_slot_value = initial_slot_value

  def slot_variables_initializers(self):
    return LaPropSlotVariables(mu=initializers.constant(float(self.initial_slot_value)),
                               nu=initializers.constant(float(self.initial_slot_value)))

  def get_decay_rate(self, step=None) -> np.ndarray:
    if step is None:
      return _f32(self.b2)
    step = np.asarray(step, dtype=np.float64)
    return _f32(self.b2 * (1.0 - np.power(self.b2, step)) / (1.0 - np.power(self.b2, step + 1.0)))

  def get_hyperparameters(self, step=None):
    return (self.get_learning_rate(step), _f32(self.b1), self.get_decay_rate(step), _f32(self.eps))

  def __hash__(self) -> int:
    return hash((self.learning_rate, self.b1, self.b2, self.eps, self.initial_slot_value))

  def short_name(self) -> str:
    return "laprop"

  def get_optimizer_primitive(self):
    return _primitive("sparse_dense_matmul_grad_with_laprop")


class F2AOptimizerSpec(OptimizerSpec):
  """Frequency-aware Adagrad: rows that are updated rarely get a larger step.

  multiplier = min((max(global_step, 1) / (local_step + 1))^rho, max_lr_multiplier).  Mirrors the
  reference's F2AOptimizerSpec (lib/nn/embedding_spec.py:833-917).
  """

  def __init__(self, learning_rate=0.01, rho: float = 0.5, initial_accumulator_value: float = 0.1,
               initial_local_step_value: float = 0.0, l1_regularization_strength: float = 0.0,
               l2_regularization_strength: float = 0.0, max_lr_multiplier: float = 1e6):
    super().__init__(learning_rate)
    self.rho = rho
    self.initial_accumulator_value = initial_accumulator_value
    self.initial_local_step_value = initial_local_step_value
    self.l1_regularization_strength = l1_regularization_strength
    self.l2_regularization_strength = l2_regularization_strength
    self.max_lr_multiplier = max_lr_multiplier

  def slot_variables_initializers(self):
    return F2ASlotVariables(accumulator=initializers.constant(float(self.initial_accumulator_value)),
                            local_step=initializers.constant(float(self.initial_local_step_value)))

  def get_hyperparameters(self, step=None):
    if step is None:
      step = 0
    return (self.get_learning_rate(step), _f32(self.rho), _f32(self.l1_regularization_strength),
            _f32(self.l2_regularization_strength), _f32(self.max_lr_multiplier), _f32(step))

  def __hash__(self) -> int:
    return hash((self.learning_rate, self.rho, self.initial_accumulator_value, self.initial_local_step_value,
                 self.l1_regularization_strength, self.l2_regularization_strength, self.max_lr_multiplier))

  def short_name(self) -> str:
    return "f2a"

  def get_optimizer_primitive(self):
    return _primitive("sparse_dense_matmul_grad_with_f2a")


@dataclasses.dataclass(eq=True, frozen=True)
class FeatureIdTransformation:
  """Where a feature's samples and ids land inside its stack."""

  row_offset: int = 0  # samples of the features stacked before this one
  col_offset: int = 0  # row_offset_in_shard * num_shards of the feature's table
  col_shift: int = 0  # shard rotation of the feature's table


@dataclasses.dataclass(eq=True, frozen=True, kw_only=True)
class TableSettingInStack:
  """Placement of one table inside the per-shard block of its stack."""

  stack_name: str
  padded_vocab_size: int  # multiple of 8 * num_shards
  padded_embedding_dim: int  # multiple of 8
  row_offset_in_shard: int = 0
  shard_rotation: int = 0  # id i lives on shard (i % num_shards + rotation) % num_shards


@dataclasses.dataclass(frozen=True, slots=True, kw_only=True)
class QuantizationConfig:
  min_value: float
  max_value: float
  num_buckets: int

  def __post_init__(self):
    if self.num_buckets < 2:
      raise ValueError("num_buckets must be ≥ 2.")
    if self.min_value >= self.max_value:
      raise ValueError("min_value must be < max_value.")

  def as_tuple(self) -> tuple[float, float, int]:
    return (self.min_value, self.max_value, self.num_buckets)


@dataclasses.dataclass(eq=True, frozen=True, kw_only=True)
class StackedTableSpec:
  """One lookup unit: several tables (or one) concatenated per shard."""

  stack_name: str
  stack_vocab_size: int
  stack_embedding_dim: int
  optimizer: OptimizerSpec
  combiner: str
  total_sample_count: int
  max_ids_per_partition: int = 256
  max_unique_ids_per_partition: int = 256
  activation_mem_bytes_limit: int = DEFAULT_ACTIVATION_MEM_BYTES_LIMIT
  suggested_coo_buffer_size_per_device: int | None = None
  quantization_config: QuantizationConfig | None = None

  def replace(self, **changes) -> "StackedTableSpec":
    return dataclasses.replace(self, **changes)


_AFTER_STACKING_OK = ("_stacked_table_spec", "_setting_in_stack", "stacked_table_spec", "setting_in_stack")
_FDO_PARAMS = ("max_ids_per_partition", "max_unique_ids_per_partition", "suggested_coo_buffer_size_per_device")


@dataclasses.dataclass(eq=True, unsafe_hash=True, kw_only=True)
class TableSpec:
  """One embedding table.  Frozen once it belongs to a stack."""

  name: str
  vocabulary_size: int
  embedding_dim: int
  initializer: CallableTableInitializer
  optimizer: OptimizerSpec
  combiner: str
  max_ids_per_partition: int = 256
  max_unique_ids_per_partition: int = 256
  suggested_coo_buffer_size_per_device: int | None = None
  quantization_config: QuantizationConfig | None = None
  _initialized: bool = dataclasses.field(init=False, default=False, compare=False)
  _stacked_table_spec: StackedTableSpec | None = dataclasses.field(default=None, compare=False)
  _setting_in_stack: TableSettingInStack | None = dataclasses.field(default=None, compare=False)

  def __setattr__(self, name: str, value: Any):
    if name not in _AFTER_STACKING_OK and self.__dict__.get("_initialized") and self.is_stacked():
      hint = (
          "If you are trying to update FDO parameters like 'max_ids_per_partition', use "
          "embedding.update_preprocessing_parameters() to update the StackedTableSpec instead."
          if name in _FDO_PARAMS else
          "If you need to modify non-FDO parameters for a stacked table, create a new table spec using "
          "`dataclasses.replace(table_spec, ...)` and feature spec using "
          "`dataclasses.replace(feature_spec, table_spec=new_table_spec)` and then re-prepare feature "
          "specs for training.")
      raise AttributeError(
          f"Cannot update parameter '{name}' on TableSpec '{self.name}' after it has been stacked. {hint}")
    object.__setattr__(self, name, value)

  def __post_init__(self):
    if self._setting_in_stack is None:
      self._setting_in_stack = TableSettingInStack(
          stack_name=self.name,
          padded_vocab_size=self.vocabulary_size,
          padded_embedding_dim=self.embedding_dim,
      )
    object.__setattr__(self, "_initialized", True)

  @property
  def setting_in_stack(self) -> TableSettingInStack:
    assert self._setting_in_stack is not None
    return self._setting_in_stack

  @setting_in_stack.setter
  def setting_in_stack(self, value: TableSettingInStack) -> None:
    self._setting_in_stack = value

  @property
  def stacked_table_spec(self) -> StackedTableSpec:
    assert self._stacked_table_spec is not None, f"Table {self.name} is not stacked."
    return self._stacked_table_spec

  @stacked_table_spec.setter
  def stacked_table_spec(self, value: StackedTableSpec) -> None:
    self._stacked_table_spec = value

  def is_stacked(self) -> bool:
    return self.__dict__.get("_stacked_table_spec") is not None


@dataclasses.dataclass(eq=True, kw_only=True)
class FeatureSpec:
  """One input feature: which table it reads and the batch shapes."""

  name: str
  table_spec: TableSpec
  input_shape: Sequence[int]  # [global_batch, valency]; valency may be omitted for ragged input
  output_shape: Sequence[int]  # [global_batch, embedding_dim]
  _id_transformation: FeatureIdTransformation | None = dataclasses.field(default=None, compare=False)

  def __hash__(self):
    return hash((self.name, self.table_spec, tuple(self.input_shape), tuple(self.output_shape)))

  @property
  def id_transformation(self) -> FeatureIdTransformation:
    assert self._id_transformation is not None, self.name
    return self._id_transformation

  @id_transformation.setter
  def id_transformation(self, value: FeatureIdTransformation) -> None:
    self._id_transformation = value
