"""Generates the committed golden fixtures (run where the reference checkout is mounted).

    python tests/golden/make_fixtures.py [--reference /path/to/jax-tpu-embedding]

1. preprocess_reference.npz - every call that the reference's own unit tests
   (jax_tpu_embedding/sparsecore/lib/core/tests/pybind_input_preprocessing_test.py) make to the
   preprocessing binding, recorded while those tests run against the CPU oracle.  A call is kept
   only if the whole reference test suite passes, i.e. the recorded outputs are the ones the
   reference's hand-written expectations accept.
2. lookup_known_answers.npz - the known-answer cases of the reference's primitive tests
   (lib/core/primitives/tests/sparse_dense_matmul_csr_test.py:30-90,343-404,499-556,
   sparse_dense_matmul_grad_with_sgd_test.py:100-163, sparse_dense_matmul_grad_with_adagrad_test.py:330-400):
   inputs restated from those files, expected values computed by the dense formulas the tests
   state, independently of the oracle's CSR walk.
3. optimizer_known_answers.npz - one weighted multi-hot batch updated by Adam (textbook form with
   bias-corrected moments) and by AdagradMomentum / FTRL / LaProp / F2A, in float64, from the
   formulas of the reference's primitive tests (cited at known_answer_optimizer_cases).
4. python_preprocessing_reference.npz - outputs of the reference's pure-Python single-feature
   preprocessing (lib/core/input_preprocessing.py, imported with numpy standing in for jax.numpy)
   on seeded random ragged batches: the four arrays in full, padding included.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (os.path.join(ROOT, "tests"), os.path.join(ROOT, "jax-tpu-embedding_b200"), ROOT, HERE):
  if p not in sys.path:
    sys.path.insert(0, p)

import fixture_io as fio  # noqa: E402


def record_reference_preprocessing(reference_root):
  import oracle_backend as ob
  import reference_harness as rh
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  rh.set_reference_root(reference_root)
  calls = []

  def recording_backend(features, feature_weights, feature_specs, local_device_count, global_device_count, **kw):
    features, feature_specs = list(features), list(feature_specs)
    weights = None if feature_weights is None else list(feature_weights)
    features = [np.array(f, copy=True) if isinstance(f, np.ndarray) and f.dtype != object else
                np.array([np.array(r) for r in f] + [None], dtype=object)[:-1] for f in features]
    entry = dict(features=features, weights=weights, specs=fio.specs_to_json(feature_specs),
                 local_device_count=int(local_device_count), global_device_count=int(global_device_count),
                 kwargs={k: (int(v) if not isinstance(v, bool) else v) for k, v in kw.items()
                         if k in ("num_sc_per_device", "sharding_strategy", "has_leading_dimension", "allow_id_dropping")})
    try:
      out = ob.oracle_preprocess(features, feature_weights, feature_specs, local_device_count, global_device_count, **kw)
    except Exception as e:  # pylint: disable=broad-except
      entry["raises"] = [type(e).__name__, str(e)]
      calls.append(entry)
      raise
    # The caller may reshape or overwrite what it receives: keep private copies.
    import copy
    entry["out"] = tuple({k: np.array(v) for k, v in d.items()} for d in out[:4]) + (out[4], copy.deepcopy(out[5]))
    calls.append(entry)
    return out

  original = pip.preprocess_sparse_dense_matmul_input
  try:
    module = rh.load_pybind_test_module(recording_backend)
    result = rh.run_cases(module)
  finally:
    pip.preprocess_sparse_dense_matmul_input = original
  problems = result.failures + result.errors
  if problems or result.testsRun < 30:
    raise SystemExit(f"reference tests did not pass on the oracle ({result.testsRun} run): {problems[:1]}")

  manifest, arrays = dict(source="pybind_input_preprocessing_test.py", tests_run=result.testsRun, calls=[]), {}
  for i, c in enumerate(calls):
    m = dict(specs=c["specs"], local_device_count=c["local_device_count"],
             global_device_count=c["global_device_count"], kwargs=c["kwargs"], features=[], raises=c.get("raises"))
    for j, f in enumerate(c["features"]):
      vals, lens, valency = fio.pack_rows(f)
      arrays[f"c{i}_f{j}_ids"], arrays[f"c{i}_f{j}_len"] = np.asarray(vals, np.int32), lens
      has_w = c["weights"] is not None and c["weights"][j] is not None
      if has_w:
        arrays[f"c{i}_f{j}_w"] = np.asarray(fio.pack_rows(c["weights"][j])[0], np.float32)
      m["features"].append(dict(valency=int(valency), weights=bool(has_w)))
    m["weights_given"] = c["weights"] is not None
    if "out" in c:
      rp, ids, sids, gains, _, stats = c["out"]
      m["stacks"] = sorted(rp)
      for name in rp:
        for key, d in (("rp", rp), ("ids", ids), ("sids", sids), ("gains", gains)):
          arrays[f"c{i}_{name}_{key}"] = np.asarray(d[name])
        arrays[f"c{i}_{name}_max_ids"] = np.asarray(stats.max_ids_per_partition[name])
        arrays[f"c{i}_{name}_max_unique"] = np.asarray(stats.max_unique_ids_per_partition[name])
        arrays[f"c{i}_{name}_required"] = np.asarray(stats.required_buffer_sizes[name])
        arrays[f"c{i}_{name}_dropped"] = np.asarray(stats.dropped_id_count[name])
    manifest["calls"].append(m)
  fio.save(os.path.join(HERE, "preprocess_reference.npz"), manifest, arrays)
  print(f"preprocess_reference.npz: {len(calls)} calls from {result.testsRun} reference tests")


def record_python_preprocessing(reference_root):
  """Runs the reference's pure-Python preprocessing on seeded random inputs and stores inputs and outputs."""
  import importlib.util
  import types

  # numpy stands in for jax.numpy; the module's own imports (constants, utils) resolve to this repository's package,
  # which mirrors them.
  saved = {k: sys.modules.get(k) for k in ("jax", "jax.numpy", "jax.sharding")}
  jax = types.ModuleType("jax")
  jnp = types.ModuleType("jax.numpy")
  jnp.asarray, jnp.ndarray, jnp.int32, jnp.float32 = np.asarray, np.ndarray, np.int32, np.float32
  sharding = types.ModuleType("jax.sharding")
  sharding.Mesh = object
  jax.numpy, jax.sharding = jnp, sharding
  sys.modules.update({"jax": jax, "jax.numpy": jnp, "jax.sharding": sharding})
  try:
    path = os.path.join(reference_root, "jax_tpu_embedding/sparsecore/lib/core/input_preprocessing.py")
    spec = importlib.util.spec_from_file_location("reference_python_preprocessing", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
  finally:
    for k, v in saved.items():
      if v is None:
        sys.modules.pop(k, None)
      else:
        sys.modules[k] = v

  class Mesh:
    def __init__(self, n):
      self.devices = list(range(n))

  rng = np.random.default_rng(20240611)
  manifest, arrays = dict(source="lib/core/input_preprocessing.py", cases=[]), {}
  for i in range(24):
    c, s = int(rng.choice([1, 2, 4])), int(rng.choice([1, 2, 4]))
    batch = s * int(rng.integers(1, 9))
    vocab = int(rng.choice([16, 64, 1000, 100000]))
    rows = [rng.integers(0, vocab, size=rng.integers(0, 7)).astype(np.int32) for _ in range(batch)]
    # Power-of-two weights: the reference sums the gains of duplicate ids in double, the kernels in float.
    weights = [rng.choice([0.5, 1.0, 2.0, 0.25], size=len(r)).astype(np.float32) for r in rows]
    rp, ids, sids, gains = ref.preprocess_sparse_dense_matmul_input(
        rows, weights, Mesh(c), max_ids_per_partition=64, max_unique_ids_per_partition=64, num_sc_per_device=s)
    manifest["cases"].append(dict(devices=c, num_sc_per_device=s, max_ids_per_partition=64,
                                  max_unique_ids_per_partition=64))
    arrays[f"p{i}_ids"] = np.concatenate(rows) if rows else np.zeros(0, np.int32)
    arrays[f"p{i}_w"] = np.concatenate(weights) if weights else np.zeros(0, np.float32)
    arrays[f"p{i}_len"] = np.asarray([len(r) for r in rows], np.int64)
    arrays[f"p{i}_rp"], arrays[f"p{i}_eids"] = np.asarray(rp, np.int32), np.asarray(ids, np.int32)
    arrays[f"p{i}_sids"], arrays[f"p{i}_gains"] = np.asarray(sids, np.int32), np.asarray(gains, np.float32)
  fio.save(os.path.join(HERE, "python_preprocessing_reference.npz"), manifest, arrays)
  print(f"python_preprocessing_reference.npz: {len(manifest['cases'])} cases")


def known_answer_lookup_cases():
  """Dense restatement of the reference's primitive tests; no CSR involved."""
  ids16 = np.array([5, 3, 9, 1, 6, 12, 0, 4, 15, 13, 11, 7, 8, 14, 2, 10], np.int32).reshape(16, 1)
  vocab, dim = 32, 8
  cases, arrays = [], {}

  def add(name, ids, weights, table, **extra):
    arrays[f"{name}_ids"], arrays[f"{name}_weights"], arrays[f"{name}_table"] = ids, weights, table
    for k, v in extra.items():
      arrays[f"{name}_{k}"] = np.asarray(v)
    cases.append(dict(name=name, keys=sorted(extra)))

  # Forward: table row i holds the value i, one id per sample -> activation = id.
  table = np.repeat(np.arange(vocab, dtype=np.float32)[:, None], dim, axis=1)
  add("forward_single_hot", ids16, np.ones((16, 1), np.float32), table,
      activations=table[ids16[:, 0]])
  # Forward, rank-1 table, every sample looks its id up twice -> 2 * (id + 1).
  ids2 = np.concatenate([np.concatenate([ids16, ids16], axis=1)] * 2, axis=0)
  table1 = (np.arange(vocab, dtype=np.float32) + 1.0).reshape(vocab, 1)
  add("forward_dim1_duplicates", ids2, np.ones(ids2.shape, np.float32), table1,
      activations=(2.0 * table1[ids2[:, 0]]))
  # SGD: gradient 0.01 everywhere, learning rate 0.01 -> touched rows move by -1e-4, then clip.
  for tag, lo, hi in (("", None, None), ("_clipped", 2.0, 12.5)):
    want = table.copy()
    rows = np.unique(ids16)
    want[rows] -= np.float32(1e-4)
    if lo is not None:
      want[rows] = np.clip(want[rows], lo, hi)
    add("sgd" + tag, ids16, np.ones((16, 1), np.float32), table, grad=np.full((16, dim), 0.01, np.float32),
        learning_rate=np.float32(0.01), clip=np.array([np.nan if lo is None else lo, np.nan if hi is None else hi], np.float32),
        table_out=want)
  # Adagrad: table row i holds i + 1, accumulator 0.002, learning rate 0.1, gradient 0.012, multi-hot with weights.
  rng = np.random.default_rng(1234)
  ids_mh = rng.integers(0, vocab, size=(16, 4)).astype(np.int32)
  w_mh = rng.choice([0.5, 1.0, 2.0], size=(16, 4)).astype(np.float32)
  table_p1 = table + 1.0
  act_grad = np.full((16, dim), 0.012, np.float32)
  g = np.zeros((vocab, dim), np.float32)
  for s in range(16):
    for j in range(4):
      g[ids_mh[s, j]] += w_mh[s, j] * act_grad[s]
  acc = np.full((vocab, dim), 0.002, np.float32)
  touched = np.zeros(vocab, bool)
  touched[np.unique(ids_mh)] = True
  acc_new = acc + g * g
  tab_new = table_p1 - (np.float32(0.1) * g) / np.sqrt(acc_new)
  add("adagrad_multi_hot", ids_mh, w_mh, table_p1, grad=act_grad, learning_rate=np.float32(0.1), accumulator=acc,
      clip=np.array([np.nan, np.nan], np.float32),
      table_out=np.where(touched[:, None], tab_new, table_p1), accumulator_out=np.where(touched[:, None], acc_new, acc))
  fio.save(os.path.join(HERE, "lookup_known_answers.npz"), dict(cases=cases, vocab=vocab), arrays)
  print(f"lookup_known_answers.npz: {len(cases)} cases")


def known_answer_optimizer_cases():
  """Known answers for Adam and the four two-slot optimizers, in float64, from the formulas that the
  reference's own tests state INDEPENDENTLY of the primitives' operand conventions:

  * Adam: the textbook form with bias-corrected m_hat, v_hat
    (primitives/tests/sparse_dense_matmul_grad_with_adam_test.py:403-411), while the primitive receives
    alpha_t and epsilon_hat (:540-542);
  * FTRL: sign / threshold form (..._ftrl_test.py:235-320);
  * AdagradMomentum (..._adagrad_momentum_test.py:274-318), LaProp (..._laprop_test.py:483-489),
    F2A (..._f2a_test.py:589-617).

  One multi-hot weighted batch; the table gradient is the dense definition sum_w w * activation_grad.
  """
  vocab, dim, batch = 32, 8, 16
  rng = np.random.default_rng(4321)
  ids = rng.integers(0, vocab, size=(batch, 4)).astype(np.int32)
  weights = rng.choice([0.5, 1.0, 2.0], size=(batch, 4)).astype(np.float32)
  table = rng.normal(0.0, 0.5, size=(vocab, dim)).astype(np.float32)
  act_grad = (rng.normal(size=(batch, dim)) * 0.05).astype(np.float32)
  slot_a = rng.uniform(0.05, 0.3, size=(vocab, dim)).astype(np.float32)   # accumulator / mu / momentum
  slot_b = rng.uniform(0.01, 0.2, size=(vocab, dim)).astype(np.float32)   # velocity / linear / nu / momentum
  steps = np.floor(rng.uniform(0.0, 5.0, size=(vocab, dim))).astype(np.float32)  # F2A local step
  g = np.zeros((vocab, dim), np.float64)
  for s in range(batch):
    for j in range(4):
      g[ids[s, j]] += float(weights[s, j]) * act_grad[s].astype(np.float64)
  touched = np.zeros(vocab, bool)
  touched[np.unique(ids)] = True
  w = table.astype(np.float64)
  a64, b64, st64 = slot_a.astype(np.float64), slot_b.astype(np.float64), steps.astype(np.float64)
  arrays = dict(ids=ids, weights=weights, table=table, grad=act_grad, slot_a=slot_a, slot_b=slot_b, steps=steps)
  cases = []

  def add(name, kind, hyper, flags, slots_in, outs):
    keep = lambda new, old: np.where(touched[:, None], new, old).astype(np.float32)
    olds = [w] + [arrays[k].astype(np.float64) for k in slots_in]
    for i, (new, old) in enumerate(zip(outs, olds)):
      arrays[f"{name}_out{i}"] = keep(new, old)
    cases.append(dict(name=name, kind=kind, hyper=[float(h) for h in hyper], flags=flags, slots=slots_in))

  # Adam, textbook: t is the number of steps taken before this one.
  for t in (0, 7):
    lr, b1, b2, eps = 1e-2, 0.9, 0.999, 1e-8
    m = b1 * a64 + (1 - b1) * g
    v = b2 * b64 + (1 - b2) * g * g
    m_hat, v_hat = m / (1 - b1 ** (t + 1)), v / (1 - b2 ** (t + 1))
    add(f"adam_step{t}", "adam", (lr, b1, b2, eps, t), {}, ["slot_a", "slot_b"],
        [w - lr * m_hat / (np.sqrt(v_hat) + eps), m, v])
  # Adagrad momentum.
  for tag, (lr, mom, beta2, eps, k, nesterov) in (("plain", (0.05, 0.9, 1.0, 1e-10, 2.0, False)),
                                                    ("nesterov_ema", (0.05, 0.8, 0.95, 1e-6, 3.0, True))):
    a_n = a64 + g * g if beta2 == 1.0 else beta2 * a64 + (1 - beta2) * g * g
    g_hat = (a_n + eps) ** (-1.0 / k) * g
    m_n = mom * b64 + g_hat
    delta = lr * (mom * m_n + g_hat) if nesterov else lr * m_n
    add(f"adagrad_momentum_{tag}", "adagrad_momentum", (lr, mom, beta2, eps, k), {"use_nesterov": nesterov},
        ["slot_a", "slot_b"], [w - delta, a_n, m_n])
  # FTRL.
  for tag, (lr, power, l1, l2, beta, mlr) in (("plain", (0.05, -0.5, 0.0, 0.0, 0.0, False)),
                                               ("regularised_mlr", (0.05, -0.5, 0.02, 0.01, 0.1, True)),
                                               ("l1_only", (0.05, -0.4, 0.05, 0.0, 0.0, False))):
    a_new = a64 + g * g
    p_old, p_new = a64 ** (-power), a_new ** (-power)  # the exponent is the negative of lr_power
    delta_p = p_new - p_old
    lin = b64 + lr * g - delta_p * w if mlr else b64 + g - (delta_p / lr) * w
    thr = lr * l1 if mlr else l1
    denom = p_new + 2 * lr * l2 + beta if mlr else (p_new + beta) / lr + 2 * l2
    w_new = np.where(np.abs(lin) > thr, (np.sign(lin) * thr - lin) / denom, 0.0)
    add(f"ftrl_{tag}", "ftrl", (lr, power, l1, l2, beta), {"multiply_linear_by_learning_rate": mlr},
        ["slot_a", "slot_b"], [w_new, a_new, lin])
  # LaProp.
  lr, b1, decay, eps = 0.01, 0.9, 0.73, 1e-12
  nu_new = decay * b64 + (1 - decay) * (g * g + eps)
  mu_new = b1 * a64 + np.sqrt(1 - b1 ** 2) * (g / np.sqrt(nu_new))
  add("laprop", "laprop", (lr, b1, decay, eps), {}, ["slot_a", "slot_b"], [w - lr * mu_new, mu_new, nu_new])
  # F2A.
  lr, rho, l1, l2, cap, gstep = 0.05, 0.5, 0.001, 0.002, 3.0, 40.0
  l_new = st64 + 1.0
  fa = np.minimum((max(gstep, 1.0) / l_new) ** rho, cap)
  a_new = a64 + g * g
  update = fa * g / np.sqrt(a_new) + l1 * np.sign(w) + l2 * w
  add("f2a", "f2a", (lr, rho, l1, l2, cap, gstep), {}, ["slot_a", "steps"], [w - lr * update, a_new, l_new])
  fio.save(os.path.join(HERE, "optimizer_known_answers.npz"), dict(cases=cases, vocab=vocab), arrays)
  print(f"optimizer_known_answers.npz: {len(cases)} cases")


if __name__ == "__main__":
  ap = argparse.ArgumentParser()
  ap.add_argument("--reference", default=os.environ.get("SC_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference")))
  args = ap.parse_args()
  known_answer_lookup_cases()
  known_answer_optimizer_cases()
  record_reference_preprocessing(args.reference)
  record_python_preprocessing(args.reference)
