"""numpy restatement of the SparseCore lookup and optimizer update (test infrastructure).

TEST INFRASTRUCTURE - NOT THE PRODUCT.  The device kernels of the reference are
closed libtpu custom calls (`SparseDenseMatmulOp`,
`SparseDenseMatmulGradOpWithOptimizerUpdate`); what they compute is pinned by the
CPU expected-value code of the reference's own tests, which this file restates:

* forward  - jax_tpu_embedding/sparsecore/lib/core/primitives/tests/
             sparse_dense_matmul_csr_test.py:343-404,499-556
* gradient - .../sparse_dense_matmul_grad_with_adagrad_test.py:356-367
             (`grad.at[cols].add(vals * activation_grad[rows])`)
* SGD      - .../sparse_dense_matmul_grad_with_sgd_test.py:149-163
* Adagrad  - .../sparse_dense_matmul_grad_with_adagrad_test.py:369-400 and the
             update body of sparse_dense_matmul_grad_with_adagrad.py:206-226
* Adam     - .../sparse_dense_matmul_grad_with_adam_test.py:403-437 and
             sparse_dense_matmul_grad_with_adam.py:296-341
* AdagradMomentum / FTRL / LaProp / F2A - the per-row update bodies of
             sparse_dense_matmul_grad_with_{adagrad_momentum,ftrl,laprop,f2a}.py (lines cited at
             each function), which are also the formulas of their tests' CPU expectations
             (tests/sparse_dense_matmul_grad_with_ftrl_test.py:235-320,
             ..._laprop_test.py:483-515, tolerance atol=1e-5 there)
* clipping - primitives/utils.py:24-59 (table only)

Everything is float32; sums run in buffer order (device, SparseCore, partition,
slot), which is ascending table row per sample and ascending sample per row.
Only the touched rows change ("lazy" update).

Parity status: pinned.  tests/test_golden.py checks forward, SGD and Adagrad against
tests/golden/lookup_known_answers.npz and Adam (textbook form with bias-corrected moments),
AdagradMomentum, FTRL, LaProp and F2A against tests/golden/optimizer_known_answers.npz; both files
hold float64 results of the formulas that the reference's primitive tests state, computed without
this module (tests/golden/make_fixtures.py).  One behaviour is unpinned in the reference: how
the device orders a non-linear optimizer when one row is hit from several source
SparseCores.  The contract here is: reduce every contribution first, apply once.
"""

from __future__ import annotations

import numpy as np

PADDING_VALUE = 2**31 - 1


def _round_up(v, m=8):
  return (v + m - 1) // m * m


def partition_ranges(row_pointers, num_sc_per_device, num_scs, coo_size):
  """Yields (local_sc, partition, begin, end) slot ranges of one device buffer."""
  rp = np.asarray(row_pointers).reshape(-1)
  r_per_sc = max(num_scs, 8)
  coo_per_sc = coo_size // num_sc_per_device
  for s in range(num_sc_per_device):
    for g in range(num_scs):
      begin = 0 if g == 0 else _round_up(int(rp[s * r_per_sc + g - 1]))
      end = int(rp[s * r_per_sc + g])
      if end > begin:
        yield s, g, s * coo_per_sc + begin, s * coo_per_sc + end


def forward(csr_per_device, shards, *, num_sc_per_device, device_batch_size):
  """Activations per device.

  csr_per_device: list over ALL devices of (row_pointers, embedding_ids,
    sample_ids, gains) 1-D arrays.
  shards: float32 [num_scs, rows_per_shard, D]; shard g holds rows
    {i : i % num_scs == g} of the stacked table at local row i // num_scs.
  """
  shards = np.asarray(shards, np.float32)
  num_scs = shards.shape[0]
  bsc = device_batch_size // num_sc_per_device
  out = []
  for rp, ids, sids, gains in csr_per_device:
    act = np.zeros((device_batch_size,) + shards.shape[2:], np.float32)
    for s, g, b, e in partition_ranges(rp, num_sc_per_device, num_scs, len(ids)):
      rows = shards[g][ids[b:e]]
      w = gains[b:e].astype(np.float32).reshape((-1,) + (1,) * (rows.ndim - 1))
      np.add.at(act, s * bsc + sids[b:e], w * rows)
    out.append(act)
  return out


def table_gradient(csr_per_device, act_grads, shard_shape, *, num_sc_per_device):
  """(G, touched): summed row gradients per shard and the touched-row mask."""
  num_scs = shard_shape[0]
  g_sum = np.zeros(shard_shape, np.float32)
  touched = np.zeros(shard_shape[:2], bool)
  for (rp, ids, sids, gains), grad in zip(csr_per_device, act_grads):
    grad = np.asarray(grad, np.float32)
    bsc = grad.shape[0] // num_sc_per_device
    for s, g, b, e in partition_ranges(rp, num_sc_per_device, num_scs, len(ids)):
      rows = grad[s * bsc + sids[b:e]]
      w = gains[b:e].astype(np.float32).reshape((-1,) + (1,) * (rows.ndim - 1))
      np.add.at(g_sum[g], ids[b:e], w * rows)
      touched[g][ids[b:e]] = True
  return g_sum, touched


def _clip(x, lo, hi):
  if lo is None and hi is None:
    return x
  return np.clip(x, lo, hi).astype(np.float32)


def apply_sgd(table, g, touched, lr, lo=None, hi=None):
  lr = np.float32(lr)
  new = _clip(table - lr * g, lo, hi)
  m = touched[..., None]
  return (np.where(m, new, table).astype(np.float32),)


def apply_adagrad(table, acc, g, touched, lr, lo=None, hi=None):
  lr = np.float32(lr)
  new_acc = acc + g * g
  with np.errstate(divide="ignore", invalid="ignore"):
    new = table - (lr * g) / np.sqrt(new_acc)
  new = _clip(new, lo, hi)
  m = touched[..., None]
  return (np.where(m, new, table).astype(np.float32),
          np.where(m, new_acc, acc).astype(np.float32))


def apply_adam(table, mom, vel, g, touched, alpha_t, beta_1, beta_2, eps_hat, lo=None, hi=None):
  alpha_t, beta_1, beta_2, eps_hat = (np.float32(x) for x in (alpha_t, beta_1, beta_2, eps_hat))
  one = np.float32(1.0)
  m_new = mom + (one - beta_1) * (g - mom)
  v_new = vel + (one - beta_2) * (g * g - vel)
  with np.errstate(divide="ignore", invalid="ignore"):
    new = table - (alpha_t * m_new) / (np.sqrt(v_new) + eps_hat)
  new = _clip(new, lo, hi)
  m = touched[..., None]
  return (np.where(m, new, table).astype(np.float32),
          np.where(m, m_new, mom).astype(np.float32),
          np.where(m, v_new, vel).astype(np.float32))


def _lazy(touched, new, old):
  return np.where(touched[..., None], new, old).astype(np.float32)


def apply_adagrad_momentum(table, acc, mom, g, touched, lr, momentum, beta2, eps, exponent, use_nesterov,
                           lo=None, hi=None):
  """sparse_dense_matmul_grad_with_adagrad_momentum.py:262-308 of the reference, on touched rows."""
  f = np.float32
  g2 = g * g
  acc_new = acc + g2 if f(beta2) == f(1.0) else f(beta2) * acc + (f(1.0) - f(beta2)) * g2
  scaled = np.power(acc_new + f(eps), f(-1.0) / f(exponent), dtype=np.float32) * g
  mom_new = f(momentum) * mom + scaled
  update = f(momentum) * mom_new + scaled if use_nesterov else mom_new
  new = _clip(table - f(lr) * update, lo, hi)
  return _lazy(touched, new, table), _lazy(touched, acc_new, acc), _lazy(touched, mom_new, mom)


def apply_ftrl(table, acc, linear, g, touched, lr, lr_power, l1, l2, beta, multiply_linear_by_learning_rate=False,
               lo=None, hi=None):
  """sparse_dense_matmul_grad_with_ftrl.py:275-334 of the reference, on touched rows."""
  f = np.float32
  lr, l1, l2, beta = f(lr), f(l1), f(l2), f(beta)
  with np.errstate(divide="ignore", invalid="ignore"):
    acc_new = acc + g * g
    p_old = np.power(acc, -f(lr_power), dtype=np.float32)
    p_new = np.power(acc_new, -f(lr_power), dtype=np.float32)
    delta_p = p_new - p_old
    if multiply_linear_by_learning_rate:
      linear_new = (linear + lr * g) - delta_p * table
      scale = lr
      denom = (p_new + f(2.0) * (lr * l2)) + beta
    else:
      linear_new = (linear + g) - (delta_p / lr) * table
      scale = f(1.0)
      denom = (p_new + beta) / lr + f(2.0) * l2
    l1s = l1 * scale
    numer = -linear_new if l1 == 0 else np.clip(linear_new, -l1s, l1s) - linear_new
    new = _clip((numer / denom).astype(np.float32), lo, hi)
  return _lazy(touched, new, table), _lazy(touched, acc_new, acc), _lazy(touched, linear_new, linear)


def apply_laprop(table, mu, nu, g, touched, lr, b1, decay_rate, eps, lo=None, hi=None):
  """sparse_dense_matmul_grad_with_laprop.py:294-335 of the reference, on touched rows."""
  f = np.float32
  with np.errstate(divide="ignore", invalid="ignore"):
    g2 = g * g + f(eps)
    nu_new = nu * f(decay_rate) + (f(1.0) - f(decay_rate)) * g2
    update = g / np.sqrt(nu_new)
    update = f(b1) * mu + np.sqrt(f(1.0) - f(b1) * f(b1), dtype=np.float32) * update
    new = _clip(table - f(lr) * update, lo, hi)
  return _lazy(touched, new, table), _lazy(touched, update, mu), _lazy(touched, nu_new, nu)


def apply_f2a(table, acc, local_step, g, touched, lr, rho, l1, l2, max_lr_multiplier, global_step, lo=None, hi=None):
  """sparse_dense_matmul_grad_with_f2a.py:257-285 of the reference, on touched rows."""
  f = np.float32
  step_new = local_step + f(1.0)
  ratio = np.maximum(f(global_step), f(1.0)) / step_new
  fa = np.minimum(np.power(ratio, f(rho), dtype=np.float32), f(max_lr_multiplier))
  acc_new = acc + g * g
  update = (g * fa) / np.sqrt(acc_new) + (f(l1) * np.sign(table) + f(l2) * table)
  new = _clip(table - f(lr) * update, lo, hi)
  return _lazy(touched, new, table), _lazy(touched, acc_new, acc), _lazy(touched, step_new, local_step)


def adam_hyperparameters(lr, beta_1, beta_2, eps, step):
  """embedding_spec.py:506-539 (AdamOptimizerSpec.get_hyperparameters), float32."""
  b1, b2 = np.float32(beta_1), np.float32(beta_2)
  b1t = np.power(b1, np.float32(step + 1), dtype=np.float32)
  b2t = np.power(b2, np.float32(step + 1), dtype=np.float32)
  c2 = np.sqrt(np.float32(1.0) - b2t)
  alpha_t = np.float32(lr) * c2 / (np.float32(1.0) - b1t)
  return np.float32(alpha_t), b1, b2, np.float32(np.float32(eps) * c2)


def shard_table(table, num_scs):
  """[V, D] -> [num_scs, V / num_scs, D] (row i -> shard i % num_scs, local row i // num_scs)."""
  table = np.asarray(table)
  return np.ascontiguousarray(
      table.reshape((-1, num_scs) + table.shape[1:]).swapaxes(0, 1))


def unshard_table(shards):
  shards = np.asarray(shards)
  return np.ascontiguousarray(shards.swapaxes(0, 1)).reshape((-1,) + shards.shape[2:])


def dense_reference(features, weights, combiner, table, act_grad=None):
  """Brute-force per-sample lookup straight from the raw inputs (float64).

  Used to cross-check the whole chain preprocessing -> forward against the
  definition of the combiners (docs: sum, mean = sum / sum(w), sqrtn = sum /
  sqrt(sum(w^2))).  Returns activations [B, D] (and the dense table gradient when
  act_grad is given).
  """
  table = np.asarray(table, np.float64)
  out = np.zeros((len(features), table.shape[1]))
  grad = np.zeros_like(table) if act_grad is not None else None
  for i, row in enumerate(features):
    row = np.asarray(row).reshape(-1)
    w = np.ones(len(row)) if weights is None else np.asarray(weights[i], np.float64).reshape(-1)
    if len(row) == 0:
      continue
    if combiner == "mean":
      w = w / w.sum()
    elif combiner == "sqrtn":
      w = w / np.sqrt((w * w).sum())
    out[i] = (w[:, None] * table[row]).sum(0)
    if grad is not None:
      np.add.at(grad, row, w[:, None] * np.asarray(act_grad[i], np.float64)[None, :])
  return (out, grad) if grad is not None else out
