"""Benchmark of the SparseCore hot path on B200: forward + fused optimizer backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5|c1] [--impl reference]

Prints ONE JSON line.  `value` is samples/s of lookup + update with the preprocessed batch
resident in HBM; `e2e` adds the host->device copy of the raw ids, GPU preprocessing and a
device->host read of a checksum of the activations, all through the public Python API.
`roofline` is the fused backward kernel (algorithmic bytes / CUDA-event time / measured HBM
peak); `preprocess` times the GPU input preprocessing alone; `phases_ms` splits a step into the
library's stages; `cpu_baseline` is the CPU oracle (C preprocessing + torch-CPU lookup/update) on
the same batch with compacted tables.  With the default workload the line also carries a `configs`
block: the other benchmark configurations run for a few steps each, with forward / backward
roofline fractions and, on one GPU, a parity check of the full-size batch against the CPU oracle.
`--impl reference` runs only the CPU arm.

Workloads are seeded synthetic configurations (shapes and id distributions of the published
benchmark configurations); no dataset is involved.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "jax-tpu-embedding_b200")):
  if _p not in sys.path:
    sys.path.insert(0, _p)

L2_BYTES = 126 * 1024 * 1024
NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool
# DRAM traffic of the backward kernels per launch (dram__bytes_read.sum + dram__bytes_write.sum of ncu, update +
# group + fix-up kernels) divided by the algorithmic bytes of the same launch, from captures of cases small enough for
# ncu's replay passes (vocabularies scaled to 0.05 for c2 and c3, 0.25 for c5; traffic and algorithmic bytes grow with
# the same quantities: lookups, distinct rows, batch).  None: no capture (c4 holds 102 GB on the device).
TRAFFIC_RATIO = {"c2": 1.02, "c3": 0.94, "c5": 0.99, "c4": None, "c1": None}


# --------------------------------------------------------------------------------- workloads


def zipf_ids(rng, vocab, size, a):
  """Bounded Zipf, P(k) ~ (k+1)^-a over [0, vocab): inverse CDF on a float64 cumulative sum."""
  cdf = np.cumsum(np.arange(1, vocab + 1, dtype=np.float64) ** (-a))
  u = rng.random(size) * cdf[-1]
  return np.minimum(np.searchsorted(cdf, u, side="left"), vocab - 1).astype(np.int32)


def workload(name, scale=1.0):
  """Returns dict(tables=[dict(vocab, dim, features=[...])], batch, combiner, optimizer, weights, stack)."""
  if name == "c1":
    return dict(seed=101, batch=64, combiner="sum", optimizer="sgd", weights=False, stack=False,
                tables=[dict(vocab=4096, dim=16, feats=[dict(kind="ragged", lo=1, hi=8, dist="uniform")])])
  if name == "c2":
    rng = np.random.default_rng(202)
    vocabs = np.round(10 ** rng.uniform(3, np.log10(4e7), size=26)).astype(np.int64)
    if scale != 1.0:
      vocabs = np.maximum(1000, (vocabs * scale).astype(np.int64))
    return dict(seed=202, batch=65536, combiner="sum", optimizer="adagrad", weights=False, stack=False,
                tables=[dict(vocab=int(v), dim=128, feats=[dict(kind="dense", valency=1, dist="zipf", a=1.05)])
                        for v in vocabs])
  if name == "c3":
    return dict(seed=303, batch=16384, combiner="sqrtn", optimizer="adagrad", weights=True, stack=False,
                tables=[dict(vocab=int(1e7 * scale), dim=64,
                             feats=[dict(kind="ragged", poisson=20, lo=1, hi=64, dist="zipf", a=1.1)])
                        for _ in range(8)])
  if name == "c4":  # per-GPU batch 16384: at 8 GPUs this is the 131072-sample, 1e8-row configuration
    return dict(seed=404, batch=16384, combiner="mean", optimizer="adagrad", weights=False, stack=False,
                tables=[dict(vocab=int(1e8 * scale), dim=128, feats=[dict(kind="ragged", lo=1, hi=32, dist="zipf", a=1.05)])])
  if name == "c5":
    return dict(seed=505, batch=32768, combiner="mean", optimizer="adam", weights=False, stack=True,
                tables=[dict(vocab=int(1e5 * scale), dim=32, feats=[dict(kind="ragged", lo=1, hi=16, dist="uniform")])
                        for _ in range(100)])
  raise ValueError(name)


def describe(name, wl, batch):
  return (f"{name}: {len(wl['tables'])} tables dim {wl['tables'][0]['dim']}, batch {batch}, combiner "
          f"{wl['combiner']}, optimizer {wl['optimizer']}")


def build_specs(wl, global_device_count=1, num_sc=1, global_batch=None):
  from jax_tpu_embedding.sparsecore.lib.nn import embedding, embedding_spec, initializers, table_stacking

  if wl["optimizer"] == "sgd":
    opt = embedding_spec.SGDOptimizerSpec(learning_rate=0.01)
  elif wl["optimizer"] == "adagrad":
    opt = embedding_spec.AdagradOptimizerSpec(learning_rate=0.01, initial_accumulator_value=0.1)
  else:
    opt = embedding_spec.AdamOptimizerSpec(learning_rate=1e-3, beta_1=0.9, beta_2=0.999)
  specs = []
  for ti, t in enumerate(wl["tables"]):
    ts = embedding_spec.TableSpec(name=f"t{ti:03d}", vocabulary_size=t["vocab"], embedding_dim=t["dim"],
                                  initializer=initializers.normal(0.01), optimizer=opt, combiner=wl["combiner"],
                                  max_ids_per_partition=1 << 24, max_unique_ids_per_partition=1 << 24)
    for fi, f in enumerate(t["feats"]):
      gb = global_batch or wl["batch"]
      shape = [gb, f["valency"]] if f["kind"] == "dense" else [gb]
      specs.append(embedding_spec.FeatureSpec(name=f"f{ti:03d}_{fi}", table_spec=ts, input_shape=shape,
                                              output_shape=[gb, t["dim"]]))
  if wl["stack"]:
    big = lambda n, b: 1 << 24
    table_stacking.stack_tables(specs, [f"t{i:03d}" for i in range(len(wl["tables"]))], global_device_count, num_sc,
                                stack_to_max_ids_per_partition=big, stack_to_max_unique_ids_per_partition=big,
                                activation_mem_bytes_limit=1 << 50, stack_name="stack")
  else:
    embedding.prepare_feature_specs_for_training(specs, global_device_count, num_sc)
  return specs


def build_inputs(wl, specs, rank=0):
  """Raw host inputs of one rank: one leaf per feature (dense int32 [B, v] or RaggedInput), optional weights."""
  from jax_tpu_embedding.sparsecore.lib.nn import embedding

  feats, weights = [], []
  fi = 0
  for ti, t in enumerate(wl["tables"]):
    for f in t["feats"]:
      rng = np.random.default_rng([wl["seed"], 2, fi, rank])
      lrng = np.random.default_rng([wl["seed"], 3, fi, rank])
      wrng = np.random.default_rng([wl["seed"], 4, fi, rank])
      b = wl["batch"]
      draw = (lambda n: zipf_ids(rng, t["vocab"], n, f["a"])) if f["dist"] == "zipf" else (
          lambda n: rng.integers(0, t["vocab"], size=n).astype(np.int32))
      if f["kind"] == "dense":
        feats.append(draw(b * f["valency"]).reshape(b, f["valency"]))
        weights.append(wrng.uniform(0.5, 1.5, size=(b, f["valency"])).astype(np.float32))
      else:
        if "poisson" in f:
          lens = np.clip(lrng.poisson(f["poisson"], size=b), f["lo"], f["hi"])
        else:
          lens = lrng.integers(f["lo"], f["hi"] + 1, size=b)
        splits = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        vals = draw(int(splits[-1]))
        w = wrng.uniform(0.5, 1.5, size=int(splits[-1])).astype(np.float32) if wl["weights"] else None
        feats.append(embedding.RaggedInput(vals, splits, w))
        weights.append(None)
      fi += 1
  use_w = wl["weights"] and all(not isinstance(f, embedding.RaggedInput) for f in feats)
  return feats, (weights if use_w else None)


# --------------------------------------------------------------------------------- helpers


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

  QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, device_index):
    self.device_index = device_index
    self.proc = None
    self.path = f"/tmp/sc_clocks_{os.getpid()}.csv"

  def start(self):
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
           "-i", str(self.device_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
    except OSError:
      self.proc = None

  def stop(self):
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
    time.sleep(0.15)
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    try:
      for line in open(self.path):
        parts = [p.strip() for p in line.split(",")]
        if len(parts) < 9:
          continue
        try:
          sm.append(float(parts[1]))
          mx.append(float(parts[2]))
        except ValueError:
          continue
        for n, v in zip(names, parts[5:9]):
          if v.lower().startswith("active"):
            reasons.add(n)
      os.remove(self.path)
    except OSError:
      pass
    return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak_gbs():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  try:
    return float(json.load(open(path))["hbm_gbs"]), "measured"
  except Exception:  # pylint: disable=broad-except
    return 6650.0, "fallback"


def table_stats(pre, name, world=1, rank=0):
  """nnz (entries after dedup), unique rows, and unique rows of the other ranks' shards, of one
  stacked table, from this rank's CSR on device."""
  import torch

  rp = pre.lhs_row_pointers[name].cpu().numpy()
  ids = pre.lhs_embedding_ids[name]
  n = u = remote = 0
  for g in range(world):
    begin = 0 if g == 0 else (int(rp[g - 1]) + 7) // 8 * 8
    end = int(rp[g])
    n += end - begin
    ug = int(torch.unique_consecutive(ids[begin:end]).numel())
    u += ug
    if g != rank:
      remote += ug
  return n, u, remote


def host_rows(feats, weights, weighted):
  """Host inputs in the form the CPU oracle takes: dense arrays or object arrays of rows."""
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  np_feats, np_weights = [], ([] if weighted else None)
  for f in feats:
    if isinstance(f, pip.RaggedInput):
      rows = np.empty(len(f.row_splits) - 1, dtype=object)
      wrows = np.empty(len(rows), dtype=object)
      for i in range(len(rows)):
        rows[i] = f.values[f.row_splits[i]:f.row_splits[i + 1]]
        if f.weights is not None:
          wrows[i] = f.weights[f.row_splits[i]:f.row_splits[i + 1]]
      np_feats.append(rows)
      if np_weights is not None:
        np_weights.append(wrows)
    else:
      np_feats.append(f)
      if np_weights is not None:
        np_weights.append(weights[len(np_feats) - 1])
  return np_feats, np_weights


# --------------------------------------------------------------------------------- CPU arm


def cpu_arm(wl, specs, feats, weights, steps=1, warmup=0, threads=None):
  """CPU baseline: C oracle preprocessing (threaded) + torch-CPU lookup and Adagrad/Adam/SGD update.

  Tables are compacted to the rows the batch touches so that the sample needs no 100 GB host
  allocation; the number of lookups, unique rows and bytes moved per row are unchanged.
  """
  import torch
  sys.path.insert(0, os.path.join(ROOT, "tests"))
  import oracle_backend as ob
  from jax_tpu_embedding.sparsecore.lib.nn import embedding

  cores = len(os.sched_getaffinity(0))
  threads = threads or cores
  torch.set_num_threads(threads)
  np_feats, np_weights = host_rows(feats, weights, wl["weights"])
  stacks = {}
  times = []
  # Set-up, not part of the timed step: size the buffers from observed statistics (the reference's
  # FDO recipe) and compact row ids to an index among the touched rows.
  if any(f.table_spec.stacked_table_spec.suggested_coo_buffer_size_per_device is None for f in specs):
    *_, st0 = ob.oracle_preprocess(np_feats, np_weights, specs, 1, 1, num_sc_per_device=1, num_threads=threads,
                                   allow_id_dropping=True)
    embedding.update_preprocessing_parameters(specs, embedding.SparseDenseMatmulInputStats.from_cc(st0), 1)
  rp, ids, sids, gains, _, _ = ob.oracle_preprocess(np_feats, np_weights, specs, 1, 1, num_sc_per_device=1,
                                                    num_threads=threads)
  for name in rp:
    n = int(rp[name][0])
    uniq, inv = torch.unique(torch.from_numpy(ids[name][:n].astype(np.int64)), return_inverse=True)
    spec = next(f.table_spec.stacked_table_spec for f in specs if f.table_spec.stacked_table_spec.stack_name == name)
    dim, bdev = spec.stack_embedding_dim, spec.total_sample_count
    gen = torch.Generator().manual_seed(1)
    stacks[name] = dict(table=torch.randn(len(uniq), dim, generator=gen) * 0.01, inv=inv,
                        s0=torch.full((len(uniq), dim), 0.1), s1=torch.zeros(len(uniq), dim),
                        grad=torch.randn(bdev, dim, generator=gen) * 0.01, bdev=bdev, dim=dim)
  for it in range(warmup + steps):
    t0 = time.perf_counter()
    rp, ids, sids, gains, _, _ = ob.oracle_preprocess(np_feats, np_weights, specs, 1, 1, num_sc_per_device=1,
                                                      num_threads=threads)
    t1 = time.perf_counter()
    for name in rp:
      n = int(rp[name][0])
      s = torch.from_numpy(sids[name][:n].astype(np.int64))
      g = torch.from_numpy(gains[name][:n])
      st = stacks[name]
      inv = st["inv"]
      # forward: act[s] += gain * table[row]
      act = torch.zeros(st["bdev"], st["dim"])
      act.index_add_(0, s, st["table"].index_select(0, inv) * g[:, None])
      # backward: G[row] += gain * grad[s]; one optimizer application per touched row
      gsum = torch.zeros_like(st["table"])
      gsum.index_add_(0, inv, st["grad"].index_select(0, s) * g[:, None])
      if wl["optimizer"] == "sgd":
        st["table"].sub_(0.01 * gsum)
      elif wl["optimizer"] == "adagrad":
        st["s0"].add_(gsum * gsum)
        st["table"].sub_(0.01 * gsum / st["s0"].sqrt())
      else:
        st["s0"].add_(0.1 * (gsum - st["s0"]))
        st["s1"].add_(0.001 * (gsum * gsum - st["s1"]))
        st["table"].sub_(1e-3 * st["s0"] / (st["s1"].sqrt() + 1e-8))
    t2 = time.perf_counter()
    if it >= warmup:
      times.append((t2 - t0, t1 - t0))
  total = float(np.mean([t[0] for t in times]))
  pre = float(np.mean([t[1] for t in times]))
  return dict(samples_per_s=wl["batch"] / total, ms_per_step=total * 1e3, preprocess_ms=pre * 1e3, cores=threads)


# --------------------------------------------------------------------------------- one workload on the GPU


class Run:
  """One workload set up on this rank: specs, host inputs, tables, the preprocessed batch and gradients."""

  def __init__(self, name, wl, world, rank, global_batch):
    import torch
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    self.name, self.wl, self.world, self.rank = name, wl, world, rank
    self.specs = build_specs(wl, global_device_count=world, global_batch=global_batch)
    self.feats, self.weights = build_inputs(wl, self.specs, rank)
    table_specs = list({f.table_spec.name: f.table_spec for f in self.specs}.values())
    layout = embedding.DeviceLayout(world, 1 if world > 1 else None, rank)
    self.variables = embedding.init_embedding_variables(1234 + rank, table_specs, layout, num_sparsecore_per_device=1)
    self.table_bytes = sum(v.table.numel() * 4 * (1 + len(v.slot)) for v in self.variables.values())
    # FDO pass (the reference's own recipe): observe limits once, then size the buffers exactly.
    _, stats = embedding.preprocess_sparse_dense_matmul_input(self.feats, self.weights, self.specs, 1, world,
                                                              num_sc_per_device=1, allow_id_dropping=True)
    if world > 1:  # all ranks must agree on limits and buffer sizes
      for d in (stats.max_ids_per_partition, stats.max_unique_ids_per_partition, stats.required_buffer_size_per_sc):
        for k in sorted(d):
          t = torch.from_numpy(np.ascontiguousarray(d[k])).cuda()
          torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
          d[k] = t.cpu().numpy()
    embedding.update_preprocessing_parameters(self.specs, stats, 1)
    self.pre, self.stats = embedding.preprocess_sparse_dense_matmul_input(self.feats, self.weights, self.specs, 1, world,
                                                                          num_sc_per_device=1)
    self.stacked = embedding.get_stacked_table_specs(self.specs)
    gen = torch.Generator(device="cuda").manual_seed(5 + rank)
    self.grads = [torch.randn((wl["batch"], f.output_shape[-1]), generator=gen, device="cuda") * 1e-2 for f in self.specs]
    self.nnz_in = sum(int(np.prod(f.shape)) if isinstance(f, np.ndarray) else len(f.values) for f in self.feats)

  def lookup(self, unstack=True):
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    return embedding.tpu_sparse_dense_matmul(self.pre, self.variables, self.specs, global_device_count=self.world,
                                             num_sc_per_device=1, perform_unstacking=unstack)

  def update(self, grads=None, stacking=True):
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    embedding.tpu_sparse_dense_matmul_grad(self.grads if grads is None else grads, self.pre, self.variables, self.specs,
                                           global_device_count=self.world, num_sc_per_device=1, step=0,
                                           perform_stacking=stacking)

  def step(self):
    acts = self.lookup()
    self.update()
    return acts

  def barrier(self):
    import torch

    if self.world > 1:
      torch.distributed.barrier()
    torch.cuda.synchronize()

  def max_over_ranks(self, value):
    import torch

    if self.world == 1:
      return value
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())

  # ---- measurements

  def timed_steps(self, steps):
    """ms per step over exactly `steps` steps: CUDA events, barrier + synchronize on both sides, max over ranks."""
    import torch
    from jax_tpu_embedding.sparsecore import _native

    self.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = _native.lib().sc_launch_count()
    ev0.record()
    for _ in range(steps):
      self.step()
    ev1.record()
    launches = int(_native.lib().sc_launch_count() - launches0)
    self.barrier()
    return self.max_over_ranks(ev0.elapsed_time(ev1) / steps), launches

  def operator_rooflines(self, reps, peak):
    """Forward and backward operators timed on their own (stacked operands, no per-feature views)."""
    import torch
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    bwd_bytes = fwd_bytes = remote_row_bytes = 0
    nnz = uniq = 0
    for name, spec in self.stacked.items():
      n, u, remote = table_stats(self.pre, name, self.world, self.rank)
      d, bdev = spec.stack_embedding_dim, spec.total_sample_count // self.world
      slots = spec.optimizer.slot_variables_count()
      nnz += n
      uniq += u
      remote_row_bytes += remote * 4 * d
      bwd_bytes += bdev * 4 * d + n * 12 + 8 * 4 + u * 4 * d * (1 + slots) * 2
      fwd_bytes += u * 4 * d + n * 12 + 8 * 4 + bdev * 4 * d
    stacked_grads = embedding.stack_embedding_gradients(self.grads, self.specs, 1, self.world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = {}
    for key, fn in (("backward", lambda: self.update(stacked_grads, stacking=False)),
                    ("forward", lambda: self.lookup(unstack=False))):
      for _ in range(3):  # warm-up of this call signature (descriptor cache, workspaces)
        fn()
      self.barrier()
      e0.record()
      for _ in range(reps):
        fn()
      e1.record()
      torch.cuda.synchronize()
      ms = self.max_over_ranks(e0.elapsed_time(e1) / reps)
      nbytes = bwd_bytes if key == "backward" else fwd_bytes
      out[key] = {"algorithmic_bytes": int(nbytes), "ms": ms, "achieved": nbytes / (ms * 1e-3) / 1e9,
                  "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
    out["nnz"], out["unique_rows"], out["remote_row_bytes"] = int(nnz), int(uniq), int(remote_row_bytes)
    return out

  def device_inputs(self):
    """Raw inputs resident on the device, in the forms the preprocessing accepts without a host copy."""
    import torch
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    dev = []
    for f in self.feats:
      if isinstance(f, np.ndarray):
        dev.append(torch.from_numpy(f).cuda())
      else:
        dev.append(embedding.RaggedInput(torch.from_numpy(f.values).cuda(), f.row_splits,
                                         None if f.weights is None else torch.from_numpy(f.weights).cuda()))
    dev_w = None if self.weights is None else [torch.from_numpy(w).cuda() for w in self.weights]
    return dev, dev_w

  def preprocess_block(self, reps, peak):
    """GPU input preprocessing alone (raw ids already on the device): time, ids/s and fraction of the HBM peak on
    the bytes that must move (ids, weights and row offsets read once; buffers written once)."""
    import torch
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    dev, dev_w = self.device_inputs()
    run = lambda: embedding.preprocess_sparse_dense_matmul_input(dev, dev_w, self.specs, 1, self.world, num_sc_per_device=1)
    for _ in range(2):
      run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
      run()
    e1.record()
    torch.cuda.synchronize()
    ms = self.max_over_ranks(e0.elapsed_time(e1) / reps)
    from jax_tpu_embedding.sparsecore import _native

    _native.phase_timing(True)
    for _ in range(reps):
      run()
    torch.cuda.synchronize()
    stages = {k: v[0] / reps for k, v in _native.phase_report().items()}
    _native.phase_timing(False)
    rows = sum(f.shape[0] if isinstance(f, np.ndarray) else len(f.row_splits) - 1 for f in self.feats)
    written = sum(table_stats(self.pre, name, self.world, self.rank)[0] for name in self.stacked)
    weighted = self.wl["weights"]
    nbytes = self.nnz_in * (4 + (4 if weighted else 0)) + rows * 4 + written * 12 + len(self.stacked) * 8 * 4
    return {"ms": ms, "ids_per_s": self.nnz_in * self.world / (ms * 1e-3), "algorithmic_bytes": int(nbytes),
            "achieved": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "stages_ms": stages,
            "includes": "all kernels of one call and its read of the statistics block (one synchronisation); "
                        "stages_ms: device time of the call's stages (CUDA events)"}

  def phases(self, reps):
    """Stage times per step (ms) from the library's CUDA events plus the barriers of the sharded step."""
    import torch
    from jax_tpu_embedding.sparsecore import _native, distributed

    self.barrier()
    _native.phase_timing(True)
    distributed.time_barriers(True)
    for _ in range(reps):
      self.step()
    torch.cuda.synchronize()
    out = {k: self.max_over_ranks(ms / reps) for k, (ms, _) in sorted(_native.phase_report().items())}
    for k, ms in sorted(distributed.barrier_times().items()):
      out[k] = self.max_over_ranks(ms / reps)
    _native.phase_timing(False)
    distributed.time_barriers(False)
    return out

  def parity(self):
    """Full-size check of this batch against the CPU oracle (one GPU, one shard).  Preprocessing: bit-exact over
    the written region.  Lookup and update: the touched rows, against float64 sums over the same CSR; the error
    is reported relative to the largest magnitude of each array and must stay below 1e-5."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_backend as ob

    if self.world != 1:
      return {"status": "not run: the check gathers whole tables and runs on one GPU only"}
    t0 = time.perf_counter()
    np_feats, np_weights = host_rows(self.feats, self.weights, self.wl["weights"])
    want = ob.oracle_preprocess(np_feats, np_weights, self.specs, 1, 1, num_sc_per_device=1,
                                num_threads=len(os.sched_getaffinity(0)))
    worst, per_array, ill_fraction = 0.0, {}, 0.0
    try:
      for name in self.stacked:
        got = [d[name].cpu().numpy() for d in self.pre.sparse_dense_matmul_input]
        ob.written_region_equal(got[0], want[0][name], got[1:], [want[i][name] for i in (1, 2, 3)], 1)
    except AssertionError as e:
      return {"status": "FAILED", "where": "preprocessing", "detail": str(e)[:300]}
    stacked_acts = self.lookup(unstack=False)
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    stacked_grads = embedding.stack_embedding_gradients(self.grads, self.specs, 1, 1)
    before = {}
    for name, spec in self.stacked.items():
      n = int(want[0][name][0])
      ids = self.pre.lhs_embedding_ids[name][:n].long()
      uniq, inv = torch.unique(ids, return_inverse=True)
      v = self.variables[name]
      before[name] = (uniq, inv.cpu(), v.table[uniq].cpu().double(), [s[uniq].cpu().double() for s in v.slot])
    self.update(stacked_grads, stacking=False)
    torch.cuda.synchronize()
    chunk = 1 << 22
    for name, spec in self.stacked.items():
      uniq, inv, tab0, slots0 = before[name]
      n = inv.numel()
      sids = torch.from_numpy(want[2][name][:n].astype(np.int64))
      gains = torch.from_numpy(want[3][name][:n]).double()
      act = torch.zeros(tuple(stacked_acts[name].shape), dtype=torch.float64)
      gsum = torch.zeros_like(tab0)
      gabs = torch.zeros_like(tab0)  # sum of the magnitudes of the terms: conditioning of gsum
      grad = stacked_grads[name].cpu().double()
      for b in range(0, n, chunk):
        sl = slice(b, min(n, b + chunk))
        act.index_add_(0, sids[sl], tab0.index_select(0, inv[sl]) * gains[sl, None])
        terms = grad.index_select(0, sids[sl]) * gains[sl, None]
        gsum.index_add_(0, inv[sl], terms)
        gabs.index_add_(0, inv[sl], terms.abs())
      hyper = [float(np.float32(h)) for h in spec.optimizer.get_hyperparameters(0)]
      kind = spec.optimizer.short_name()
      if kind == "sgd":
        want_rows = [tab0 - hyper[0] * gsum]
      elif kind == "adagrad":
        acc = slots0[0] + gsum * gsum
        want_rows = [tab0 - hyper[0] * gsum / acc.sqrt(), acc]
      else:
        alpha_t, b1, b2, eps_hat = hyper
        m = slots0[0] + (1 - b1) * (gsum - slots0[0])
        vel = slots0[1] + (1 - b2) * (gsum * gsum - slots0[1])
        want_rows = [tab0 - alpha_t * m / (vel.sqrt() + eps_hat), m, vel]
      v = self.variables[name]
      got_rows = [v.table[uniq].cpu().double()] + [s[uniq].cpu().double() for s in v.slot]
      pairs = [(stacked_acts[name].cpu().double(), act)] + list(zip(got_rows, want_rows))
      for label, (got, ref) in zip(("activations", "table", "slot0", "slot1"), pairs):
        scale = float(ref.abs().max()) or 1.0
        diff = (got - ref).abs()
        if kind == "adam" and label == "table":
          # Adam steps by m / sqrt(v), of size ~alpha_t whatever |g| is: where the gradient terms of an element
          # cancel to below 1e-3 of their magnitudes, the float32 rounding of that sum - not the kernel - decides
          # the step.  Those elements are checked through momentum and velocity only.
          ill = gsum.abs() < 1e-3 * gabs
          ill_fraction = max(ill_fraction, float(ill.double().mean()))
          diff = torch.where(ill, torch.zeros_like(diff), diff)
        err = float(diff.max()) / scale
        per_array[label] = max(per_array.get(label, 0.0), err)
        worst = max(worst, err)
    status = "ok" if worst <= 1e-5 else "FAILED"
    return {"status": status, "preprocessing": "bit-exact with the oracle over the written region",
            "lookup_update_max_err": worst, "max_err_per_array": per_array, "tolerance": 1e-5,
            "ill_conditioned_fraction": ill_fraction,
            "seconds": round(time.perf_counter() - t0, 1),
            "checked": "activations of every sample; table and slot rows of every touched row"}

  def e2e(self, steps):
    """Wall-clock step through the public API with HOST inputs: copy of the raw ids from pinned memory, GPU
    preprocessing, lookup, read-back of a checksum of the activations, update; copy + preprocessing of batch
    i + 1 run on a second stream while batch i is looked up and updated."""
    import torch
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    feats, weights, specs, world = self.feats, self.weights, self.specs, self.world
    pinned = []
    for f in feats:
      if isinstance(f, np.ndarray):
        pinned.append(torch.from_numpy(f).pin_memory())
      else:
        pinned.append(embedding.RaggedInput(torch.from_numpy(f.values).pin_memory(), f.row_splits,
                                            None if f.weights is None else torch.from_numpy(f.weights).pin_memory()))
    h2d = sum((p.numel() * 4) if isinstance(p, torch.Tensor) else (p.values.numel() * 4 + len(p.row_splits) * 4 +
                                                                   (0 if p.weights is None else p.weights.numel() * 4))
              for p in pinned)
    pinned_w = None
    if weights is not None:
      pinned_w = [torch.from_numpy(w).pin_memory() for w in weights]
      h2d += sum(w.numel() * 4 for w in pinned_w)
    # Dense id matrices travel as ONE pinned buffer and one copy per step; the features are views of it.
    dense_all = None
    if all(isinstance(p, torch.Tensor) for p in pinned) and pinned_w is None:
      shapes = [tuple(p.shape) for p in pinned]
      sizes = [p.numel() for p in pinned]
      dense_all = torch.cat([p.reshape(-1) for p in pinned]).pin_memory()
    main_stream = torch.cuda.current_stream()
    # The input pipeline's stream has the higher priority: its many short kernels take the SM slots that free up
    # while the long lookup / update kernels of the other stream run, instead of queueing behind their blocks.
    side_stream = torch.cuda.Stream(priority=-1)
    rows_1024 = max(1, 1024 // self.specs[0].output_shape[-1])

    def prepare_batch():
      with torch.cuda.stream(side_stream):
        dev_feats = []
        if dense_all is not None:
          dev_feats = [v.view(shape) for v, shape in zip(dense_all.cuda(non_blocking=True).split(sizes), shapes)]
        for p in ([] if dense_all is not None else pinned):
          if isinstance(p, torch.Tensor):
            dev_feats.append(p.cuda(non_blocking=True))
          else:
            dev_feats.append(embedding.RaggedInput(p.values.cuda(non_blocking=True), p.row_splits,
                                                   None if p.weights is None else p.weights.cuda(non_blocking=True)))
        dev_w = None if pinned_w is None else [w.cuda(non_blocking=True) for w in pinned_w]
        # sync_stats=False: the statistics stay on their way to the host until somebody reads them (an FDO client
        # would, every few hundred steps); the call does not wait for the GPU.
        p2, _ = embedding.preprocess_sparse_dense_matmul_input(dev_feats, dev_w, specs, 1, world, num_sc_per_device=1,
                                                               sync_stats=False)
        done = torch.cuda.Event()
        done.record(side_stream)
      # The buffers were allocated on the side stream and are read on the main one.
      for d in p2.sparse_dense_matmul_input:
        for t in d.values():
          t.record_stream(main_stream)
          break
      return p2, done

    # The input pipeline runs in a second host thread, as a data loader would: it issues the copy and the
    # preprocessing of batch i + 1 while this thread issues lookup, read-back and update of batch i.
    import concurrent.futures

    pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)
    device = torch.cuda.current_device()

    def prepare_in_worker():
      torch.cuda.set_device(device)
      return prepare_batch()

    # The step's result is read back every step, but the host does not stall on it: the checksum of step i is
    # copied to pinned memory behind the step's kernels and read by the host during step i + 1 (what a training
    # loop does with its loss), so the GPU always has the next kernels queued.
    results = [torch.zeros(1, pin_memory=True) for _ in range(2)]
    landed = [None, None]
    checksums = []

    def collect(k):
      if landed[k] is not None:
        landed[k].synchronize()
        checksums.append(float(results[k][0]))
        landed[k] = None

    def lookup_update_step(batch, index):
      p2, done = batch
      nxt = pool.submit(prepare_in_worker)
      main_stream.wait_event(done)
      acts = embedding.tpu_sparse_dense_matmul(p2, self.variables, specs, global_device_count=world, num_sc_per_device=1)
      # A checksum over the first 1024 values of every feature's activations; the activations themselves stay on
      # the device for the dense part of a model.
      base = getattr(acts[0], "_base", None)
      if base is not None and base.dim() == 2 and base.shape[0] == len(acts) * acts[0].shape[0]:
        # (the activations of all features are pieces of one buffer: one strided view instead of a slice per feature)
        checksum = base.view(len(acts), acts[0].shape[0], -1)[:, :rows_1024].sum()
      else:
        checksum = torch.cat([a[:rows_1024] for a in acts]).sum()
      k = index % 2
      collect(k)  # the read-back of two steps ago has long landed
      results[k].copy_(checksum.reshape(1), non_blocking=True)
      landed[k] = torch.cuda.Event()
      landed[k].record()
      embedding.tpu_sparse_dense_matmul_grad(self.grads, p2, self.variables, specs, global_device_count=world,
                                             num_sc_per_device=1, step=0)
      collect(1 - k)  # the previous step's result, while this step's kernels run
      return nxt.result()

    # Warm-up: the caching allocator hands the buffers of a step out at a few alternating addresses, and the first
    # call on every such set of addresses builds and validates its launch descriptors (milliseconds of Python).
    warm = 20
    batch = prepare_batch()
    for i in range(warm):
      batch = lookup_update_step(batch, i)
    collect(0), collect(1)
    blocks = []
    cache_before = dict(embedding.CALL_CACHE_STATS)
    for _ in range(3):  # three timed blocks of `steps` steps; the median block is reported
      self.barrier()
      t0 = time.perf_counter()
      for i in range(steps):
        batch = lookup_update_step(batch, i)
      collect(0), collect(1)  # every step's result has reached the host before the clock stops
      self.barrier()
      blocks.append(self.max_over_ranks((time.perf_counter() - t0) / steps * 1e3))
    pool.shutdown()
    assert len(checksums) == 3 * steps + warm and all(np.isfinite(checksums))
    ms = sorted(blocks)[1]
    return {"value": self.wl["batch"] * world / (ms * 1e-3), "unit": "samples/s", "ms_per_step": ms,
            "blocks_ms": blocks,
            "descriptor_cache": {k: embedding.CALL_CACHE_STATS[k] - cache_before[k] for k in cache_before},
            "timing": f"{warm} warm-up steps, then 3 blocks of {steps} steps; median block",
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 + 4 * sum(2 * 1 + 1 + 3 for _ in self.stacked),
            "host": "two Python threads: one issues copy + preprocessing of the next batch, one lookup, read-back and update",
            "read_back": "a 4-byte checksum of 1024 activations per feature, every step, copied to pinned memory behind the "
                         "step's kernels and read by the host during the next step; the activations stay on the device and "
                         "the preprocessing statistics are copied to pinned memory without a wait (sync_stats=False)",
            "pipeline": "copy + preprocessing of batch i+1 on a second stream while batch i is looked up and updated"}

  def release(self):
    """Frees the tables and buffers of this workload (the next one may need all of the GPU's memory)."""
    import torch
    from jax_tpu_embedding.sparsecore import _native, distributed
    from jax_tpu_embedding.sparsecore.lib.nn import embedding

    self.variables = self.pre = self.grads = None
    embedding.clear_caches()
    _native.clear_workspaces()
    gc.collect()
    if self.world > 1:
      distributed.release_all()
    torch.cuda.empty_cache()


def config_block(name, world, rank, args, peak):
  """A short run of one of the other configurations: step time, operator rooflines, preprocessing, parity."""
  wl = workload(name, args.scale)
  strong = name == "c4"
  if strong:  # the sharded 1e8-row configuration: 131072 samples per step whatever the number of GPUs
    wl = dict(wl, batch=131072 // world)
  global_batch = wl["batch"] * world
  run = Run(name, wl, world, rank, global_batch)
  for _ in range(10):
    run.step()
  ms, launches = run.timed_steps(10)
  roof = run.operator_rooflines(10, peak)
  out = {"workload": describe(name, wl, wl["batch"]), "global_batch": global_batch,
         "scaling": "strong" if strong else "weak", "steps": 10, "warmup": 10, "ms_per_step": ms,
         "value": global_batch / (ms * 1e-3), "unit": "samples/s", "gpu_launches": launches,
         "forward": roof["forward"], "backward": roof["backward"], "nnz": roof["nnz"], "unique_rows": roof["unique_rows"],
         "table_bytes": int(run.table_bytes), "preprocess": run.preprocess_block(5, peak)}
  ratio = TRAFFIC_RATIO.get(name)
  out["backward"]["traffic"] = None if ratio is None else int(roof["backward"]["algorithmic_bytes"] * ratio)
  hbm_ms = (roof["forward"]["algorithmic_bytes"] + roof["backward"]["algorithmic_bytes"]) / (peak * 1e9) * 1e3
  out["hbm_bound_ms"] = hbm_ms
  if world > 1:
    out["nvlink_bound_ms"] = 2 * roof["remote_row_bytes"] / (NVLINK_GBS * 1e9) * 1e3
    out["bound_ms"] = max(hbm_ms, out["nvlink_bound_ms"])
    out["phases_ms"] = run.phases(5)
  out["parity"] = run.parity()
  run.release()
  return out


# --------------------------------------------------------------------------------- main


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=100)
  ap.add_argument("--warmup", type=int, default=10)
  ap.add_argument("--workload", default="c2")
  ap.add_argument("--scale", type=float, default=1.0, help="scales vocabulary sizes (profiling only)")
  ap.add_argument("--impl", default="b200")
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--no-configs", action="store_true", help="skip the short runs of the other configurations")
  ap.add_argument("--parity", action="store_true", help="full-size parity check of the headline workload too")
  ap.add_argument("--profile-range", action="store_true",
                  help="bracket the timed steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
  args = ap.parse_args()
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  wl = workload(args.workload, args.scale)
  config = {"workload": describe(args.workload, wl, wl["batch"]),
            "l2_policy": "tables and activations far exceed L2 (126 MB); no flush needed", "scale": args.scale}

  if args.impl == "reference":
    if rank != 0:
      return
    specs = build_specs(wl)
    feats, weights = build_inputs(wl, specs)
    r = cpu_arm(wl, specs, feats, weights, steps=max(1, args.steps), warmup=max(0, args.warmup))
    line = {"impl": "reference", "metric": "samples/s fwd+Adagrad bwd", "value": r["samples_per_s"], "unit": "samples/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "cpu_baseline": {"value": r["samples_per_s"], "unit": "samples/s", "cores": r["cores"], "kind": "port",
                             "sample": "full batch per step, tables compacted to touched rows; includes C "
                                       f"preprocessing ({r['preprocess_ms']:.1f} ms/step)"},
            "e2e": {"value": r["samples_per_s"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return

  import torch
  from jax_tpu_embedding.sparsecore import _native

  if not torch.cuda.is_available() or not _native.available():
    raise SystemExit("bench.py needs a CUDA device and the built libsc_b200.so (no CPU fallback)")
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local_rank)
  if world > 1:
    from jax_tpu_embedding.sparsecore import distributed

    torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    distributed.init()
    config["sharding"] = (f"every stacked table row-sharded mod {world} over {world} GPUs (one process per GPU); forward "
                          "fetches each distinct remote row once over NVLink; backward reduces per (source, row) first, "
                          "then the owner of a shard pulls one gradient row per source and row")
  peak, peak_kind = measured_peak_gbs()

  # Weak scaling: every GPU brings its own batch of wl['batch'] samples; tables are shared.
  run = Run(args.workload, wl, world, rank, wl["batch"] * world)

  # The clock sampler runs from the warm-up to the end of the timed region (the GPU is under the same
  # load throughout); the warm-up lasts at least `--warmup` steps and long enough for several samples.
  sampler = ClockSampler(local_rank)
  sampler.start()
  warm_steps = max(args.warmup, 3)
  for _ in range(warm_steps):
    run.step()
  torch.cuda.synchronize()
  t_warm = time.time()
  flag = torch.zeros(1, device="cuda")
  while True:
    for _ in range(20):
      run.step()
    torch.cuda.synchronize()
    flag.fill_(1.0 if time.time() - t_warm < 0.4 else 0.0)
    if world > 1:  # all ranks leave the loop together
      torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX)
    if float(flag.item()) == 0.0:
      break
  if args.profile_range:
    torch.cuda.profiler.start()
  ms, gpu_launches = run.timed_steps(args.steps)
  if args.profile_range:
    torch.cuda.profiler.stop()
  clocks = sampler.stop()
  samples_per_s = wl["batch"] * world / (ms * 1e-3)

  # ---- roofline of the fused backward (dominant kernel): CUDA events around its launches only.
  reps = max(3, min(args.steps, 20))
  roof = run.operator_rooflines(reps, peak)
  bwd, fwd = roof["backward"], roof["forward"]
  ratio = TRAFFIC_RATIO.get(args.workload)
  traffic = None if ratio is None else int(bwd["algorithmic_bytes"] * ratio)
  preprocess = run.preprocess_block(max(3, min(args.steps, 10)), peak)
  phases = run.phases(max(3, min(args.steps, 10)))
  parity = run.parity() if args.parity else None
  e2e = None if args.no_e2e else run.e2e(max(3, min(args.steps, 50)))

  cpu = None
  if rank == 0 and world == 1 and not args.no_cpu_baseline:
    r = cpu_arm(wl, run.specs, run.feats, run.weights, steps=3, warmup=1)
    cpu = {"value": r["samples_per_s"], "unit": "samples/s", "cores": r["cores"], "kind": "port",
           "sample": f"1 step of the full batch, tables compacted to touched rows ({r['ms_per_step']:.0f} ms, of which "
                     f"C preprocessing {r['preprocess_ms']:.0f} ms)"}
  nnz_in, table_bytes = run.nnz_in, run.table_bytes
  remote_row_bytes = roof["remote_row_bytes"]

  configs = None
  if args.workload == "c2" and args.scale == 1.0 and not args.no_configs:
    run.release()
    configs = {}
    for name in ("c3", "c4", "c5"):
      try:
        configs[name] = config_block(name, world, rank, args, peak)
      except Exception as e:  # pylint: disable=broad-except
        configs[name] = {"error": f"{type(e).__name__}: {e}"[:400]}
        break  # a failed collective set-up leaves the ranks out of step: stop here

  if rank == 0:
    line = {
        "metric": "samples/s fwd+Adagrad bwd", "value": samples_per_s, "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "lookups_per_s": nnz_in * world / (ms * 1e-3),
        "roofline": {"bound": "hbm",
                     "kernel": ("bwd_lane_groups_kernel" if max(t["dim"] for t in wl["tables"]) <= 64 else "bwd_pipe_kernel") +
                               " + bwd_group_kernel + bwd_fixup_kernel (fused backward, all tables)",
                     "achieved": bwd["achieved"], "peak": peak, "unit": "GB/s", "frac": bwd["frac"], "peak_kind": peak_kind,
                     "traffic": traffic, "algorithmic_bytes": bwd["algorithmic_bytes"], "ms": bwd["ms"], "forward": fwd},
        "preprocess": preprocess, "phases_ms": phases, "parity": parity,
        "nvlink": None if world == 1 else {
            "forward_bytes_per_gpu": int(remote_row_bytes),
            "backward_bytes_per_gpu": int(remote_row_bytes),
            "bound_ms": 2 * remote_row_bytes / (NVLINK_GBS * 1e9) * 1e3,
            "undeduplicated_bytes_per_gpu": int(nnz_in * (world - 1) / world * 4 * wl["tables"][0]["dim"]),
            "note": "rank 0: one table row (forward) and one reduced gradient row (backward) per DISTINCT remote row "
                    "of the batch, at the measured 770 GB/s per direction; the step cannot be faster than "
                    "max(HBM time, this)"},
        "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
        "gpu_launches": gpu_launches,
        "table_bytes": int(table_bytes),
        "configs": configs,
    }
    print(json.dumps(line))
  if world > 1:
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
  main()
