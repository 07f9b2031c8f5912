"""Benchmark of the SparseCore hot path on B200: forward + fused Adagrad backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5|c1] [--impl reference]

Prints ONE JSON line.  `value` is samples/s of lookup + update with the preprocessed batch
resident in HBM; `e2e` adds the host->device copy of the raw ids, GPU preprocessing and a
device->host read of a checksum of the activations, all through the public Python API.
`roofline` is the fused backward kernel (algorithmic bytes / CUDA-event time / measured HBM
peak); `cpu_baseline` is the CPU oracle (C preprocessing + torch-CPU lookup/update) on the same
batch with compacted tables.  `--impl reference` runs only that CPU arm.

Workloads are the seeded synthetic configurations of BASELINE.json; no dataset is involved.
"""

from __future__ import annotations

import argparse
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


def table_stats(pre, specs, name, world=1, rank=0):
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


# --------------------------------------------------------------------------------- CPU arm


def cpu_arm(wl, specs, feats, weights, steps=1, warmup=0, threads=None):
  """CPU baseline: C oracle preprocessing (threaded) + torch-CPU lookup and Adagrad/Adam/SGD update.

  Tables are compacted to the rows the batch touches so that the sample needs no 100 GB host
  allocation; the number of lookups, unique rows and bytes moved per row are unchanged.
  """
  import torch
  sys.path.insert(0, os.path.join(ROOT, "tests"))
  import oracle_backend as ob
  from jax_tpu_embedding.sparsecore.lib.core import pybind_input_preprocessing as pip

  cores = len(os.sched_getaffinity(0))
  threads = threads or cores
  torch.set_num_threads(threads)
  np_feats, np_weights = [], ([] if wl["weights"] else None)
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
  stacks = {}
  times = []
  # Set-up, not part of the timed step: size the buffers from observed statistics (the reference's
  # FDO recipe) and compact row ids to an index among the touched rows.
  from jax_tpu_embedding.sparsecore.lib.nn import embedding

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
  ap.add_argument("--profile-range", action="store_true",
                  help="bracket the timed steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
  args = ap.parse_args()
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  wl = workload(args.workload, args.scale)
  config = {"workload": f"{args.workload}: {len(wl['tables'])} tables dim {wl['tables'][0]['dim']}, batch "
                        f"{wl['batch']}, combiner {wl['combiner']}, optimizer {wl['optimizer']}",
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
  from jax_tpu_embedding.sparsecore.lib.nn import embedding

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

  # Weak scaling: every GPU brings its own batch of wl['batch'] samples; tables are shared.
  specs = build_specs(wl, global_device_count=world, global_batch=wl["batch"] * world)
  feats, weights = build_inputs(wl, specs, rank)
  stacked = embedding.get_stacked_table_specs(specs)
  table_specs = list({f.table_spec.name: f.table_spec for f in specs}.values())
  layout = embedding.DeviceLayout(world, 1 if world > 1 else None, rank)
  variables = embedding.init_embedding_variables(1234 + rank, table_specs, layout, num_sparsecore_per_device=1)
  table_bytes = sum(v.table.numel() * 4 * (1 + len(v.slot)) for v in variables.values())

  # FDO pass (the reference's own recipe): observe limits once, then size the buffers exactly.
  pre, stats = embedding.preprocess_sparse_dense_matmul_input(feats, weights, specs, 1, world, num_sc_per_device=1,
                                                              allow_id_dropping=True)
  if world > 1:  # all ranks must agree on limits and buffer sizes
    for d in (stats.max_ids_per_partition, stats.max_unique_ids_per_partition, stats.required_buffer_size_per_sc):
      for k in sorted(d):
        t = torch.from_numpy(np.ascontiguousarray(d[k])).cuda()
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        d[k] = t.cpu().numpy()
  embedding.update_preprocessing_parameters(specs, stats, 1)
  pre, stats = embedding.preprocess_sparse_dense_matmul_input(feats, weights, specs, 1, world, num_sc_per_device=1)
  stacked = embedding.get_stacked_table_specs(specs)
  gen = torch.Generator(device="cuda").manual_seed(5 + rank)
  grads = [torch.randn((wl["batch"], f.output_shape[-1]), generator=gen, device="cuda") * 1e-2 for f in specs]
  def lookup_update():
    acts = embedding.tpu_sparse_dense_matmul(pre, variables, specs, global_device_count=world, num_sc_per_device=1)
    embedding.tpu_sparse_dense_matmul_grad(grads, pre, variables, specs, global_device_count=world,
                                           num_sc_per_device=1, step=0)
    return acts

  def barrier():
    if world > 1:
      torch.distributed.barrier()
    torch.cuda.synchronize()

  # The clock sampler runs from the warm-up to the end of the timed region (the GPU is under the same
  # load throughout); the warm-up lasts at least `--warmup` steps and long enough for several samples.
  sampler = ClockSampler(local_rank)
  sampler.start()
  warm_steps = max(args.warmup, 3)
  for _ in range(warm_steps):
    lookup_update()
  torch.cuda.synchronize()
  t_warm = time.time()
  flag = torch.zeros(1, device="cuda")
  while True:
    for _ in range(20):
      lookup_update()
    torch.cuda.synchronize()
    flag.fill_(1.0 if time.time() - t_warm < 0.4 else 0.0)
    if world > 1:  # all ranks leave the loop together
      torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX)
    if float(flag.item()) == 0.0:
      break
  barrier()
  ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  if args.profile_range:
    torch.cuda.profiler.start()
  launches0 = _native.lib().sc_launch_count()
  ev0.record()
  for _ in range(args.steps):
    lookup_update()
  ev1.record()
  gpu_launches = int(_native.lib().sc_launch_count() - launches0)
  barrier()
  if args.profile_range:
    torch.cuda.profiler.stop()
  clocks = sampler.stop()
  ms = ev0.elapsed_time(ev1) / args.steps
  if world > 1:
    t = torch.tensor([ms], device="cuda")
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t.item())
  samples_per_s = wl["batch"] * world / (ms * 1e-3)
  nnz_in = sum(int(np.prod(f.shape)) if isinstance(f, np.ndarray) else len(f.values) for f in feats)

  # ---- roofline of the fused backward (dominant kernel): CUDA events around its launches only.
  algo_bytes, bwd_ms, remote_row_bytes = 0, 0.0, 0
  per = {}
  for name, spec in stacked.items():
    n, u, remote = table_stats(pre, specs, name, world, rank)
    d, bdev = spec.stack_embedding_dim, spec.total_sample_count // world
    slots = spec.optimizer.slot_variables_count()
    per[name] = (n, u)
    remote_row_bytes += remote * 4 * d
    algo_bytes += bdev * 4 * d + n * 12 + 8 * 4 + u * 4 * d * (1 + slots) * 2
  stacked_grads = embedding.stack_embedding_gradients(grads, specs, 1, world)
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  reps = max(3, min(args.steps, 20))
  for _ in range(3):  # warm-up of this call signature (descriptor cache, workspaces)
    embedding.tpu_sparse_dense_matmul_grad(stacked_grads, pre, variables, specs, global_device_count=world,
                                           num_sc_per_device=1, step=0, perform_stacking=False)
  barrier()
  e0.record()
  for _ in range(reps):
    embedding.tpu_sparse_dense_matmul_grad(stacked_grads, pre, variables, specs, global_device_count=world,
                                           num_sc_per_device=1, step=0, perform_stacking=False)
  e1.record()
  torch.cuda.synchronize()
  bwd_ms = e0.elapsed_time(e1) / reps
  peak, peak_kind = measured_peak_gbs()
  # DRAM traffic of the backward kernels per launch: ncu measured 1.03 x the algorithmic bytes on a
  # scaled-down c2 case (profiles/c2_small_bwd_pipe_fwd_gather_full.md); traffic grows with the same
  # quantities as the algorithmic figure, so it is scaled to this launch.
  traffic_ratio = 1.03
  achieved = algo_bytes / (bwd_ms * 1e-3) / 1e9
  fwd_bytes = sum(per[n][1] * 4 * s.stack_embedding_dim + per[n][0] * 12 + 32
                  + s.total_sample_count // world * 4 * s.stack_embedding_dim for n, s in stacked.items())
  for _ in range(3):
    embedding.tpu_sparse_dense_matmul(pre, variables, specs, global_device_count=world, num_sc_per_device=1,
                                      perform_unstacking=False)
  barrier()
  e0.record()
  for _ in range(reps):
    embedding.tpu_sparse_dense_matmul(pre, variables, specs, global_device_count=world, num_sc_per_device=1,
                                      perform_unstacking=False)
  e1.record()
  torch.cuda.synchronize()
  fwd_ms = e0.elapsed_time(e1) / reps

  # ---- end to end through the public API with host buffers.
  e2e = None
  if not args.no_e2e:
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
    if weights is not None:
      pinned_w = [torch.from_numpy(w).pin_memory() for w in weights]
      h2d += sum(w.numel() * 4 for w in pinned_w)
    else:
      pinned_w = None

    # Dense id matrices travel as ONE pinned buffer and one copy per step; the features are views of it.
    dense_all = None
    if all(isinstance(p, torch.Tensor) for p in pinned) and pinned_w is None:
      shapes = [tuple(p.shape) for p in pinned]
      sizes = [p.numel() for p in pinned]
      dense_all = torch.cat([p.reshape(-1) for p in pinned]).pin_memory()

    # Software pipeline, as a training loop would run it: the host->device copy and the preprocessing of batch
    # i + 1 are issued on a second stream while the GPU runs lookup + update of batch i.  Every step still does
    # one copy, one preprocessing, one lookup, one result read-back and one update.
    main_stream = torch.cuda.current_stream()
    side_stream = torch.cuda.Stream()

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
        p2, _ = embedding.preprocess_sparse_dense_matmul_input(dev_feats, dev_w, specs, 1, world, num_sc_per_device=1)
        done = torch.cuda.Event()
        done.record(side_stream)
      # The buffers were allocated on the side stream and are read on the main one.
      for d in p2.sparse_dense_matmul_input:
        for t in d.values():
          t.record_stream(main_stream)
          break
      return p2, done

    def lookup_update_step(batch):
      p2, done = batch
      main_stream.wait_event(done)
      acts = embedding.tpu_sparse_dense_matmul(p2, variables, specs, global_device_count=world, num_sc_per_device=1)
      # The step's result read back by the host: a checksum over the first 1024 values of every feature's
      # activations (the dense part of a model, which would consume them all, is not part of this path).
      checksum = torch.cat([a.reshape(-1)[:1024] for a in acts]).sum()
      embedding.tpu_sparse_dense_matmul_grad(grads, p2, variables, specs, global_device_count=world,
                                             num_sc_per_device=1, step=0)
      nxt = prepare_batch()  # overlaps the kernels just launched
      return float(checksum.item()), nxt

    batch = prepare_batch()
    for _ in range(2):
      _, batch = lookup_update_step(batch)
    barrier()
    t0 = time.perf_counter()
    n_e2e = max(3, min(args.steps, 50))
    for _ in range(n_e2e):
      _, batch = lookup_update_step(batch)
    barrier()
    e2e_ms = (time.perf_counter() - t0) / n_e2e * 1e3
    if world > 1:
      t = torch.tensor([e2e_ms], device="cuda")
      torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
      e2e_ms = float(t.item())
    e2e = {"value": wl["batch"] * world / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 + 4 * sum(2 * 1 + 1 + 3 for _ in stacked),
           "pipeline": "copy + preprocessing of batch i+1 on a second stream while batch i is looked up and updated"}

  cpu = None
  if rank == 0 and world == 1 and not args.no_cpu_baseline:
    r = cpu_arm(wl, specs, feats, weights, steps=3, warmup=1)
    cpu = {"value": r["samples_per_s"], "unit": "samples/s", "cores": r["cores"], "kind": "port",
           "sample": f"1 step of the full batch, tables compacted to touched rows ({r['ms_per_step']:.0f} ms, of which "
                     f"C preprocessing {r['preprocess_ms']:.0f} ms)"}

  if rank == 0:
    line = {
        "metric": "samples/s fwd+Adagrad bwd", "value": samples_per_s, "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "lookups_per_s": nnz_in * world / (ms * 1e-3),
        "roofline": {"bound": "hbm", "kernel": "bwd_pipe_kernel + bwd_group_kernel + bwd_fixup_kernel (fused backward, all tables)", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": int(algo_bytes * traffic_ratio) if args.workload == "c2" else None,
                     "algorithmic_bytes": int(algo_bytes), "ms": bwd_ms,
                     "forward": {"algorithmic_bytes": int(fwd_bytes), "ms": fwd_ms,
                                 "achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                                 "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak}},
        "nvlink": None if world == 1 else {
            "forward_bytes_per_gpu": int(remote_row_bytes),
            "backward_bytes_per_gpu": int(remote_row_bytes),
            "bound_ms": 2 * remote_row_bytes / 770e9 * 1e3,
            "undeduplicated_bytes_per_gpu": int(nnz_in * (world - 1) / world * 4 * wl["tables"][0]["dim"]),
            "note": "rank 0: one table row (forward) and one reduced gradient row (backward) per DISTINCT remote row "
                    "of the batch, at the measured 770 GB/s per direction; the step cannot be faster than "
                    "max(HBM time, this)"},
        "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
        "gpu_launches": gpu_launches,
        "table_bytes": int(table_bytes),
    }
    print(json.dumps(line))
  if world > 1:
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
  main()
