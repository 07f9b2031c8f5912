"""Worker of the multi-GPU parity test: one process per GPU (launched by torch.distributed.run).

Every rank preprocesses its slice of a global batch, looks up rows of all shards (remote ones over
NVLink) and updates the shard it owns; all results are compared with the CPU oracle computed for
the whole job.
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "jax-tpu-embedding_b200"), os.path.join(ROOT, "tests")):
  if p not in sys.path:
    sys.path.insert(0, p)


def main():
  import torch
  import torch.distributed as dist

  import cases
  import oracle_backend as ob
  from oracle import lookup_oracle as lo
  from jax_tpu_embedding.sparsecore import distributed
  from jax_tpu_embedding.sparsecore.lib.nn import embedding

  rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
  torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
  dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
  distributed.init()
  c = world

  # Row lengths 128, 64 and 32 floats: one, two and four rows per warp instruction in the update kernels.
  for optimizer, combiner, weights, dim in (("adagrad", "mean", None, 128), ("sgd", "sum", True, 64),
                                            ("adam", "sqrtn", None, 32)):
    case = cases.make_case(
        "dist", seed=4040 + c, global_device_count=c, local_device_count=c, batch=256 * c, combiner=combiner,
        optimizer=optimizer, weights=weights, stack=True, max_ids=4096, max_unique=4096, dup_prob=0.1,
        tables=[dict(vocab=3000, dim=dim, features=[dict(kind="ragged", max_len=12, dist="zipf", a=1.05)]),
                dict(vocab=500, dim=dim, features=[dict(kind="dense", valency=3)])])
    specs = case.feature_specs
    want = ob.oracle_preprocess(case.features, case.weights, specs, c, c, num_sc_per_device=1, has_leading_dimension=True)
    name = next(iter(want[0]))
    spec = specs[0].table_spec.stacked_table_spec
    rows, dim, bdev = spec.stack_vocab_size // c, spec.stack_embedding_dim, spec.total_sample_count // c

    per = [f.shape[0] // c for f in case.features]
    local_feats = [f[rank * n:(rank + 1) * n] for f, n in zip(case.features, per)]
    local_w = None if case.weights is None else [w[rank * n:(rank + 1) * n] for w, n in zip(case.weights, per)]
    pre, stats = embedding.preprocess_sparse_dense_matmul_input(local_feats, local_w, specs, 1, c, num_sc_per_device=1)
    ob.written_region_equal(pre.lhs_row_pointers[name].cpu().numpy(), want[0][name][rank],
                            [pre.lhs_embedding_ids[name].cpu().numpy(), pre.lhs_sample_ids[name].cpu().numpy(),
                             pre.lhs_gains[name].cpu().numpy()], [want[i][name][rank] for i in (1, 2, 3)], 1)

    rng = np.random.default_rng(99)
    shards = rng.normal(0, 0.01, size=(c, rows, dim)).astype(np.float32)
    slot0 = rng.uniform(0.05, 0.2, size=shards.shape).astype(np.float32)
    slot1 = rng.uniform(0.0, 1e-4, size=shards.shape).astype(np.float32)
    grads = [(rng.normal(size=(bdev, dim)) * 1e-2).astype(np.float32) for _ in range(c)]
    nslots = spec.optimizer.slot_variables_count()

    def peer_tensor(a):
      t = distributed.alloc(a.shape)
      t.copy_(torch.from_numpy(a))
      return t

    table = peer_tensor(shards[rank])
    slots = tuple(peer_tensor(x[rank]) for x in (slot0, slot1)[:nslots])
    slot_type = type(spec.optimizer.slot_variables_initializers())
    variables = {name: embedding.EmbeddingVariables(table, slot_type(*slots) if nslots else slot_type())}

    csr = [tuple(want[i][name][d] for i in range(4)) for d in range(c)]
    for step in range(2):  # the second step starts from the updated shards and reuses every buffer
      want_act = lo.forward(csr, shards, num_sc_per_device=1, device_batch_size=bdev)[rank]
      acts = embedding.tpu_sparse_dense_matmul(pre, variables, specs, global_device_count=c, num_sc_per_device=1,
                                               perform_unstacking=False)
      np.testing.assert_array_equal(acts[name].cpu().numpy(), want_act)

      g, touched = lo.table_gradient(csr, grads, shards.shape, num_sc_per_device=1)
      if optimizer == "sgd":
        new = lo.apply_sgd(shards, g, touched, 0.01)
      elif optimizer == "adagrad":
        new = lo.apply_adagrad(shards, slot0, g, touched, 0.01)
      else:
        new = lo.apply_adam(shards, slot0, slot1, g, touched, *lo.adam_hyperparameters(1e-3, 0.9, 0.999, 1e-8, step))
      updated = embedding.tpu_sparse_dense_matmul_grad(
          {name: torch.from_numpy(grads[rank]).cuda()}, pre, variables, specs, global_device_count=c,
          num_sc_per_device=1, perform_stacking=False, step=step)
      got = [updated[name].table, *updated[name].slot]
      for a, b in zip(got, new):
        b = b[rank]
        np.testing.assert_allclose(a.cpu().numpy(), b, rtol=1e-5, atol=1e-6 * float(np.abs(b).max()) + 1e-12)
      # Carry the oracle state forward exactly as the GPUs hold it.
      shards = new[0]
      if nslots >= 1:
        slot0 = new[1]
      if nslots >= 2:
        slot1 = new[2]
      gathered = [torch.empty_like(table) for _ in range(c)]
      dist.all_gather(gathered, table)
      shards = np.stack([t.cpu().numpy() for t in gathered])
      for si, (slot_np, slot_t) in enumerate(zip((slot0, slot1)[:nslots], slots)):
        gs = [torch.empty_like(slot_t) for _ in range(c)]
        dist.all_gather(gs, slot_t)
        if si == 0:
          slot0 = np.stack([t.cpu().numpy() for t in gs])
        else:
          slot1 = np.stack([t.cpu().numpy() for t in gs])
    if rank == 0:
      print(f"multi-gpu parity ok: world={c} optimizer={optimizer} combiner={combiner}", flush=True)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
