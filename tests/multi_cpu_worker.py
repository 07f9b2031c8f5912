"""Worker of the world_size-2 CPU test (gloo): the data-parallel protocol with the oracle as compute.

Every rank owns shard `rank` of a stacked table and preprocesses only its slice of the global
batch (local_device_count=1, global_device_count=world).  The exchange that the GPU path performs
through peer memory is done here with gloo collectives:

* forward  - a rank needs rows of every shard: shards are all-gathered, the lookup runs on the
             rank's own CSR buffers;
* backward - every rank publishes its CSR buffers and activation gradients (all-gather); the owner
             of shard g reduces partition g of every source in (source, slot) order and applies the
             optimizer once.

The results must equal the oracle run for the whole job in one process (all devices local).
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

  rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
  dist.init_process_group("gloo")
  c = world

  def all_gather(a):
    out = [torch.empty_like(torch.from_numpy(a)) for _ in range(c)]
    dist.all_gather(out, torch.from_numpy(np.ascontiguousarray(a)))
    return [t.numpy() for t in out]

  for optimizer, combiner, weights in (("adagrad", "mean", None), ("sgd", "sum", True)):
    case = cases.make_case(
        "dist_cpu", seed=5150 + c, global_device_count=c, local_device_count=c, batch=64 * c, combiner=combiner,
        optimizer=optimizer, weights=weights, stack=True, max_ids=2048, max_unique=2048, dup_prob=0.1,
        tables=[dict(vocab=600, dim=16, features=[dict(kind="ragged", max_len=9, dist="zipf", a=1.05)]),
                dict(vocab=100, dim=16, features=[dict(kind="dense", valency=3)])])
    specs = case.feature_specs
    # Whole job in one process: the expectation.
    want = ob.oracle_preprocess(case.features, case.weights, specs, c, c, num_sc_per_device=1, has_leading_dimension=True)
    name = next(iter(want[0]))
    spec = specs[0].table_spec.stacked_table_spec
    rows, dim, bdev = spec.stack_vocab_size // c, spec.stack_embedding_dim, spec.total_sample_count // c

    # This rank's slice only.
    per = [f.shape[0] // c for f in case.features]
    local_feats = [f[rank * n:(rank + 1) * n] for f, n in zip(case.features, per)]
    local_w = None if case.weights is None else [w[rank * n:(rank + 1) * n] for w, n in zip(case.weights, per)]
    mine = ob.oracle_preprocess(local_feats, local_w, specs, 1, c, num_sc_per_device=1, has_leading_dimension=True)
    my_csr = tuple(mine[i][name][0] for i in range(4))
    for i in range(4):
      np.testing.assert_array_equal(my_csr[i], want[i][name][rank])
    # Statistics are reported per device: the ranks' values side by side are the single-process value,
    # and their maximum (what a job feeds back into its limits) is the same either way.
    stat = np.asarray(mine[5].max_ids_per_partition[name]).copy()
    np.testing.assert_array_equal(np.concatenate(all_gather(stat)), np.asarray(want[5].max_ids_per_partition[name]))
    top = torch.tensor([int(stat.max())])
    dist.all_reduce(top, op=dist.ReduceOp.MAX)
    assert int(top) == int(np.asarray(want[5].max_ids_per_partition[name]).max())

    rng = np.random.default_rng(77)
    shards = rng.normal(0, 0.01, size=(c, rows, dim)).astype(np.float32)
    acc = rng.uniform(0.05, 0.2, size=shards.shape).astype(np.float32)
    grads = [(rng.normal(size=(bdev, dim)) * 1e-2).astype(np.float32) for _ in range(c)]
    my_shard, my_acc = shards[rank].copy(), acc[rank].copy()

    # Forward: rows of all shards, this rank's samples.
    gathered = np.stack(all_gather(my_shard))
    act = lo.forward([my_csr], gathered, num_sc_per_device=1, device_batch_size=bdev)[0]
    csr_all = [tuple(want[i][name][d] for i in range(4)) for d in range(c)]
    np.testing.assert_array_equal(act, lo.forward(csr_all, shards, num_sc_per_device=1, device_batch_size=bdev)[rank])

    # Backward: publish buffers, pull partition `rank` of every source, apply once.
    pulled = [tuple(x) for x in zip(*[all_gather(a) for a in my_csr])]
    pulled_grads = all_gather(grads[rank])
    g, touched = lo.table_gradient(pulled, pulled_grads, shards.shape, num_sc_per_device=1)
    g_ref, touched_ref = lo.table_gradient(csr_all, grads, shards.shape, num_sc_per_device=1)
    np.testing.assert_array_equal(g[rank], g_ref[rank])
    one = lambda a: a[rank:rank + 1]
    if optimizer == "sgd":
      (new_shard,) = lo.apply_sgd(one(gathered), one(g), one(touched), 0.01)
      want_new = lo.apply_sgd(shards, g_ref, touched_ref, 0.01)
    else:
      new_shard, new_acc = lo.apply_adagrad(one(gathered), my_acc[None], one(g), one(touched), 0.01)
      want_new = lo.apply_adagrad(shards, acc, g_ref, touched_ref, 0.01)
      np.testing.assert_array_equal(new_acc[0], want_new[1][rank])
    np.testing.assert_array_equal(new_shard[0], want_new[0][rank])
    # Every rank ends with the same global table.
    final = np.stack(all_gather(np.ascontiguousarray(new_shard[0])))
    np.testing.assert_array_equal(final, want_new[0])
  dist.barrier()
  dist.destroy_process_group()
  print(f"rank {rank} ok")


if __name__ == "__main__":
  main()
