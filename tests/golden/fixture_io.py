"""Reading and writing the committed golden fixtures (test infrastructure).

A fixture file is one `.npz` of plain arrays plus a JSON manifest stored inside it under the key
`manifest`; nothing is pickled.  Feature specs are stored as the handful of numbers the
preprocessing reads from them and rebuilt as real spec objects when a fixture is loaded.
"""

from __future__ import annotations

import dataclasses
import json
import os

import numpy as np

from jax_tpu_embedding.sparsecore.lib.nn import embedding_spec

HERE = os.path.dirname(os.path.abspath(__file__))


# ---------------------------------------------------------------------------- ragged inputs

def pack_rows(feature):
  """2-D array or array of rows -> (values, row lengths, valency or -1)."""
  if isinstance(feature, np.ndarray) and feature.dtype != object and feature.ndim == 2:
    return feature.reshape(-1), np.full(feature.shape[0], feature.shape[1], np.int64), feature.shape[1]
  rows = [np.asarray(r).reshape(-1) for r in feature]
  values = np.concatenate(rows) if rows else np.zeros(0)
  return values, np.asarray([len(r) for r in rows], np.int64), -1


def unpack_rows(values, lengths, valency, dtype):
  values = np.asarray(values, dtype)
  if valency >= 0:
    return values.reshape(len(lengths), valency)
  out = np.empty(len(lengths), dtype=object)
  pos = 0
  for i, n in enumerate(lengths):
    out[i] = values[pos:pos + n].copy()
    pos += n
  return out


# ---------------------------------------------------------------------------- specs

def _optimizer_to_json(opt):
  return {"class": type(opt).__name__, "learning_rate": float(opt.learning_rate)
          if isinstance(opt.learning_rate, (int, float)) else 0.01}


def _optimizer_from_json(d):
  return getattr(embedding_spec, d["class"])(learning_rate=d["learning_rate"])


def specs_to_json(feature_specs):
  tables, features = {}, []
  for f in feature_specs:
    t = f.table_spec
    if t.name not in tables:
      st, sis = t._stacked_table_spec, t.setting_in_stack  # pylint: disable=protected-access
      tables[t.name] = dict(
          name=t.name, vocabulary_size=t.vocabulary_size, embedding_dim=t.embedding_dim, combiner=t.combiner,
          optimizer=_optimizer_to_json(t.optimizer), max_ids_per_partition=t.max_ids_per_partition,
          max_unique_ids_per_partition=t.max_unique_ids_per_partition,
          suggested_coo_buffer_size_per_device=t.suggested_coo_buffer_size_per_device,
          stacked=None if st is None else dict(stack_name=st.stack_name, stack_vocab_size=st.stack_vocab_size,
                       stack_embedding_dim=st.stack_embedding_dim, combiner=st.combiner,
                       optimizer=_optimizer_to_json(st.optimizer), total_sample_count=st.total_sample_count,
                       max_ids_per_partition=st.max_ids_per_partition,
                       max_unique_ids_per_partition=st.max_unique_ids_per_partition,
                       suggested_coo_buffer_size_per_device=st.suggested_coo_buffer_size_per_device),
          setting=dict(stack_name=sis.stack_name, padded_vocab_size=sis.padded_vocab_size,
                       padded_embedding_dim=sis.padded_embedding_dim, row_offset_in_shard=sis.row_offset_in_shard,
                       shard_rotation=sis.shard_rotation))
    idt = f._id_transformation  # pylint: disable=protected-access
    features.append(dict(name=f.name, table=t.name, input_shape=list(f.input_shape), output_shape=list(f.output_shape),
                         id_transformation=None if idt is None else dataclasses.asdict(idt)))
  return dict(tables=list(tables.values()), features=features)


def specs_from_json(d):
  tables = {}
  for t in d["tables"]:
    spec = embedding_spec.TableSpec(
        name=t["name"], vocabulary_size=t["vocabulary_size"], embedding_dim=t["embedding_dim"], initializer=None,
        optimizer=_optimizer_from_json(t["optimizer"]), combiner=t["combiner"],
        max_ids_per_partition=t["max_ids_per_partition"],
        max_unique_ids_per_partition=t["max_unique_ids_per_partition"],
        suggested_coo_buffer_size_per_device=t["suggested_coo_buffer_size_per_device"])
    if t["stacked"] is not None:
      st = dict(t["stacked"])
      st["optimizer"] = _optimizer_from_json(st["optimizer"])
      spec.stacked_table_spec = embedding_spec.StackedTableSpec(**st)
    spec.setting_in_stack = embedding_spec.TableSettingInStack(**t["setting"])
    tables[t["name"]] = spec
  features = []
  for f in d["features"]:
    spec = embedding_spec.FeatureSpec(name=f["name"], table_spec=tables[f["table"]], input_shape=f["input_shape"],
                                      output_shape=f["output_shape"])
    if f["id_transformation"] is not None:
      spec.id_transformation = embedding_spec.FeatureIdTransformation(**f["id_transformation"])
    features.append(spec)
  return features


# ---------------------------------------------------------------------------- files

def save(path, manifest, arrays):
  np.savez_compressed(path, manifest=np.frombuffer(json.dumps(manifest).encode(), dtype=np.uint8), **arrays)


def load(name):
  data = np.load(os.path.join(HERE, name))
  manifest = json.loads(bytes(data["manifest"]).decode())
  return manifest, data
