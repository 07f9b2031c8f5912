"""NPZ and CSV FDO clients: the expectations of the reference's own tests
(jax_tpu_embedding/sparsecore/lib/fdo/file_fdo_client_test.py, csv_file_fdo_client_test.py)."""

import csv

import numpy as np
import pytest

from jax_tpu_embedding.sparsecore.lib.fdo import csv_file_fdo_client
from jax_tpu_embedding.sparsecore.lib.fdo import file_fdo_client
from jax_tpu_embedding.sparsecore.lib.nn import embedding

CLIENTS = {"npz": file_fdo_client.NPZFileFDOClient, "csv": csv_file_fdo_client.CSVFileFDOClient}


def _equal(actual, expected):
  assert len(actual) == len(expected)
  for key in expected:
    assert key in actual
    np.testing.assert_array_equal(expected[key], actual[key])


def _stats(ids=(10, 20, 30, 40), uniq=(1, 2, 3, 4), size=None):
  return embedding.SparseDenseMatmulInputStats(
      max_ids_per_partition={"tab_one": np.array(ids)}, max_unique_ids_per_partition={"tab_one": np.array(uniq)},
      required_buffer_size_per_sc={} if size is None else {"tab_one": np.array([size])})


@pytest.mark.parametrize("kind", CLIENTS)
def test_record_publish_load(kind, tmp_path):
  client = CLIENTS[kind](tmp_path)
  stats = _stats()
  client.record(stats)
  client.publish()
  loaded = client.load()
  _equal(loaded.max_ids_per_partition, stats.max_ids_per_partition)
  _equal(loaded.max_unique_ids_per_partition, stats.max_unique_ids_per_partition)
  _equal(loaded.required_buffer_size_per_sc, {})


@pytest.mark.parametrize("kind", CLIENTS)
def test_recording_twice_stacks_rows(kind, tmp_path):
  client = CLIENTS[kind](tmp_path)
  client.record(_stats(size=256))
  client.record(_stats(size=256))
  client.publish()
  loaded = client.load()
  _equal(loaded.max_ids_per_partition, {"tab_one": np.array([[10, 20, 30, 40]] * 2)})
  _equal(loaded.max_unique_ids_per_partition, {"tab_one": np.array([[1, 2, 3, 4]] * 2)})
  _equal(loaded.required_buffer_size_per_sc, {"tab_one": np.array([[256], [256]])})


def test_csv_without_history_keeps_the_maximum(tmp_path):
  client = csv_file_fdo_client.CSVFileFDOClient(tmp_path, retain_history=False)
  client.record(_stats(size=256))
  client.record(_stats(ids=(5, 25, 15, 45), uniq=(0, 3, 2, 5), size=512))
  client.publish()
  loaded = client.load()
  _equal(loaded.max_ids_per_partition, {"tab_one": np.array([10, 25, 30, 45])})
  _equal(loaded.max_unique_ids_per_partition, {"tab_one": np.array([1, 3, 3, 5])})
  _equal(loaded.required_buffer_size_per_sc, {"tab_one": np.array([512])})


def _two_process_files(kind, base):
  files = {
      "fdo_stats_0_10": {"t_one_max_ids": [10, 20, 30, 40], "t_two_max_ids": [50, 60, 70, 80],
                         "t_one_max_unique_ids": [1, 2, 3, 4], "t_two_max_unique_ids": [5, 6, 7, 8],
                         "t_one_required_buffer_size": [64], "t_two_required_buffer_size": [128]},
      "fdo_stats_1_11": {"t_one_max_ids": [20, 10, 40, 30], "t_two_max_ids": [60, 60, 80, 70],
                         "t_one_max_unique_ids": [2, 1, 4, 3], "t_two_max_unique_ids": [6, 5, 8, 7],
                         "t_one_required_buffer_size": [128], "t_two_required_buffer_size": [256]},
  }
  for name, arrays in files.items():
    if kind == "npz":
      np.savez(base / f"{name}.npz", **{k: np.array(v) for k, v in arrays.items()})
    else:
      with open(base / f"{name}.csv", "w", newline="") as f:
        writer = csv.writer(f)
        writer.writerow(["key", "values"])
        for k, v in arrays.items():
          writer.writerow([k, " ".join(map(str, v))])


@pytest.mark.parametrize("kind", CLIENTS)
def test_load_merges_processes_with_maximum(kind, tmp_path):
  _two_process_files(kind, tmp_path)
  loaded = CLIENTS[kind](tmp_path).load()
  _equal(loaded.max_ids_per_partition, {"t_one": np.array([20, 20, 40, 40]), "t_two": np.array([60, 60, 80, 80])})
  _equal(loaded.max_unique_ids_per_partition, {"t_one": np.array([2, 2, 4, 4]), "t_two": np.array([6, 6, 8, 8])})
  _equal(loaded.required_buffer_size_per_sc, {"t_one": np.array([128]), "t_two": np.array([256])})


@pytest.mark.parametrize("kind", CLIENTS)
def test_files_not_found(kind, tmp_path):
  with pytest.raises(FileNotFoundError):
    CLIENTS[kind](tmp_path).load()


def test_unexpected_key_is_rejected(tmp_path):
  np.savez(tmp_path / "fdo_stats_0_1.npz", t_one_bogus=np.array([1]))
  with pytest.raises(ValueError, match="Unexpected key"):
    file_fdo_client.NPZFileFDOClient(tmp_path).load()


def test_latest_files_by_process(tmp_path):
  files = ["temp/fdo_dumps/fdo_stats_0_10.npz", "temp/fdo_dumps/fdo_stats_0_20.npz", "temp/fdo_dumps/fdo_stats_0_30.npz",
           "temp/fdo_dumps/fdo_stats_1_09.npz", "temp/fdo_dumps/fdo_stats_0_40.npz", "temp/fdo_dumps/fdo_stats_2_10.npz"]
  client = file_fdo_client.NPZFileFDOClient(tmp_path)
  assert client._get_latest_files_by_process(files) == [  # pylint: disable=protected-access
      "temp/fdo_dumps/fdo_stats_2_10.npz", "temp/fdo_dumps/fdo_stats_1_09.npz", "temp/fdo_dumps/fdo_stats_0_40.npz"]


def test_loaded_stats_update_the_specs(tmp_path):
  """The loop the clients exist for: observed statistics -> limits and buffer sizes of the specs."""
  import cases

  case = cases.make_case("fdo", seed=2, tables=[dict(vocab=1000, dim=16)], batch=256, num_sc_per_device=2)
  name = "table_0"
  client = file_fdo_client.NPZFileFDOClient(tmp_path)
  client.record(embedding.SparseDenseMatmulInputStats(
      max_ids_per_partition={name: np.array([300, 280])}, max_unique_ids_per_partition={name: np.array([250, 260])},
      required_buffer_size_per_sc={name: np.array([592, 600])}))
  client.publish()
  embedding.update_preprocessing_parameters(case.feature_specs, client.load(), 2)
  spec = case.feature_specs[0].table_spec.stacked_table_spec
  assert (spec.max_ids_per_partition, spec.max_unique_ids_per_partition) == (300, 260)
  assert spec.suggested_coo_buffer_size_per_device == 1200
