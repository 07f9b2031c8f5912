// GPU input preprocessing: ragged ids of one device -> CSR-wrapped COO buffers.
//
// Replaces the host C++ pipeline of the reference (extract -> 64-bit keys -> VQSort ->
// sequential group/dedup -> fill; jax_tpu_embedding/sparsecore/lib/core/
// input_preprocessing.cc, sort_and_group_coo_tensors_impl.h, input_preprocessing_util.cc)
// with data-parallel kernels whose output is bit-identical over the region the reference
// writes:
//
//   extract   one thread per sample row: column id with table-stack shift/offset, sample id
//             with split-then-stack row offsets, f32 gain with the reference's rounding order;
//   sort      the reference orders entries by (SparseCore, shard, row of the shard, sample).
//             Entries are already in ascending sample order per SparseCore, so a STABLE radix
//             sort on the compact key (SparseCore | shard | local row) alone is enough: 3-4
//             byte passes over 32-bit keys instead of 64-bit keys;
//   group     head flags of (row, sample) pairs and of rows -> one 64-bit exclusive scan gives
//             the rank of every pair and of every unique row inside its partition; the
//             sequential drop rules of the reference reduce to "keep a prefix of each partition";
//   pack      per-partition 8-aligned offsets, row pointers, padding, duplicate gains summed
//             left to right in float32.
#include <math.h>

#include "sc_common.cuh"
#include "sc_sort.cuh"

namespace sc {
namespace {

constexpr int kBlock = 256;
constexpr int kMaxPartitions = 4 * SC_MAX_SHARDS;  // local SparseCores x shards handled by one call

struct PreParams {
  int32_t S, P, C;           // SparseCores per device, shards, devices
  int32_t pbits, lbits;      // bits of the shard id and of the row inside a shard
  int32_t bslice;            // samples per SparseCore slice (ceil(batch / S))
  int32_t combiner, has_weights;
  int32_t max_ids, max_unique, allow_drop;
  int32_t coo_per_sc, R;
  int32_t num_features;
  int64_t nnz, total_rows;
};

// ---- extract ---------------------------------------------------------------------------
// Restates ProcessCooTensors (process_coo_tensors_impl.h:79-136), ComputeWeightDivisor
// (:39-77), CooFormat::GetColId (coo_format.h:120-135) and the slice arithmetic of
// ExtractCooTensorsForAllFeaturesPerLocalDevice (input_preprocessing.cc:79-123, 312-436).
__global__ void extract_kernel(PreParams p, const sc_feature_desc_t* __restrict__ feats, const int32_t* __restrict__ ids,
                               const int32_t* __restrict__ offsets, const float* __restrict__ weights,
                               uint32_t* __restrict__ keys, int32_t* __restrict__ row_of, float* __restrict__ gain_of,
                               float* __restrict__ row_gain, int32_t* __restrict__ error_flag) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= p.total_rows) return;
  int lo = 0, hi = p.num_features - 1;  // last feature with row_begin <= r
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (feats[mid].row_begin <= r) lo = mid; else hi = mid - 1;
  }
  const sc_feature_desc_t fd = feats[lo];
  const int rf = (int)(r - fd.row_begin);
  const int per_slice = fd.rows / p.S;
  const int s = min(rf / max(per_slice, 1), p.S - 1);
  int row_id = s * p.bslice + fd.row_offset / (p.C * p.S) + (rf - s * per_slice);
  if (row_id < 0 || row_id >= p.S * p.bslice) {  // row offsets inconsistent with the batch
    atomicOr(error_flag, 1);
    row_id = 0;
  }
  const int b = offsets[r], e = offsets[r + 1];
  const int cnt = e - b;
  float divisor = 1.0f;
  if (!p.has_weights) {
    float g = 1.0f;
    if (p.combiner == SC_COMBINER_MEAN) g = 1.0f / (float)cnt;
    else if (p.combiner == SC_COMBINER_SQRTN) g = 1.0f / sqrtf((float)cnt);
    row_gain[row_id] = g;
  } else if (p.combiner == SC_COMBINER_MEAN) {
    float sum = 0.0f;
    for (int i = b; i < e; ++i) sum += weights[i];
    divisor = sum;
  } else if (p.combiner == SC_COMBINER_SQRTN) {
    // The reference squares with std::pow(float, int): the square is a double that is added
    // to a float accumulator.
    float sum = 0.0f;
    for (int i = b; i < e; ++i) {
      const double w = (double)weights[i];
      sum = (float)((double)sum + w * w);
    }
    divisor = sqrtf(sum);
  }
  const int mod = p.P - 1;
  const uint32_t local_limit = 1u << p.lbits;
  for (int i = b; i < e; ++i) {
    const int id = ids[i];
    const int col = ((id + fd.col_shift) & mod) + (id & ~mod) + fd.col_offset;
    const uint32_t shard = (uint32_t)(col & mod);
    uint32_t local = (uint32_t)col >> p.pbits;
    if (id < 0 || local >= local_limit) {
      atomicOr(error_flag, 1);
      local = local_limit - 1;
    }
    keys[i] = ((uint32_t)s << (p.pbits + p.lbits)) | (shard << p.lbits) | local;
    row_of[i] = row_id;
    if (p.has_weights) gain_of[i] = weights[i] / divisor;
  }
}

// ---- group -----------------------------------------------------------------------------
// flags[p] = (pair head) | (row head) << 32, in sorted order; also keeps the sample of
// every sorted entry.  A pair head is the first entry of a (local SparseCore, column, sample)
// group, i.e. what GroupAndDeduplicateCooTensorsForLocalSparseCore
// (sort_and_group_coo_tensors_impl.h:235-310) treats as a new id.
__global__ void flags_kernel(int64_t n, const uint32_t* __restrict__ keys, const uint32_t* __restrict__ vals,
                             const int32_t* __restrict__ row_of, int32_t* __restrict__ row_sorted, uint64_t* __restrict__ flags) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  const uint32_t k = keys[p];
  const int32_t row = row_of[vals[p]];
  row_sorted[p] = row;
  bool new_col = true, new_pair = true;
  if (p > 0) {
    const uint32_t pk = keys[p - 1];
    new_col = pk != k;
    new_pair = new_col || row_of[vals[p - 1]] != row;
  }
  flags[p] = (uint64_t)(new_pair ? 1u : 0u) | ((uint64_t)(new_col ? 1u : 0u) << 32);
}

// bounds[q] = first sorted position whose partition id (key >> lbits) is >= q, q in [0, S*P].
__global__ void bounds_kernel(int64_t n, const uint32_t* __restrict__ keys, int lbits, int parts, int32_t* __restrict__ bounds) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q > parts) return;
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if ((int)(keys[mid] >> lbits) < q) lo = mid + 1; else hi = mid;
  }
  bounds[q] = (int32_t)lo;
}

__device__ __forceinline__ uint32_t lo32(uint64_t v) { return (uint32_t)v; }
__device__ __forceinline__ uint32_t hi32(uint64_t v) { return (uint32_t)(v >> 32); }
__device__ __forceinline__ int round8(int v) { return (v + kAlign - 1) & ~(kAlign - 1); }

// One block.  Thread q < S*P measures partition q; thread s < S then lays out SparseCore s.
// cnt is the exclusive scan of flags with the grand total at cnt[n].
__global__ void layout_kernel(PreParams p, const uint64_t* __restrict__ cnt, const int32_t* __restrict__ bounds,
                              int32_t* __restrict__ part_start, int32_t* __restrict__ part_written,
                              int32_t* __restrict__ row_pointers, int32_t* __restrict__ stats, const int32_t* __restrict__ error_flag) {
  __shared__ int32_t s_ids[kMaxPartitions], s_uniq[kMaxPartitions], s_kept[kMaxPartitions];
  __shared__ int32_t s_drop_limit[kMaxPartitions], s_drop_static[kMaxPartitions];
  const int parts = p.S * p.P;
  const int q = threadIdx.x;
  if (q < parts) {
    const int a = bounds[q], b = bounds[q + 1];
    const uint64_t ca = cnt[a], cb = cnt[b];
    const int ids = (int)(lo32(cb) - lo32(ca));
    const int uniq = (int)(hi32(cb) - hi32(ca));
    int kept = ids;
    int covered = b - a;  // raw entries represented by the kept pairs
    if (p.allow_drop) {
      // The pair with rank j and row rank u survives iff j < max_ids and u < max_unique;
      // both ranks grow along the partition, so the survivors are a prefix.
      int lo = a, hi = b;  // first position whose row rank reaches max_unique
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if ((int)(hi32(cnt[mid + 1]) - hi32(ca)) > p.max_unique) hi = mid; else lo = mid + 1;
      }
      const int by_unique = (int)(lo32(cnt[lo]) - lo32(ca));
      kept = min(ids, min(p.max_ids, by_unique));
      if (kept < ids) {
        lo = a; hi = b;  // position of pair number `kept`
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if ((int)(lo32(cnt[mid + 1]) - lo32(ca)) > kept) hi = mid; else lo = mid + 1;
        }
        covered = lo - a;
      }
    }
    s_ids[q] = ids; s_uniq[q] = uniq; s_kept[q] = kept;
    s_drop_limit[q] = (b - a) - covered;
  }
  __syncthreads();
  if (q < p.S) {
    // FillBufferSegment (input_preprocessing_util.cc:167-208): partitions are laid out in
    // order, each starting on a multiple of 8; writing stops at the end of the slice.
    const int s = q;
    int cursor = 0, required = 0;
    for (int g = 0; g < p.P; ++g) {
      const int idx = s * p.P + g;
      const int written = max(0, min(s_kept[idx], p.coo_per_sc - cursor));
      part_start[idx] = cursor;
      part_written[idx] = written;
      s_drop_static[idx] = s_kept[idx] - written;
      const int end = cursor + s_kept[idx];
      row_pointers[s * p.R + g] = min(end, p.coo_per_sc);
      cursor = round8(end);
      required += round8(s_ids[idx]);
    }
    for (int g = p.P; g < p.R; ++g) row_pointers[s * p.R + g] = min(cursor, p.coo_per_sc);
    stats[2 * p.P + s] = required;
  }
  __syncthreads();
  if (q < p.P) {
    int m_ids = 0, m_uniq = 0;
    for (int s = 0; s < p.S; ++s) {
      m_ids = max(m_ids, s_ids[s * p.P + q]);
      m_uniq = max(m_uniq, s_uniq[s * p.P + q]);
    }
    stats[q] = m_ids;
    stats[p.P + q] = m_uniq;
  }
  if (q == 0) {
    int dropped = 0, written = 0, over = 0;
    for (int i = 0; i < parts; ++i) {
      dropped += s_drop_limit[i] + s_drop_static[i];
      written += s_kept[i] - s_drop_static[i];
      if (s_ids[i] > p.max_ids || s_uniq[i] > p.max_unique) over = 1;
    }
    stats[2 * p.P + p.S] = dropped;
    int status = SC_OK;
    if (over && !p.allow_drop) status = SC_ID_LIMIT_EXCEEDED;
    if (*error_flag) status = SC_INVALID_ARGUMENT;
    stats[2 * p.P + p.S + 1] = status;
    stats[2 * p.P + p.S + 2] = written;
  }
}

__global__ void fill_kernel(int32_t coo, int32_t* __restrict__ ids, int32_t* __restrict__ sids, float* __restrict__ gains) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= coo) return;
  ids[q] = SC_PADDING_VALUE;
  sids[q] = SC_PADDING_VALUE;
  gains[q] = nanf("");
}

// One thread per sorted entry; pair heads that survive write their slot.  Duplicates are
// summed left to right, as PartitionedCooTensors::MergeWithLastCoo does
// (partitioned_coo_tensors.h:94-101).
__global__ void pack_kernel(PreParams p, const uint32_t* __restrict__ keys, const uint32_t* __restrict__ vals,
                            const int32_t* __restrict__ row_sorted, const float* __restrict__ gain_of,
                            const float* __restrict__ row_gain, const uint64_t* __restrict__ cnt,
                            const int32_t* __restrict__ bounds, const int32_t* __restrict__ part_start,
                            const int32_t* __restrict__ part_written, int32_t* __restrict__ out_ids, int32_t* __restrict__ out_sids,
                            float* __restrict__ out_gains) {
  const int64_t pos = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (pos >= p.nnz) return;
  const uint64_t c0 = cnt[pos], c1 = cnt[pos + 1];
  if (lo32(c1) == lo32(c0)) return;  // duplicate of an earlier entry
  const uint32_t key = keys[pos];
  const int part = (int)(key >> p.lbits);
  const int a = bounds[part], b = bounds[part + 1];
  const int j = (int)(lo32(c0) - lo32(cnt[a]));
  if (j >= part_written[part]) return;
  const int row = row_sorted[pos];
  float gain = p.has_weights ? gain_of[vals[pos]] : row_gain[row];
  for (int64_t t = pos + 1; t < b && lo32(cnt[t + 1]) == lo32(cnt[t]); ++t) {
    gain += p.has_weights ? gain_of[vals[t]] : row_gain[row];
  }
  const int s = part / p.P;
  const int64_t slot = (int64_t)s * p.coo_per_sc + part_start[part] + j;
  out_ids[slot] = (int32_t)(key & ((1u << p.lbits) - 1u));
  out_sids[slot] = row % p.bslice;
  out_gains[slot] = gain;
}

struct PreScratch {
  sc_feature_desc_t* feats;
  SortBuffers sort;
  int32_t* row_of;
  int32_t* row_sorted;
  float* gain_of;
  float* row_gain;
  uint64_t* cnt;
  uint64_t* scan_temp;
  int32_t* bounds;
  int32_t* part_start;
  int32_t* part_written;
  int32_t* error_flag;
};

bool carve(Workspace& ws, int64_t nnz, int64_t total_rows, int S, int P, PreScratch* s) {
  const size_t n = (size_t)(nnz > 0 ? nnz : 1);
  s->feats = ws.take<sc_feature_desc_t>(SC_MAX_FEATURES);
  s->sort.keys[0] = ws.take<uint32_t>(n); s->sort.keys[1] = ws.take<uint32_t>(n);
  s->sort.vals[0] = ws.take<uint32_t>(n); s->sort.vals[1] = ws.take<uint32_t>(n);
  s->sort.hist = ws.take<uint32_t>(sort_hist_elems(n));
  s->sort.scan_temp = ws.take<uint32_t>(scan_temp_elems(sort_hist_elems(n)));
  s->row_of = ws.take<int32_t>(n);
  s->row_sorted = ws.take<int32_t>(n);
  s->gain_of = ws.take<float>(n);
  s->row_gain = ws.take<float>((size_t)total_rows + (size_t)S + 8);
  s->cnt = ws.take<uint64_t>(n + 1);
  s->scan_temp = ws.take<uint64_t>(scan_temp_elems(n));
  s->bounds = ws.take<int32_t>((size_t)S * P + 2);
  s->part_start = ws.take<int32_t>((size_t)S * P);
  s->part_written = ws.take<int32_t>((size_t)S * P);
  s->error_flag = ws.take<int32_t>(1);
  return ws.ok();
}

int check_options(const sc_preprocess_options_t* o) {
  if (!o) SC_FAIL(SC_INVALID_ARGUMENT, "options are null");
  // PreprocessSparseDenseMatmulInputOptions::Validate (input_preprocessing_util.cc:490-522).
  if (o->global_device_count <= 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "global_device_count must be greater than 0, but got %d", o->global_device_count);
  if (o->num_sc_per_device <= 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "num_sc_per_device must be greater than 0, but got %d", o->num_sc_per_device);
  const int64_t P = (int64_t)o->global_device_count * o->num_sc_per_device;
  if (P & (P - 1)) SC_FAIL(SC_INVALID_ARGUMENT, "Total number of SparseCores (%lld) must be a power of 2.", (long long)P);
  if (P > SC_MAX_SHARDS || o->num_sc_per_device * P > kMaxPartitions)
    SC_FAIL(SC_UNSUPPORTED, "%lld shards exceed the supported maximum of %d", (long long)P, SC_MAX_SHARDS);
  if (o->combiner < 0 || o->combiner > 2) SC_FAIL(SC_INVALID_ARGUMENT, "unknown combiner %d", o->combiner);
  if (o->max_ids_per_partition <= 0 || o->max_unique_ids_per_partition <= 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "max_ids_per_partition and max_unique_ids_per_partition must be positive");
  if (o->coo_buffer_size_per_device <= 0 || o->coo_buffer_size_per_device % (kAlign * o->num_sc_per_device) != 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "coo_buffer_size_per_device (%d) must be a positive multiple of 8 * num_sc_per_device",
            o->coo_buffer_size_per_device);
  if (o->stack_vocab_size <= 0 || o->stack_vocab_size % P != 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "stack_vocab_size (%d) must be a positive multiple of the shard count", o->stack_vocab_size);
  return SC_OK;
}

}  // namespace
}  // namespace sc

using namespace sc;

extern "C" int32_t sc_preprocess_stats_size(int32_t global_device_count, int32_t num_sc_per_device) {
  return 2 * global_device_count * num_sc_per_device + num_sc_per_device + 3;
}

extern "C" size_t sc_preprocess_workspace_bytes(int64_t nnz, int64_t total_rows, const sc_preprocess_options_t* o) {
  if (check_options(o) != SC_OK) return 0;
  Workspace ws(nullptr, 0);
  PreScratch s;
  carve(ws, nnz, total_rows, o->num_sc_per_device, o->num_sc_per_device * o->global_device_count, &s);
  return ws.used();
}

extern "C" int32_t sc_preprocess_table(const int32_t* ids, const int32_t* row_offsets, const float* weights, int64_t nnz,
                                       int64_t total_rows, const sc_feature_desc_t* features, int32_t num_features,
                                       const sc_preprocess_options_t* o, int32_t* row_pointers, int32_t* embedding_ids,
                                       int32_t* sample_ids, float* gains, int32_t* stats, void* workspace, size_t workspace_bytes,
                                       sc_stream_t stream) {
  int st = check_options(o);
  if (st != SC_OK) return st;
  if (num_features <= 0 || !features) SC_FAIL(SC_INVALID_ARGUMENT, "input_batches cannot be empty.");
  if (num_features > SC_MAX_FEATURES) SC_FAIL(SC_UNSUPPORTED, "%d features exceed SC_MAX_FEATURES", num_features);
  if (nnz < 0 || nnz >= (1LL << 31) || total_rows <= 0 || total_rows >= (1LL << 31)) SC_FAIL(SC_INVALID_ARGUMENT, "bad nnz or row count");
  if (!row_offsets || (nnz > 0 && !ids) || !row_pointers || !embedding_ids || !sample_ids || !gains || !stats)
    SC_FAIL(SC_INVALID_ARGUMENT, "null input or output pointer");
  const int S = o->num_sc_per_device, C = o->global_device_count, P = S * C;
  int64_t rows = 0;
  for (int f = 0; f < num_features; ++f) {
    if (features[f].row_begin != rows || features[f].rows < 0) SC_FAIL(SC_INVALID_ARGUMENT, "features must tile the row range in order");
    if (features[f].rows % S) SC_FAIL(SC_INVALID_ARGUMENT, "rows of feature %d (%d) must be divisible by num_sc_per_device (%d)", f, features[f].rows, S);
    if (features[f].col_offset & (P - 1)) SC_FAIL(SC_INVALID_ARGUMENT, "col_offset must be a multiple of the shard count");
    rows += features[f].rows;
  }
  if (rows != total_rows) SC_FAIL(SC_INVALID_ARGUMENT, "feature rows (%lld) do not add up to total_rows (%lld)", (long long)rows, (long long)total_rows);
  // ValidateLocalBatchSizeLimits (input_preprocessing.cc:757-786): 26-bit sample field.
  if (total_rows > ((1 << 26) - 1))
    SC_FAIL(SC_INVALID_ARGUMENT,
            "The total local batch size for device (including stacked tables) exceeds the maximum limit supported by the "
            "SparseCore CooFormat sorting key (%d).", (1 << 26) - 1);
  if (nnz > (1LL << 26) * S) SC_FAIL(SC_UNSUPPORTED, "too many ids for one device");

  PreParams p;
  p.S = S; p.P = P; p.C = C;
  p.pbits = bit_width_u32((uint32_t)P - 1);
  p.lbits = bit_width_u32((uint32_t)(o->stack_vocab_size / P) - 1);
  if (p.lbits == 0) p.lbits = 1;
  const int sbits = bit_width_u32((uint32_t)S - 1);
  if (sbits + p.pbits + p.lbits > 32) SC_FAIL(SC_UNSUPPORTED, "stacked vocabulary too large for a 32-bit sort key");
  p.bslice = (int32_t)ceil_div(total_rows, S);
  p.combiner = o->combiner; p.has_weights = weights != nullptr;
  p.max_ids = o->max_ids_per_partition; p.max_unique = o->max_unique_ids_per_partition; p.allow_drop = o->allow_id_dropping != 0;
  p.coo_per_sc = o->coo_buffer_size_per_device / S; p.R = P > kAlign ? P : kAlign;
  p.num_features = num_features; p.nnz = nnz; p.total_rows = total_rows;

  Workspace ws(workspace, workspace_bytes);
  PreScratch s;
  if (!carve(ws, nnz, total_rows, S, P, &s))
    SC_FAIL(SC_WORKSPACE_TOO_SMALL, "preprocessing needs %zu workspace bytes, got %zu", ws.used(), workspace_bytes);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const int coo = o->coo_buffer_size_per_device;

  SC_CUDA_OK(cudaMemcpyAsync(s.feats, features, sizeof(sc_feature_desc_t) * num_features, cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(cudaMemsetAsync(s.error_flag, 0, sizeof(int32_t), cs));
  extract_kernel<<<(unsigned)ceil_div(total_rows, kBlock), kBlock, 0, cs>>>(p, s.feats, ids, row_offsets, weights, s.sort.keys[0],
                                                                         s.row_of, s.gain_of, s.row_gain, s.error_flag);
  SC_LAUNCH_OK("extract_kernel");
  int res = 0;
  SC_CUDA_OK(radix_sort_pairs(s.sort, (size_t)nnz, sbits + p.pbits + p.lbits, true, &res, cs));
  const uint32_t* keys = s.sort.keys[res];
  const uint32_t* vals = s.sort.vals[res];
  if (nnz > 0) {
    flags_kernel<<<(unsigned)ceil_div(nnz, kBlock), kBlock, 0, cs>>>(nnz, keys, vals, s.row_of, s.row_sorted, s.cnt);
    SC_LAUNCH_OK("flags_kernel");
  }
  SC_CUDA_OK(exclusive_scan<uint64_t>(s.cnt, s.cnt, (size_t)nnz, s.scan_temp, s.cnt + nnz, cs));
  const int parts = S * P;
  bounds_kernel<<<(unsigned)ceil_div(parts + 1, kBlock), kBlock, 0, cs>>>(nnz, keys, p.lbits, parts, s.bounds);
  SC_LAUNCH_OK("bounds_kernel");
  layout_kernel<<<1, kMaxPartitions, 0, cs>>>(p, s.cnt, s.bounds, s.part_start, s.part_written, row_pointers, stats, s.error_flag);
  SC_LAUNCH_OK("layout_kernel");
  fill_kernel<<<(unsigned)ceil_div(coo, kBlock), kBlock, 0, cs>>>(coo, embedding_ids, sample_ids, gains);
  SC_LAUNCH_OK("fill_kernel");
  if (nnz > 0) {
    pack_kernel<<<(unsigned)ceil_div(nnz, kBlock), kBlock, 0, cs>>>(p, keys, vals, s.row_sorted, s.gain_of, s.row_gain, s.cnt, s.bounds,
                                                                 s.part_start, s.part_written, embedding_ids, sample_ids, gains);
    SC_LAUNCH_OK("pack_kernel");
  }
  return SC_OK;
}
