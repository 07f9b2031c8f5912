// GPU input preprocessing: ragged ids of one device -> CSR-wrapped COO buffers.
//
// Replaces the host C++ pipeline of the reference (extract -> 64-bit keys -> VQSort ->
// sequential group/dedup -> fill; jax_tpu_embedding/sparsecore/lib/core/
// input_preprocessing.cc, sort_and_group_coo_tensors_impl.h, input_preprocessing_util.cc)
// with data-parallel kernels whose output is bit-identical over the region the reference
// writes.  One call serves a GROUP of stacked tables: every kernel below is launched once for
// all of them (the reference runs one thread-pool task per table, device and SparseCore).
//
//   extract   one thread per sample row: column id with table-stack shift/offset, sample id
//             with split-then-stack row offsets, f32 gain with the reference's rounding order;
//   sort      the reference orders entries by (SparseCore, shard, row of the shard, sample).
//             Entries are already in ascending sample order per SparseCore, so a STABLE radix
//             sort on the compact key (table | SparseCore | shard | local row) alone is enough:
//             3-4 byte passes over 32-bit keys instead of 64-bit keys;
//   group     head flags of (row, sample) pairs and of rows -> one 64-bit exclusive scan gives
//             the rank of every pair and of every unique row inside its partition; the
//             sequential drop rules of the reference reduce to "keep a prefix of each partition";
//   pack      per-partition 8-aligned offsets, row pointers, padding, duplicate gains summed
//             left to right in float32;
//   plan      (optional) the sample-major view the forward needs: the input is sample-major and
//             every kept entry knows its slot, so the slot is scattered back to the entry's input
//             position and each sample's slots are put in ascending order.
#include <math.h>

#include <vector>

#include "sc_common.cuh"
#include "sc_sort.cuh"

namespace sc {
namespace {

constexpr int kBlock = 256;
constexpr int kMaxPartitions = 4 * SC_MAX_SHARDS;  // local SparseCores x shards of one table
constexpr uint32_t kNoSlot = 0xffffffffu;          // forward plan: input position whose id was merged or dropped
constexpr uint32_t kSerialBagLimit = 64;           // longer bags are ordered by a whole warp

// One stacked table of a grouped call (device memory).
struct PreTable {
  const int32_t* ids;
  const int32_t* offsets;  // [rows + 1], or nullptr when every feature has a fixed valency
  const float* weights;    // nullptr = unity weights
  int32_t* row_pointers;
  int32_t* out_ids;
  int32_t* out_sids;
  float* out_gains;
  int32_t* stats;
  uint32_t* plan_slots;     // [nnz] forward plan (nullptr: not wanted)
  uint32_t* plan_bags;      // [2 * rows]
  int32_t S, P, C;          // SparseCores per device, shards, devices
  int32_t pbits, lbits;     // bits of the shard id and of the row inside a shard
  int32_t bslice;           // samples per SparseCore slice (ceil(batch / S))
  int32_t combiner, has_weights;
  int32_t max_ids, max_unique, allow_drop;
  int32_t coo, coo_per_sc, R;
  int32_t num_features;
  uint32_t feat_base;       // first entry of this table in the feature array
  uint32_t id_base;         // first global id index
  uint32_t row_base;        // first global input row
  uint32_t gain_base;       // first entry in the per-sample gain array
  uint32_t part_base;       // first global partition (bounds has one extra entry per table)
  uint32_t slot_base;       // first global output slot
  uint32_t nnz, rows;
};

struct PreGroup {
  const PreTable* tabs;
  const sc_feature_desc_t* feats;
  int32_t count;
  int32_t tshift;  // bit position of the table index inside the sort key
  uint32_t total_ids, total_rows, total_slots, total_parts;
};

template <typename F>
__device__ __forceinline__ int find_table(int count, uint32_t x, F base_of) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (base_of(mid) <= x) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ---- extract ---------------------------------------------------------------------------
// Restates ProcessCooTensors (process_coo_tensors_impl.h:79-136), ComputeWeightDivisor
// (:39-77), CooFormat::GetColId (coo_format.h:120-135) and the slice arithmetic of
// ExtractCooTensorsForAllFeaturesPerLocalDevice (input_preprocessing.cc:79-123, 312-436).
__global__ void extract_kernel(PreGroup g, uint32_t* __restrict__ keys, int32_t* __restrict__ row_of,
                               float* __restrict__ gain_of, float* __restrict__ row_gain, int32_t* __restrict__ error_flags) {
  const uint32_t gr = blockIdx.x * blockDim.x + threadIdx.x;
  if (gr >= g.total_rows) return;
  const int t = find_table(g.count, gr, [&](int i) { return g.tabs[i].row_base; });
  const PreTable& p = g.tabs[t];
  const int r = (int)(gr - p.row_base);
  const sc_feature_desc_t* feats = g.feats + p.feat_base;
  int lo = 0, hi = p.num_features - 1;  // last feature with row_begin <= r
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (feats[mid].row_begin <= r) lo = mid; else hi = mid - 1;
  }
  const sc_feature_desc_t fd = feats[lo];
  const int rf = r - fd.row_begin;
  const int per_slice = fd.rows / p.S;
  const int s = min(rf / max(per_slice, 1), p.S - 1);
  int row_id = s * p.bslice + fd.row_offset / (p.C * p.S) + (rf - s * per_slice);
  if (row_id < 0 || row_id >= p.S * p.bslice) {  // row offsets inconsistent with the batch
    atomicOr(&error_flags[t], 1);
    row_id = 0;
  }
  int b, e;
  if (fd.valency > 0) {
    b = fd.id_begin + rf * fd.valency;
    e = b + fd.valency;
  } else {
    b = p.offsets[r];
    e = p.offsets[r + 1];
  }
  const int cnt = e - b;
  if (p.plan_bags != nullptr) reinterpret_cast<uint2*>(p.plan_bags)[row_id] = make_uint2((uint32_t)b, (uint32_t)e);
  const int32_t* ids = p.ids;
  const float* weights = p.weights;
  float divisor = 1.0f;
  if (!p.has_weights) {
    float gain = 1.0f;
    if (p.combiner == SC_COMBINER_MEAN) gain = 1.0f / (float)cnt;
    else if (p.combiner == SC_COMBINER_SQRTN) gain = 1.0f / sqrtf((float)cnt);
    row_gain[p.gain_base + row_id] = gain;
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
  const uint32_t key_hi = (g.tshift < 32 ? ((uint32_t)t << g.tshift) : 0u) | ((uint32_t)s << (p.pbits + p.lbits));
  for (int i = b; i < e; ++i) {
    const int id = ids[i];
    const int col = ((id + fd.col_shift) & mod) + (id & ~mod) + fd.col_offset;
    const uint32_t shard = (uint32_t)(col & mod);
    uint32_t local = (uint32_t)col >> p.pbits;
    if (id < 0 || local >= local_limit) {
      atomicOr(&error_flags[t], 1);
      local = local_limit - 1;
    }
    keys[p.id_base + i] = key_hi | (shard << p.lbits) | local;
    row_of[p.id_base + i] = row_id;
    if (p.has_weights) gain_of[p.id_base + i] = weights[i] / divisor;
    if (p.plan_slots != nullptr) p.plan_slots[i] = kNoSlot;
  }
}

// ---- group -----------------------------------------------------------------------------
// flags[p] = (pair head) | (row head) << 32, in sorted order; also keeps the sample of
// every sorted entry.  A pair head is the first entry of a (table, SparseCore, column, sample)
// group, i.e. what GroupAndDeduplicateCooTensorsForLocalSparseCore
// (sort_and_group_coo_tensors_impl.h:235-310) treats as a new id.
__global__ void flags_kernel(uint32_t n, const uint32_t* __restrict__ keys, const uint32_t* __restrict__ vals,
                             const int32_t* __restrict__ row_of, int32_t* __restrict__ row_sorted, uint64_t* __restrict__ flags) {
  const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
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

// bounds[part_base(t) + t + q] = first sorted position whose (table, partition) is >= (t, q),
// for q in [0, S*P] of every table t.
__global__ void bounds_kernel(PreGroup g, uint32_t n, const uint32_t* __restrict__ keys, int32_t* __restrict__ bounds) {
  const uint32_t x = blockIdx.x * blockDim.x + threadIdx.x;
  if (x >= g.total_parts + (uint32_t)g.count) return;
  const int t = find_table(g.count, x, [&](int i) { return g.tabs[i].part_base + (uint32_t)i; });
  const PreTable& p = g.tabs[t];
  const uint32_t q = x - (p.part_base + (uint32_t)t);
  const uint64_t target = ((uint64_t)t << g.tshift) + ((uint64_t)q << p.lbits);  // q == S*P carries into the table bits
  uint32_t lo = 0, hi = n;
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    if ((uint64_t)keys[mid] < target) lo = mid + 1; else hi = mid;
  }
  bounds[x] = (int32_t)lo;
}

__device__ __forceinline__ uint32_t lo32(uint64_t v) { return (uint32_t)v; }
__device__ __forceinline__ uint32_t hi32(uint64_t v) { return (uint32_t)(v >> 32); }
__device__ __forceinline__ int round8(int v) { return (v + kAlign - 1) & ~(kAlign - 1); }

// One block per table.  Thread q < S*P measures partition q; thread s < S then lays out
// SparseCore s.  cnt is the exclusive scan of flags with the grand total at cnt[n].
__global__ void layout_kernel(PreGroup g, const uint64_t* __restrict__ cnt, const int32_t* __restrict__ bounds_all,
                              int32_t* __restrict__ part_start_all, int32_t* __restrict__ part_written_all,
                              const int32_t* __restrict__ error_flags) {
  __shared__ int32_t s_ids[kMaxPartitions], s_uniq[kMaxPartitions], s_kept[kMaxPartitions];
  __shared__ int32_t s_drop_limit[kMaxPartitions], s_drop_static[kMaxPartitions];
  const int t = blockIdx.x;
  const PreTable& p = g.tabs[t];
  const int32_t* bounds = bounds_all + p.part_base + t;
  int32_t* part_start = part_start_all + p.part_base;
  int32_t* part_written = part_written_all + p.part_base;
  int32_t* stats = p.stats;
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
    for (int sh = 0; sh < p.P; ++sh) {
      const int idx = s * p.P + sh;
      const int written = max(0, min(s_kept[idx], p.coo_per_sc - cursor));
      part_start[idx] = cursor;
      part_written[idx] = written;
      s_drop_static[idx] = s_kept[idx] - written;
      const int end = cursor + s_kept[idx];
      p.row_pointers[s * p.R + sh] = min(end, p.coo_per_sc);
      cursor = round8(end);
      required += round8(s_ids[idx]);
    }
    for (int sh = p.P; sh < p.R; ++sh) p.row_pointers[s * p.R + sh] = min(cursor, p.coo_per_sc);
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
    if (error_flags[t]) status = SC_INVALID_ARGUMENT;
    stats[2 * p.P + p.S + 1] = status;
    stats[2 * p.P + p.S + 2] = written;
  }
}

__global__ void fill_kernel(PreGroup g) {
  const uint32_t gq = blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= g.total_slots) return;
  const int t = find_table(g.count, gq, [&](int i) { return g.tabs[i].slot_base; });
  const PreTable& p = g.tabs[t];
  const uint32_t q = gq - p.slot_base;
  p.out_ids[q] = SC_PADDING_VALUE;
  p.out_sids[q] = SC_PADDING_VALUE;
  p.out_gains[q] = nanf("");
}

// One thread per sorted entry; pair heads that survive write their slot.  Duplicates are
// summed left to right, as PartitionedCooTensors::MergeWithLastCoo does
// (partitioned_coo_tensors.h:94-101).
__global__ void pack_kernel(PreGroup g, uint32_t n, const uint32_t* __restrict__ keys, const uint32_t* __restrict__ vals,
                            const int32_t* __restrict__ row_sorted, const float* __restrict__ gain_of,
                            const float* __restrict__ row_gain, const uint64_t* __restrict__ cnt,
                            const int32_t* __restrict__ bounds_all, const int32_t* __restrict__ part_start_all,
                            const int32_t* __restrict__ part_written_all) {
  const uint32_t pos = blockIdx.x * blockDim.x + threadIdx.x;
  if (pos >= n) return;
  const uint64_t c0 = cnt[pos], c1 = cnt[pos + 1];
  if (lo32(c1) == lo32(c0)) return;  // duplicate of an earlier entry
  const uint32_t key = keys[pos];
  const int t = g.tshift < 32 ? (int)(key >> g.tshift) : 0;
  const PreTable& p = g.tabs[t];
  const uint32_t local_key = key & ((g.tshift >= 32) ? 0xffffffffu : ((1u << g.tshift) - 1u));
  const int part = (int)(local_key >> p.lbits);
  const int32_t* bounds = bounds_all + p.part_base + t;
  const int a = bounds[part], b = bounds[part + 1];
  const int j = (int)(lo32(c0) - lo32(cnt[a]));
  if (j >= part_written_all[p.part_base + part]) return;
  const int row = row_sorted[pos];
  float gain = p.has_weights ? gain_of[vals[pos]] : row_gain[p.gain_base + row];
  for (uint32_t u = pos + 1; u < (uint32_t)b && lo32(cnt[u + 1]) == lo32(cnt[u]); ++u) {
    gain += p.has_weights ? gain_of[vals[u]] : row_gain[p.gain_base + row];
  }
  const int s = part / p.P;
  const int64_t slot = (int64_t)s * p.coo_per_sc + part_start_all[p.part_base + part] + j;
  p.out_ids[slot] = (int32_t)(local_key & ((1u << p.lbits) - 1u));
  p.out_sids[slot] = row % p.bslice;
  p.out_gains[slot] = gain;
  if (p.plan_slots != nullptr) p.plan_slots[vals[pos] - p.id_base] = (uint32_t)slot;
}

// Forward plan, last step.  Thread per sample row: the row's input positions now hold the slots of
// its kept entries (kNoSlot elsewhere); they are put in ascending order, kNoSlot last, and the bag
// is shortened to the kept ones.  Slots are unique, so the result does not depend on the order in
// which pack_kernel ran.  Bags longer than kSerialBagLimit go to plan_bigrow_kernel.
__global__ void plan_sort_kernel(PreGroup g, uint32_t* __restrict__ big_rows, uint32_t* __restrict__ big_count) {
  const uint32_t gr = blockIdx.x * blockDim.x + threadIdx.x;
  if (gr >= g.total_rows) return;
  const int t = find_table(g.count, gr, [&](int i) { return g.tabs[i].row_base; });
  const PreTable& p = g.tabs[t];
  if (p.plan_bags == nullptr) return;
  uint2* bag = reinterpret_cast<uint2*>(p.plan_bags) + (gr - p.row_base);
  const uint32_t b = bag->x, n = bag->y - b;
  uint32_t* a = p.plan_slots + b;
  if (n > kSerialBagLimit) {
    big_rows[atomicAdd(big_count, 1u)] = gr;
    return;
  }
  uint32_t kept = 0;
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t x = a[i];
    if (x == kNoSlot) continue;
    uint32_t j = kept++;
    while (j > 0 && a[j - 1] > x) { a[j] = a[j - 1]; --j; }
    a[j] = x;
  }
  bag->y = b + kept;
}

// Warp per long bag: rank sort.  The bag is copied to `scratch` (indexed like the group's id array);
// the rank of a kept slot is the number of smaller kept slots.
__global__ void __launch_bounds__(kBlock) plan_bigrow_kernel(PreGroup g, const uint32_t* __restrict__ big_rows,
                                                             const uint32_t* __restrict__ big_count,
                                                             uint32_t* __restrict__ scratch) {
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (kBlock / 32);
  const uint32_t todo = *big_count;
  for (uint32_t w = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); w < todo; w += warps) {
    const uint32_t gr = big_rows[w];
    const int t = find_table(g.count, gr, [&](int i) { return g.tabs[i].row_base; });
    const PreTable& p = g.tabs[t];
    uint2* bag = reinterpret_cast<uint2*>(p.plan_bags) + (gr - p.row_base);
    const uint32_t b = bag->x, n = bag->y - b;
    uint32_t* a = p.plan_slots + b;
    uint32_t* tmp = scratch + p.id_base + b;
    uint32_t kept = 0;
    for (uint32_t i = lane; i < n; i += 32) {
      const uint32_t x = a[i];
      tmp[i] = x;
      kept += x != kNoSlot ? 1u : 0u;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) kept += __shfl_xor_sync(0xffffffffu, kept, d);
    __syncwarp();
    for (uint32_t i = lane; i < n; i += 32) {
      const uint32_t x = tmp[i];
      if (x == kNoSlot) continue;
      uint32_t rank = 0;
      for (uint32_t j = 0; j < n; ++j) rank += tmp[j] < x ? 1u : 0u;
      a[rank] = x;
    }
    __syncwarp();
    if (lane == 0) bag->y = b + kept;
    __syncwarp();
  }
}

// ---- host side ---------------------------------------------------------------------------

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

struct PrePlan {
  std::vector<PreTable> tabs;
  std::vector<sc_feature_desc_t> feats;
  uint64_t total_ids = 0, total_rows = 0, total_slots = 0, total_parts = 0, total_gain = 0;
  int key_bits = 0;  // bits of the per-table part of the key
  int tshift = 0, total_bits = 0;
  bool any_plan = false;
};

int plan(const sc_preprocess_item_t* items, int count, PrePlan* pl) {
  if (!items || count <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "input_batches cannot be empty.");
  pl->tabs.resize(count);
  for (int t = 0; t < count; ++t) {
    const sc_preprocess_item_t& it = items[t];
    const sc_preprocess_options_t* o = &it.options;
    int st = check_options(o);
    if (st != SC_OK) return st;
    if (it.num_features <= 0 || !it.features) SC_FAIL(SC_INVALID_ARGUMENT, "input_batches cannot be empty.");
    if (it.num_features > SC_MAX_FEATURES) SC_FAIL(SC_UNSUPPORTED, "%d features exceed SC_MAX_FEATURES", it.num_features);
    if (it.nnz < 0 || it.nnz >= (1LL << 31) || it.total_rows <= 0 || it.total_rows >= (1LL << 31))
      SC_FAIL(SC_INVALID_ARGUMENT, "bad nnz or row count");
    if ((it.nnz > 0 && !it.ids) || !it.row_pointers || !it.embedding_ids || !it.sample_ids || !it.gains || !it.stats)
      SC_FAIL(SC_INVALID_ARGUMENT, "null input or output pointer");
    const int S = o->num_sc_per_device, C = o->global_device_count, P = S * C;
    int64_t rows = 0;
    bool need_offsets = false;
    for (int f = 0; f < it.num_features; ++f) {
      const sc_feature_desc_t& fd = it.features[f];
      if (fd.row_begin != rows || fd.rows < 0) SC_FAIL(SC_INVALID_ARGUMENT, "features must tile the row range in order");
      if (fd.rows % S)
        SC_FAIL(SC_INVALID_ARGUMENT, "rows of feature %d (%d) must be divisible by num_sc_per_device (%d)", f, fd.rows, S);
      if (fd.col_offset & (P - 1)) SC_FAIL(SC_INVALID_ARGUMENT, "col_offset must be a multiple of the shard count");
      if (fd.valency < 0) SC_FAIL(SC_INVALID_ARGUMENT, "negative valency");
      if (fd.valency == 0) need_offsets = true;
      else if (fd.id_begin < 0 || (int64_t)fd.id_begin + (int64_t)fd.rows * fd.valency > it.nnz)
        SC_FAIL(SC_INVALID_ARGUMENT, "fixed-valency feature %d exceeds the id array", f);
      rows += fd.rows;
      pl->feats.push_back(fd);
    }
    if (need_offsets && !it.row_offsets) SC_FAIL(SC_INVALID_ARGUMENT, "row_offsets are required for ragged features");
    if (rows != it.total_rows)
      SC_FAIL(SC_INVALID_ARGUMENT, "feature rows (%lld) do not add up to total_rows (%lld)", (long long)rows, (long long)it.total_rows);
    // ValidateLocalBatchSizeLimits (input_preprocessing.cc:757-786): 26-bit sample field.
    if (it.total_rows > ((1 << 26) - 1))
      SC_FAIL(SC_INVALID_ARGUMENT,
              "The total local batch size for device (including stacked tables) exceeds the maximum limit supported by the "
              "SparseCore CooFormat sorting key (%d).", (1 << 26) - 1);
    if (it.nnz > (1LL << 26) * S) SC_FAIL(SC_UNSUPPORTED, "too many ids for one device");

    PreTable& p = pl->tabs[t];
    memset(&p, 0, sizeof p);
    p.ids = it.ids; p.offsets = it.row_offsets; p.weights = it.weights;
    p.row_pointers = it.row_pointers; p.out_ids = it.embedding_ids; p.out_sids = it.sample_ids; p.out_gains = it.gains;
    p.stats = it.stats;
    if ((it.plan_slots == nullptr) != (it.plan_bags == nullptr))
      SC_FAIL(SC_INVALID_ARGUMENT, "plan_slots and plan_bags must be given together");
    p.plan_slots = it.plan_slots; p.plan_bags = it.plan_bags;
    pl->any_plan = pl->any_plan || it.plan_bags != nullptr;
    p.S = S; p.P = P; p.C = C;
    p.pbits = bit_width_u32((uint32_t)P - 1);
    p.lbits = bit_width_u32((uint32_t)(o->stack_vocab_size / P) - 1);
    if (p.lbits == 0) p.lbits = 1;
    const int bits = bit_width_u32((uint32_t)S - 1) + p.pbits + p.lbits;
    // One more bit so that the end sentinel (S*P << lbits) of a table stays below the next table.
    pl->key_bits = bits > pl->key_bits ? bits : pl->key_bits;
    p.bslice = (int32_t)ceil_div(it.total_rows, S);
    p.combiner = o->combiner; p.has_weights = it.weights != nullptr;
    p.max_ids = o->max_ids_per_partition; p.max_unique = o->max_unique_ids_per_partition; p.allow_drop = o->allow_id_dropping != 0;
    p.coo = o->coo_buffer_size_per_device; p.coo_per_sc = p.coo / S; p.R = P > kAlign ? P : kAlign;
    p.num_features = it.num_features;
    p.feat_base = (uint32_t)(pl->feats.size() - it.num_features);
    p.id_base = (uint32_t)pl->total_ids; p.row_base = (uint32_t)pl->total_rows; p.gain_base = (uint32_t)pl->total_gain;
    p.part_base = (uint32_t)pl->total_parts; p.slot_base = (uint32_t)pl->total_slots;
    p.nnz = (uint32_t)it.nnz; p.rows = (uint32_t)it.total_rows;
    pl->total_ids += (uint64_t)it.nnz; pl->total_rows += (uint64_t)it.total_rows;
    pl->total_gain += (uint64_t)S * p.bslice + 8;
    pl->total_parts += (uint64_t)S * P; pl->total_slots += (uint64_t)p.coo;
  }
  pl->tshift = pl->key_bits;
  pl->total_bits = pl->tshift + bit_width_u32((uint32_t)count - 1);
  if (pl->total_bits > 32)
    SC_FAIL(SC_UNSUPPORTED, "group needs a %d-bit sort key; preprocess fewer tables per call", pl->total_bits);
  if (pl->total_ids >= 0x7fffffffull || pl->total_rows >= 0x7fffffffull || pl->total_slots >= 0xffffffffull)
    SC_FAIL(SC_UNSUPPORTED, "group too large for 32-bit indices");
  return SC_OK;
}

struct PreScratch {
  PreTable* tabs;
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
  int32_t* error_flags;
  uint32_t* big_rows;  // forward plan: rows with long bags, then their count
};

bool carve(Workspace& ws, const PrePlan& pl, int count, PreScratch* s) {
  const size_t n = (size_t)(pl.total_ids > 0 ? pl.total_ids : 1);
  s->tabs = ws.take<PreTable>((size_t)count);
  s->feats = ws.take<sc_feature_desc_t>(pl.feats.size() + 1);
  s->sort.keys[0] = ws.take<uint32_t>(n); s->sort.keys[1] = ws.take<uint32_t>(n);
  s->sort.vals[0] = ws.take<uint32_t>(n); s->sort.vals[1] = ws.take<uint32_t>(n);
  s->sort.hist = ws.take<uint32_t>(sort_hist_elems(n));
  s->sort.scan_temp = ws.take<uint32_t>(scan_temp_elems(sort_hist_elems(n)));
  s->row_of = ws.take<int32_t>(n);
  s->row_sorted = ws.take<int32_t>(n);
  s->gain_of = ws.take<float>(n);
  s->row_gain = ws.take<float>((size_t)pl.total_gain + 8);
  s->cnt = ws.take<uint64_t>(n + 1);
  s->scan_temp = ws.take<uint64_t>(scan_temp_elems(n));
  s->bounds = ws.take<int32_t>((size_t)pl.total_parts + (size_t)count + 1);
  s->part_start = ws.take<int32_t>((size_t)pl.total_parts + 1);
  s->part_written = ws.take<int32_t>((size_t)pl.total_parts + 1);
  s->error_flags = ws.take<int32_t>((size_t)count);
  s->big_rows = ws.take<uint32_t>(pl.any_plan ? n / kSerialBagLimit + 2 : 0);
  return ws.ok();
}

}  // namespace
}  // namespace sc

using namespace sc;

extern "C" int32_t sc_preprocess_stats_size(int32_t global_device_count, int32_t num_sc_per_device) {
  return 2 * global_device_count * num_sc_per_device + num_sc_per_device + 3;
}

extern "C" size_t sc_preprocess_grouped_workspace_bytes(const sc_preprocess_item_t* items, int32_t count) {
  PrePlan pl;
  if (plan(items, count, &pl) != SC_OK) return 0;
  Workspace ws(nullptr, 0);
  PreScratch s;
  carve(ws, pl, count, &s);
  return ws.used();
}

extern "C" int32_t sc_preprocess_grouped(const sc_preprocess_item_t* items, int32_t count, void* workspace,
                                         size_t workspace_bytes, sc_stream_t stream) {
  PrePlan pl;
  int st = plan(items, count, &pl);
  if (st != SC_OK) return st;
  Workspace ws(workspace, workspace_bytes);
  PreScratch s;
  if (!carve(ws, pl, count, &s))
    SC_FAIL(SC_WORKSPACE_TOO_SMALL, "preprocessing needs %zu workspace bytes, got %zu", ws.used(), workspace_bytes);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  // Pageable sources: each call returns once the bytes are staged, so the vectors may go away.
  SC_CUDA_OK(cudaMemcpyAsync(s.tabs, pl.tabs.data(), sizeof(PreTable) * count, cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(cudaMemcpyAsync(s.feats, pl.feats.data(), sizeof(sc_feature_desc_t) * pl.feats.size(), cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(cudaMemsetAsync(s.error_flags, 0, sizeof(int32_t) * count, cs));
  PreGroup g;
  g.tabs = s.tabs; g.feats = s.feats; g.count = count; g.tshift = pl.tshift;
  g.total_ids = (uint32_t)pl.total_ids; g.total_rows = (uint32_t)pl.total_rows;
  g.total_slots = (uint32_t)pl.total_slots; g.total_parts = (uint32_t)pl.total_parts;
  const uint32_t n = g.total_ids;

  PhaseScope whole("jax_sc_embedding::PreprocessSparseDenseMatmulInput", cs);
  {
    PhaseScope phase("ExtractCooTensors", cs);
    extract_kernel<<<(unsigned)ceil_div(g.total_rows, kBlock), kBlock, 0, cs>>>(g, s.sort.keys[0], s.row_of, s.gain_of, s.row_gain,
                                                                              s.error_flags);
    SC_LAUNCH_OK("extract_kernel");
  }
  int res = 0;
  const uint32_t* keys = nullptr;
  const uint32_t* vals = nullptr;
  {
    PhaseScope phase("SortAndGroup", cs);
    SC_CUDA_OK(radix_sort_pairs(s.sort, (size_t)n, pl.total_bits, true, &res, cs));
    keys = s.sort.keys[res];
    vals = s.sort.vals[res];
    if (n > 0) {
      flags_kernel<<<(unsigned)ceil_div(n, kBlock), kBlock, 0, cs>>>(n, keys, vals, s.row_of, s.row_sorted, s.cnt);
      SC_LAUNCH_OK("flags_kernel");
    }
    SC_CUDA_OK(exclusive_scan<uint64_t>(s.cnt, s.cnt, (size_t)n, s.scan_temp, s.cnt + n, cs));
    bounds_kernel<<<(unsigned)ceil_div((int64_t)g.total_parts + count, kBlock), kBlock, 0, cs>>>(g, n, keys, s.bounds);
    SC_LAUNCH_OK("bounds_kernel");
    layout_kernel<<<count, kMaxPartitions, 0, cs>>>(g, s.cnt, s.bounds, s.part_start, s.part_written, s.error_flags);
    SC_LAUNCH_OK("layout_kernel");
  }
  {
    PhaseScope phase("FillBuffer", cs);
    fill_kernel<<<(unsigned)ceil_div(g.total_slots, kBlock), kBlock, 0, cs>>>(g);
    SC_LAUNCH_OK("fill_kernel");
    if (n > 0) {
      pack_kernel<<<(unsigned)ceil_div(n, kBlock), kBlock, 0, cs>>>(g, n, keys, vals, s.row_sorted, s.gain_of, s.row_gain, s.cnt,
                                                                  s.bounds, s.part_start, s.part_written);
      SC_LAUNCH_OK("pack_kernel");
    }
  }
  if (pl.any_plan) {
    PhaseScope phase("ForwardPlan", cs);
    uint32_t* big_count = s.big_rows + n / kSerialBagLimit + 1;
    SC_CUDA_OK(cudaMemsetAsync(big_count, 0, sizeof(uint32_t), cs));
    plan_sort_kernel<<<(unsigned)ceil_div(g.total_rows, kBlock), kBlock, 0, cs>>>(g, s.big_rows, big_count);
    SC_LAUNCH_OK("plan_sort_kernel");
    // The sort buffer that does not hold the sorted keys is free by now.
    plan_bigrow_kernel<<<(unsigned)sm_count(), kBlock, 0, cs>>>(g, s.big_rows, big_count, s.sort.keys[1 - res]);
    SC_LAUNCH_OK("plan_bigrow_kernel");
  }
  return SC_OK;
}

// ---- single-table entry points: groups of one ----------------------------------------------

static sc_preprocess_item_t make_item(const int32_t* ids, const int32_t* row_offsets, const float* weights, int64_t nnz,
                                      int64_t total_rows, const sc_feature_desc_t* features, int32_t num_features,
                                      const sc_preprocess_options_t* o, int32_t* row_pointers, int32_t* embedding_ids,
                                      int32_t* sample_ids, float* gains, int32_t* stats) {
  sc_preprocess_item_t it;
  memset(&it, 0, sizeof it);
  it.ids = ids; it.row_offsets = row_offsets; it.weights = weights; it.nnz = nnz; it.total_rows = total_rows;
  it.features = features; it.num_features = num_features;
  if (o) it.options = *o;
  it.row_pointers = row_pointers; it.embedding_ids = embedding_ids; it.sample_ids = sample_ids; it.gains = gains;
  it.stats = stats;
  return it;
}

extern "C" size_t sc_preprocess_workspace_bytes(int64_t nnz, int64_t total_rows, const sc_preprocess_options_t* o) {
  if (!o || total_rows <= 0) return 0;
  // Geometry only: one ragged feature spanning all rows.
  sc_feature_desc_t fd;
  memset(&fd, 0, sizeof fd);
  fd.rows = (int32_t)(total_rows - total_rows % (o->num_sc_per_device > 0 ? o->num_sc_per_device : 1));
  int32_t* dummy = reinterpret_cast<int32_t*>(256);
  sc_preprocess_item_t it = make_item(dummy, dummy, nullptr, nnz, fd.rows, &fd, 1, o, dummy, dummy, dummy,
                                      reinterpret_cast<float*>(256), dummy);
  return sc_preprocess_grouped_workspace_bytes(&it, 1) + (size_t)SC_MAX_FEATURES * sizeof(sc_feature_desc_t);
}

extern "C" int32_t sc_preprocess_table(const int32_t* ids, const int32_t* row_offsets, const float* weights, int64_t nnz,
                                       int64_t total_rows, const sc_feature_desc_t* features, int32_t num_features,
                                       const sc_preprocess_options_t* o, int32_t* row_pointers, int32_t* embedding_ids,
                                       int32_t* sample_ids, float* gains, int32_t* stats, void* workspace, size_t workspace_bytes,
                                       sc_stream_t stream) {
  if (!o) SC_FAIL(SC_INVALID_ARGUMENT, "options are null");
  sc_preprocess_item_t it = make_item(ids, row_offsets, weights, nnz, total_rows, features, num_features, o, row_pointers,
                                      embedding_ids, sample_ids, gains, stats);
  return sc_preprocess_grouped(&it, 1, workspace, workspace_bytes, stream);
}
