/*
 * TEST INFRASTRUCTURE - NOT THE PRODUCT.
 *
 * CPU restatement (plain C11 + pthreads) of the SparseCore input preprocessing
 * of jax-tpu-embedding, used only as the checker in tests/, in the smoke test
 * and as the timed CPU baseline of bench.py.  The shipped path never links,
 * loads or calls this file.
 *
 * Parity status: PINNED.  This restatement is checked against the reference's
 * own hand-written golden vectors by running the reference's Python unit tests
 * (jax_tpu_embedding/sparsecore/lib/core/tests/pybind_input_preprocessing_test.py)
 * on top of it, and against the reference's pure-Python preprocessing
 * (jax_tpu_embedding/sparsecore/lib/core/input_preprocessing.py); see
 * tests/test_oracle_vs_reference.py and tests/golden/.
 *
 * Every function cites the reference lines it restates; paths are relative to
 * jax_tpu_embedding/sparsecore/lib/core/ of the reference project.
 */
#include <limits.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SC_ALIGN 8 /* TPU_VECTOR_REGISTER_ALIGNMENT_SIZE, input_preprocessing_util.h:54 */
#define SC_DATA_BITS 26u /* CooFormat::kDataBits, coo_format.h:62 */
#define SC_DATA_MASK ((1u << SC_DATA_BITS) - 1u)

enum { SC_SUM = 0, SC_MEAN = 1, SC_SQRTN = 2 }; /* RowCombiner, input_preprocessing_util.h:87-91 */

enum {
  SC_OK = 0,
  SC_INVALID_ARGUMENT = 1,
  SC_ID_LIMIT_EXCEEDED = 3, /* the reference LOG(FATAL)s here */
};

/* One feature of a stacked table: a CSR view of this process's rows. */
typedef struct {
  const int32_t* ids;     /* flat embedding ids */
  const int64_t* offsets; /* [rows + 1] */
  const float* weights;   /* NULL when the stack has unity weights */
  int64_t rows;           /* samples held by this process */
  int32_t row_offset;     /* FeatureIdTransformation.row_offset (global) */
  int32_t col_offset;
  int32_t col_shift;
} sc_oracle_feature_t;

typedef struct {
  int32_t local_device_count, global_device_count, num_sc_per_device;
  int32_t combiner;      /* SC_SUM / SC_MEAN / SC_SQRTN */
  int32_t has_weights;   /* stack has variable weights */
  int32_t max_ids_per_partition, max_unique_ids_per_partition;
  int32_t allow_id_dropping;
  int32_t coo_buffer_size_per_device;
  int32_t num_threads;   /* worker threads for the per-SparseCore tasks */
} sc_oracle_options_t;

/* coo_format.h:120-135 GetColId */
static inline int32_t get_col_id(int32_t id, int32_t shift, int32_t off, int32_t mod) {
  return ((id + shift) & mod) + (id & ~mod) + off;
}
static inline uint32_t rotr32(uint32_t v, uint32_t s) {
  s &= 31u;
  return s ? (v >> s) | (v << (32u - s)) : v;
}
static inline uint32_t rotl32(uint32_t v, uint32_t s) {
  s &= 31u;
  return s ? (v << s) | (v >> (32u - s)) : v;
}
/* coo_format.h:154-173 GetGroupingKey with create_buckets=false */
static inline uint64_t grouping_key(uint32_t col_id, uint32_t data, uint32_t bits) {
  return ((uint64_t)rotr32(col_id, bits) << SC_DATA_BITS) | (uint64_t)data;
}
static inline int32_t round_up(int32_t v, int32_t m) { return (v + m - 1) / m * m; }

/* LSD radix sort of 64-bit keys; stands in for hwy::VQSort
 * (sort_and_group_coo_tensors_impl.h:469): keys are unique or identical, so any
 * correct ascending sort yields the same sequence. */
static void sort_u64(uint64_t* keys, uint64_t* tmp, size_t n) {
  if (n < 2) return;
  uint64_t all_or = 0, all_and = ~(uint64_t)0;
  for (size_t i = 0; i < n; ++i) { all_or |= keys[i]; all_and &= keys[i]; }
  uint64_t varying = all_or ^ all_and;
  uint64_t* src = keys; uint64_t* dst = tmp;
  for (int pass = 0; pass < 8; ++pass) {
    int sh = pass * 8;
    if (((varying >> sh) & 0xFF) == 0) continue;
    size_t cnt[256]; memset(cnt, 0, sizeof cnt);
    for (size_t i = 0; i < n; ++i) cnt[(src[i] >> sh) & 0xFF]++;
    size_t sum = 0;
    for (int d = 0; d < 256; ++d) { size_t c = cnt[d]; cnt[d] = sum; sum += c; }
    for (size_t i = 0; i < n; ++i) dst[cnt[(src[i] >> sh) & 0xFF]++] = src[i];
    uint64_t* t = src; src = dst; dst = t;
  }
  if (src != keys) memcpy(keys, src, n * sizeof(uint64_t));
}

typedef struct { int32_t row_id, col_id; float gain; } coo_t; /* coo_format.h:51 CooFormat */

typedef struct {
  /* inputs */
  const sc_oracle_feature_t* feats; int nfeat;
  const sc_oracle_options_t* opt;
  int local_device, local_sc;
  int32_t batch_size_for_device;
  /* outputs (per local device rows) */
  int32_t *row_pointers, *embedding_ids, *sample_ids; float* gains;
  int32_t *max_ids, *max_unique, *required; /* [P], [P], [S] for this device */
  int64_t dropped; int status;
} sc_task_t;

/* One (local device, local SparseCore) task: extraction, key generation, sort,
 * group + dedup (+ drop), stats, buffer fill. */
static void run_task(sc_task_t* t) {
  const sc_oracle_options_t* o = t->opt;
  const int S = o->num_sc_per_device;
  const int P = S * o->global_device_count;
  const int mod = P - 1;
  uint32_t bits = 0; while ((1 << bits) < P) ++bits;
  /* input_preprocessing.cc:348-349 batch_size_per_slice = ceil(batch_for_device / S) */
  const int32_t bslice = (t->batch_size_for_device + S - 1) / S;
  const int sc = t->local_sc;

  /* ---- exact id count for this SC (input_preprocessing.cc:359-397) ---- */
  size_t n = 0;
  for (int f = 0; f < t->nfeat; ++f) {
    const sc_oracle_feature_t* ft = &t->feats[f];
    const int64_t per_split = ft->rows / ((int64_t)o->local_device_count * S);
    int64_t start = ((int64_t)t->local_device * S + sc) * per_split;
    int64_t end = start + per_split; if (end > ft->rows) end = ft->rows;
    n += (size_t)(ft->offsets[end] - ft->offsets[start]);
  }
  uint64_t* keys = (uint64_t*)malloc((n ? n : 1) * 2 * sizeof(uint64_t));
  uint64_t* tmp = keys + (n ? n : 1);
  int32_t* x_row = NULL; int32_t* x_col = NULL; float* x_gain = NULL; /* variable weights */
  int32_t* row_token_counts = NULL; float* row_gains = NULL;          /* unity weights */
  if (o->has_weights) {
    x_row = (int32_t*)malloc((n ? n : 1) * sizeof(int32_t));
    x_col = (int32_t*)malloc((n ? n : 1) * sizeof(int32_t));
    x_gain = (float*)malloc((n ? n : 1) * sizeof(float));
  } else if (o->combiner == SC_MEAN) {
    row_token_counts = (int32_t*)calloc((size_t)bslice, sizeof(int32_t));
  } else if (o->combiner == SC_SQRTN) {
    row_gains = (float*)calloc((size_t)bslice, sizeof(float));
  }

  /* ---- extraction: process_coo_tensors_impl.h:79-136, slice math
   * input_preprocessing.cc:79-123 and :359-383 ---- */
  size_t k = 0;
  for (int f = 0; f < t->nfeat; ++f) {
    const sc_oracle_feature_t* ft = &t->feats[f];
    const int64_t per_split = ft->rows / ((int64_t)o->local_device_count * S);
    int64_t start = ((int64_t)t->local_device * S + sc) * per_split;
    int64_t end = start + per_split; if (end > ft->rows) end = ft->rows;
    const int32_t row_offset_per_slice = ft->row_offset / (o->global_device_count * S);
    const int32_t row_offset = sc * bslice + row_offset_per_slice;
    for (int64_t r = start; r < end; ++r) {
      const int32_t sample_id = (int32_t)(r - start) + row_offset;
      const int32_t in_sc = sample_id % bslice;
      const int64_t b = ft->offsets[r], e = ft->offsets[r + 1];
      const int32_t num_cols = (int32_t)(e - b);
      if (!o->has_weights) {
        if (o->combiner == SC_MEAN) {
          row_token_counts[in_sc] = num_cols;
        } else if (o->combiner == SC_SQRTN) {
          /* ComputeWeightDivisor(UnityWeightsStream), :39-51 */
          float divisor = sqrtf((float)num_cols);
          row_gains[in_sc] = 1.0f / divisor;
        }
        for (int64_t i = b; i < e; ++i) {
          int32_t col = get_col_id(ft->ids[i], ft->col_shift, ft->col_offset, mod);
          keys[k++] = grouping_key((uint32_t)col, (uint32_t)sample_id, bits);
        }
      } else {
        /* ComputeWeightDivisor (generic), :54-77.  std::pow(float, int) promotes
         * to double; the double is added to a float accumulator. */
        float divisor = 1.0f;
        if (o->combiner == SC_MEAN) {
          float sum = 0.0f;
          for (int64_t i = b; i < e; ++i) sum += ft->weights[i];
          divisor = sum;
        } else if (o->combiner == SC_SQRTN) {
          float sum = 0.0f;
          for (int64_t i = b; i < e; ++i) sum = (float)((double)sum + pow((double)ft->weights[i], 2.0));
          divisor = sqrtf(sum);
        }
        for (int64_t i = b; i < e; ++i) {
          x_col[k] = get_col_id(ft->ids[i], ft->col_shift, ft->col_offset, mod);
          x_row[k] = sample_id;
          x_gain[k] = ft->weights[i] / divisor;
          /* GenerateKeysFromIds, sort_and_group_coo_tensors_impl.h:313-326 */
          keys[k] = grouping_key((uint32_t)x_col[k], (uint32_t)k, bits);
          ++k;
        }
      }
    }
  }

  sort_u64(keys, tmp, n);

  /* ---- GroupAndDeduplicateCooTensorsForLocalSparseCore,
   * sort_and_group_coo_tensors_impl.h:196-311 (kCreateBuckets = false) ---- */
  coo_t* grouped = (coo_t*)malloc((n ? n : 1) * sizeof(coo_t));
  size_t gsize = 0;
  int32_t* observed_ids = (int32_t*)calloc((size_t)P * 4, sizeof(int32_t));
  int32_t* observed_unique = observed_ids + P;
  int32_t* kept_ids = observed_unique + P;
  int32_t* kept_unique = kept_ids + P;
  const int perform_drop = o->allow_id_dropping; /* minibatching disabled => can_drop_id */
  uint32_t prev_col = UINT32_MAX, prev_row = UINT32_MAX;
  uint32_t dedup_col = UINT32_MAX, dedup_row = UINT32_MAX; /* partitioned_coo_tensors.h:47-48 */
  int dropping_current_unique_col = 0;
  int64_t dropped = 0;
  for (size_t i = 0; i < n; ++i) {
    const uint64_t key = keys[i];
    const uint32_t col_id = rotl32((uint32_t)((key >> SC_DATA_BITS) & 0xFFFFFFFFu), bits);
    const uint32_t g = col_id & (uint32_t)mod;
    uint32_t row_id; float gain;
    /* GetCooFormatWithGain, input_preprocessing_util.h:216-236 */
    if (o->has_weights) {
      const uint32_t idx = (uint32_t)(key & SC_DATA_MASK);
      row_id = (uint32_t)x_row[idx]; gain = x_gain[idx];
    } else {
      row_id = (uint32_t)(key & SC_DATA_MASK);
      if (o->combiner == SC_MEAN) gain = 1.0f / (float)row_token_counts[row_id % (uint32_t)bslice];
      else if (o->combiner == SC_SQRTN) gain = row_gains[row_id % (uint32_t)bslice];
      else gain = 1.0f;
    }
    /* MaybeMerge, partitioned_coo_tensors.h:103-113 */
    if (row_id == dedup_row && col_id == dedup_col) { grouped[gsize - 1].gain += gain; continue; }
    if (perform_drop && row_id == prev_row && col_id == prev_col) { ++dropped; continue; }
    const int is_new_col = col_id != prev_col;
    observed_ids[g] += 1;
    if (is_new_col) observed_unique[g] += 1;
    if (!perform_drop) {
      grouped[gsize].row_id = (int32_t)row_id; grouped[gsize].col_id = (int32_t)col_id; grouped[gsize].gain = gain;
      ++gsize; dedup_col = col_id; dedup_row = row_id;
    } else {
      const int exceeds = (kept_ids[g] + 1) > o->max_ids_per_partition;
      if (is_new_col) dropping_current_unique_col = (kept_unique[g] + 1) > o->max_unique_ids_per_partition;
      if (exceeds || dropping_current_unique_col) {
        ++dropped;
      } else {
        grouped[gsize].row_id = (int32_t)row_id; grouped[gsize].col_id = (int32_t)col_id; grouped[gsize].gain = gain;
        ++gsize; dedup_col = col_id; dedup_row = row_id;
      }
      kept_ids[g] += 1;
      if (is_new_col) kept_unique[g] += 1;
    }
    prev_col = col_id; prev_row = row_id;
  }

  /* ---- stats: sort_and_group_coo_tensors_impl.h:525-570 ---- */
  int32_t req = 0, obs_max = 0, obs_max_unique = 0;
  for (int g = 0; g < P; ++g) {
    t->max_ids[g] = observed_ids[g]; t->max_unique[g] = observed_unique[g];
    req += round_up(observed_ids[g], SC_ALIGN);
    if (observed_ids[g] > obs_max) obs_max = observed_ids[g];
    if (observed_unique[g] > obs_max_unique) obs_max_unique = observed_unique[g];
  }
  *t->required = req;
  /* ValidateMaxIdsOrDie, :45-89 */
  if (!o->allow_id_dropping &&
      (obs_max > o->max_ids_per_partition || obs_max_unique > o->max_unique_ids_per_partition)) {
    t->status = SC_ID_LIMIT_EXCEEDED;
  }

  /* ---- FillBufferSegment, input_preprocessing_util.cc:167-208 with
   * ValidIndices :74-95, PadCooBuffer :120-133, AdvanceAndPadPartitions :146-162 ---- */
  const int R = P > SC_ALIGN ? P : SC_ALIGN;
  const int coo_per_sc = o->coo_buffer_size_per_device / S;
  const int coo_begin = sc * coo_per_sc, coo_end = coo_begin + coo_per_sc;
  const int lhs_begin = sc * R, lhs_end = lhs_begin + R;
  int lhs = lhs_begin, coo = coo_begin, cur = 0; size_t processed = 0;
#define VALID() (((processed == gsize) && (coo == coo_end)) ? 1 : ((lhs >= lhs_end || coo >= coo_end) ? 0 : 1))
#define ADVANCE(target)                                                        \
  while (cur < (target)) {                                                     \
    if (!VALID()) break;                                                       \
    t->row_pointers[lhs++] = coo - coo_begin;                                  \
    while (coo % SC_ALIGN != 0 && coo < coo_end) {                             \
      t->embedding_ids[coo] = INT_MAX; t->sample_ids[coo] = INT_MAX;           \
      t->gains[coo] = nanf(""); ++coo;                                         \
    }                                                                          \
    ++cur;                                                                     \
  }
  for (size_t i = 0; i < gsize; ++i) {
    const int target = grouped[i].col_id % P;
    ADVANCE(target);
    if (!VALID()) { dropped += (int64_t)(gsize - processed); break; }
    t->embedding_ids[coo] = grouped[i].col_id / P;
    t->sample_ids[coo] = grouped[i].row_id % bslice;
    t->gains[coo] = grouped[i].gain;
    ++coo; ++processed;
  }
  ADVANCE(P);
  while (lhs < lhs_end) t->row_pointers[lhs++] = coo - coo_begin; /* PadRowPointersBuffer :98-103 */
#undef ADVANCE
#undef VALID
  t->dropped = dropped;

  free(observed_ids); free(grouped); free(keys);
  free(x_row); free(x_col); free(x_gain); free(row_token_counts); free(row_gains);
}

typedef struct { sc_task_t* tasks; int ntasks; int next; pthread_mutex_t mu; } pool_t;
static void* worker(void* arg) {
  pool_t* p = (pool_t*)arg;
  for (;;) {
    pthread_mutex_lock(&p->mu);
    int i = p->next < p->ntasks ? p->next++ : -1;
    pthread_mutex_unlock(&p->mu);
    if (i < 0) break;
    run_task(&p->tasks[i]);
  }
  return NULL;
}

/* input_preprocessing_util.cc:242-312 buffer sizing (minibatching disabled).
 * Returns -1 when the suggested size exceeds the theoretical maximum (a CHECK
 * failure in the reference) or the result leaves (0, INT_MAX). */
int64_t sc_oracle_coo_buffer_size(int32_t max_ids_per_partition, int32_t global_device_count,
                                  int32_t num_sc_per_device, int64_t suggested /* <0: none */) {
  const int64_t num_scs = (int64_t)global_device_count * num_sc_per_device;
  const int64_t rounded = ((int64_t)max_ids_per_partition + SC_ALIGN - 1) / SC_ALIGN * SC_ALIGN;
  const int64_t theoretical = rounded * num_sc_per_device * num_scs;
  int64_t v = theoretical;
  if (suggested >= 0) {
    const int64_t m = (int64_t)SC_ALIGN * num_sc_per_device;
    v = (suggested + m - 1) / m * m;
    if (v > theoretical) return -1;
  }
  if (!(v > 0 && v < INT_MAX)) return -1;
  return v;
}

/* PreprocessSparseDenseMatmulInput for ONE stacked table (input_preprocessing.cc:800-959).
 * `feats` must already be ordered by row_offset (pybind_input_preprocessing.cc:114-120).
 * Output arrays are row-major [local_device_count, size]; slots the reference never
 * writes are left untouched.  Stats are [local_device_count * P] and
 * [local_device_count * S] like the flattened StatsPerHost. */
int sc_oracle_preprocess_table(const sc_oracle_feature_t* feats, int nfeat, const sc_oracle_options_t* opt,
                               int32_t* row_pointers, int32_t* embedding_ids, int32_t* sample_ids, float* gains,
                               int32_t* max_ids, int32_t* max_unique, int32_t* required, int64_t* dropped_out) {
  const int L = opt->local_device_count, C = opt->global_device_count, S = opt->num_sc_per_device;
  /* PreprocessSparseDenseMatmulInputOptions::Validate, input_preprocessing_util.cc:490-522 */
  if (L <= 0 || C <= 0 || C < L || S <= 0) return SC_INVALID_ARGUMENT;
  const int P = S * C;
  if (P & (P - 1)) return SC_INVALID_ARGUMENT;
  if (nfeat <= 0) return SC_INVALID_ARGUMENT;
  int64_t bdev = 0;
  for (int f = 0; f < nfeat; ++f) bdev += feats[f].rows / L;
  /* ValidateLocalBatchSizeLimits, input_preprocessing.cc:757-786 */
  if (bdev > (int64_t)SC_DATA_MASK) return SC_INVALID_ARGUMENT;
  /* CheckDeviceBatchSize, input_preprocessing.cc:125-131 (a CHECK in the reference) */
  if (bdev % S) return SC_INVALID_ARGUMENT;
  const int R = P > SC_ALIGN ? P : SC_ALIGN;
  const int ntasks = L * S;
  sc_task_t* tasks = (sc_task_t*)calloc((size_t)ntasks, sizeof(sc_task_t));
  int32_t* sc_max_ids = (int32_t*)calloc((size_t)ntasks * P * 2, sizeof(int32_t));
  int32_t* sc_max_unique = sc_max_ids + (size_t)ntasks * P;
  for (int d = 0; d < L; ++d)
    for (int s = 0; s < S; ++s) {
      sc_task_t* t = &tasks[d * S + s];
      t->feats = feats; t->nfeat = nfeat; t->opt = opt; t->local_device = d; t->local_sc = s;
      t->batch_size_for_device = (int32_t)bdev;
      t->row_pointers = row_pointers + (size_t)d * R * S;
      t->embedding_ids = embedding_ids + (size_t)d * opt->coo_buffer_size_per_device;
      t->sample_ids = sample_ids + (size_t)d * opt->coo_buffer_size_per_device;
      t->gains = gains + (size_t)d * opt->coo_buffer_size_per_device;
      t->max_ids = sc_max_ids + (size_t)(d * S + s) * P;
      t->max_unique = sc_max_unique + (size_t)(d * S + s) * P;
      t->required = required + (size_t)d * S + s;
    }
  int nthreads = opt->num_threads > 0 ? opt->num_threads : 1;
  if (nthreads > ntasks) nthreads = ntasks;
  pool_t pool = {tasks, ntasks, 0, PTHREAD_MUTEX_INITIALIZER};
  if (nthreads <= 1) {
    worker(&pool);
  } else {
    pthread_t* th = (pthread_t*)malloc((size_t)nthreads * sizeof(pthread_t));
    for (int i = 0; i < nthreads; ++i) pthread_create(&th[i], NULL, worker, &pool);
    for (int i = 0; i < nthreads; ++i) pthread_join(th[i], NULL);
    free(th);
  }
  /* max over local SparseCores: sort_and_group_coo_tensors_impl.h:105-113,609-621 */
  int status = SC_OK; int64_t dropped = 0;
  for (int d = 0; d < L; ++d) {
    for (int g = 0; g < P; ++g) {
      int32_t a = 0, b = 0;
      for (int s = 0; s < S; ++s) {
        int32_t x = sc_max_ids[(size_t)(d * S + s) * P + g]; if (x > a) a = x;
        int32_t y = sc_max_unique[(size_t)(d * S + s) * P + g]; if (y > b) b = y;
      }
      max_ids[(size_t)d * P + g] = a; max_unique[(size_t)d * P + g] = b;
    }
    for (int s = 0; s < S; ++s) {
      dropped += tasks[d * S + s].dropped;
      if (tasks[d * S + s].status != SC_OK) status = tasks[d * S + s].status;
    }
  }
  *dropped_out = dropped;
  free(sc_max_ids); free(tasks);
  return status;
}
