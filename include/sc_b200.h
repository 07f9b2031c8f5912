/*
 * sc_b200 - C ABI of the B200-native SparseCore embedding path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an
 * int32 status (SC_OK == 0) and never throws or aborts.  Pointers named "device"
 * are CUDA device pointers of the current device; everything else is host
 * memory.  No entry point allocates: scratch memory is a caller-owned device
 * workspace whose size comes from the matching *_workspace_bytes query.  Work is
 * enqueued on the given stream (a cudaStream_t passed as void*; NULL = default
 * stream) and is asynchronous unless stated otherwise.  The lookup / update entry points copy
 * their descriptors from host memory that does not outlive the call, so none of them may be called
 * on a stream that is being captured into a CUDA graph; such calls fail without enqueuing work.
 *
 * Each declaration cites the interface of the reference project
 * (jax-ml/jax-tpu-embedding, paths relative to jax_tpu_embedding/sparsecore/)
 * that it replaces.
 */
#ifndef SC_B200_H_
#define SC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* sc_stream_t;

enum sc_status {
  SC_OK = 0,
  SC_INVALID_ARGUMENT = 1,    /* maps to ValueError, like absl::InvalidArgument in pybind_input_preprocessing.cc:163-170 */
  SC_WORKSPACE_TOO_SMALL = 2,
  SC_ID_LIMIT_EXCEEDED = 3,   /* the reference LOG(FATAL)s: sort_and_group_coo_tensors_impl.h:61-68 */
  SC_CUDA_ERROR = 4,          /* maps to RuntimeError */
  SC_UNSUPPORTED = 5
};

enum sc_combiner { SC_COMBINER_SUM = 0, SC_COMBINER_MEAN = 1, SC_COMBINER_SQRTN = 2 };

#define SC_MAX_SHARDS 64       /* largest num_scs one call can address */
#define SC_MAX_FEATURES 1024   /* features per stacked table in one preprocessing call */
#define SC_PADDING_VALUE 2147483647 /* lib/core/constants.py:17 */

/* Library identification and the message of the last failing call on this thread. */
int32_t sc_version(void);
const char* sc_status_name(int32_t status);
int32_t sc_last_error(char* buffer, int32_t buffer_bytes);
/* Number of CUDA kernels this library has launched in the process so far. */
int64_t sc_launch_count(void);
/* Stages.  Every call brackets its stages with NVTX ranges named after the reference's trace
 * annotations (tsl::profiler::TraceMe in lib/core/input_preprocessing.cc:210-214, 413-417, 632-636:
 * "ExtractCooTensors", "SortAndGroup", "FillBuffer"; @jax.named_call in lib/nn/embedding.py:1047, 1297).
 * sc_phase_timing(1) additionally records a pair of CUDA events per stage on the call's stream and
 * clears earlier records; sc_phase_report waits for them and writes "name=total_ms/count;..." in
 * first-seen order, then clears; sc_phase_timing(0) stops recording.  Meant for benchmarks. */
int32_t sc_phase_timing(int32_t enable);
int32_t sc_phase_report(char* buffer, int32_t buffer_bytes);

/* ---------------------------------------------------------------- buffer sizing
 * Replaces ComputeCooBufferSizePerDevice / GetRowPointersSizePerDevice
 * (lib/core/input_preprocessing_util.cc:242-312, input_preprocessing_util.h:503-511;
 * Python bindings pybind_input_preprocessing.cc:218-253).  Host arithmetic only.
 * A negative result means the suggested size exceeds the theoretical maximum or
 * the size leaves (0, INT_MAX). */
int64_t sc_compute_theoretical_max_coo_buffer_size(int32_t max_ids_per_partition, int32_t global_device_count,
                                                   int32_t num_sc_per_device);
int64_t sc_compute_coo_buffer_size_per_device(int32_t max_ids_per_partition, int32_t global_device_count,
                                              int32_t num_sc_per_device, int64_t suggested_or_negative);
int32_t sc_compute_row_pointers_size_per_device(int32_t global_device_count, int32_t num_sc_per_device);

/* ---------------------------------------------------------------- preprocessing
 * Replaces PreprocessSparseDenseMatmulInput for one stacked table and one local
 * device (lib/core/input_preprocessing.h:62-68, input_preprocessing.cc:800-959):
 * extract -> sort by (SparseCore, shard, row of the shard, sample) -> dedup with
 * f32 gain sums -> optional id dropping -> stats -> CSR-wrapped COO buffers,
 * bit-exact with the reference over the region the reference writes.  The rest of
 * each buffer is filled with (SC_PADDING_VALUE, SC_PADDING_VALUE, NaN).
 *
 * The batch of the device is given as one CSR: `ids`/`weights` hold the ids of
 * all features back to back (features ordered by row_offset, rows in order) and
 * `row_offsets[total_rows + 1]` delimits the rows. */
typedef struct {
  int32_t row_begin;  /* first row of this feature inside row_offsets */
  int32_t rows;       /* rows of this feature held by the device (divisible by num_sc_per_device) */
  int32_t row_offset; /* FeatureIdTransformation.row_offset (global samples before this feature) */
  int32_t col_offset; /* row_offset_in_shard * num_scs of the feature's table */
  int32_t col_shift;  /* shard rotation of the feature's table */
  int32_t valency;    /* > 0: every row has exactly `valency` ids and row_offsets is not read for it */
  int32_t id_begin;   /* with valency > 0: index of the feature's first id inside `ids` */
} sc_feature_desc_t;

typedef struct {
  int32_t global_device_count;
  int32_t num_sc_per_device;
  int32_t combiner;                      /* enum sc_combiner */
  int32_t max_ids_per_partition;
  int32_t max_unique_ids_per_partition;
  int32_t allow_id_dropping;
  int32_t coo_buffer_size_per_device;    /* from sc_compute_coo_buffer_size_per_device */
  int32_t stack_vocab_size;              /* padded vocabulary of the stack; bounds the sort key */
} sc_preprocess_options_t;

/* Layout of the int32 stats block written on the device (P = num_scs, S = num_sc_per_device):
 * [0, P) ids per partition (max over local SparseCores), [P, 2P) unique ids per partition,
 * [2P, 2P+S) required buffer size per SparseCore, [2P+S] dropped id count,
 * [2P+S+1] status (SC_OK or SC_ID_LIMIT_EXCEEDED), [2P+S+2] ids written to the buffers. */
int32_t sc_preprocess_stats_size(int32_t global_device_count, int32_t num_sc_per_device);
size_t sc_preprocess_workspace_bytes(int64_t nnz, int64_t total_rows, const sc_preprocess_options_t* options);
int32_t sc_preprocess_table(const int32_t* ids_device, const int32_t* row_offsets_device, const float* weights_device_or_null,
                            int64_t nnz, int64_t total_rows, const sc_feature_desc_t* features_host, int32_t num_features,
                            const sc_preprocess_options_t* options, int32_t* row_pointers_device,
                            int32_t* embedding_ids_device, int32_t* sample_ids_device, float* gains_device,
                            int32_t* stats_device, void* workspace_device, size_t workspace_bytes, sc_stream_t stream);

/* Grouped variant: all stacked tables of a model (and all local devices) in one call; every
 * kernel is launched once for the whole group.  The group's sort key must fit 32 bits:
 * bits(table index) + max over tables of bits(num_sc_per_device * stack_vocab_size). */
typedef struct {
  const int32_t* ids;          /* device */
  const int32_t* row_offsets;  /* device, may be NULL when every feature has a fixed valency */
  const float* weights;        /* device or NULL */
  int64_t nnz;
  int64_t total_rows;
  const sc_feature_desc_t* features; /* host */
  int32_t num_features;
  sc_preprocess_options_t options;
  int32_t* row_pointers;       /* device outputs */
  int32_t* embedding_ids;
  int32_t* sample_ids;
  float* gains;
  int32_t* stats;
  /* Optional (both or neither, device): the forward plan of the emitted buffers, for
   * sc_fwd_item_t.plan_slots / plan_bags.  plan_slots[nnz] and plan_bags[2 * total_rows]; bag r covers
   * the activation row `SparseCore * (total_rows / num_sc_per_device) + sample`. */
  uint32_t* plan_slots;
  uint32_t* plan_bags;
} sc_preprocess_item_t;

size_t sc_preprocess_grouped_workspace_bytes(const sc_preprocess_item_t* items, int32_t count);
int32_t sc_preprocess_grouped(const sc_preprocess_item_t* items, int32_t count, void* workspace_device,
                              size_t workspace_bytes, sc_stream_t stream);

/* ---------------------------------------------------------------- lookup / update
 * One device buffer of CSR-wrapped COO input plus the geometry of the stacked table. */
typedef struct {
  const int32_t* row_pointers;   /* device, [num_sc_per_device * max(num_scs, 8)] */
  const int32_t* embedding_ids;  /* device, [coo_buffer_size] row inside the destination shard */
  const int32_t* sample_ids;     /* device, [coo_buffer_size] sample inside the source SparseCore */
  const float* gains;            /* device, [coo_buffer_size] */
  int32_t coo_buffer_size;
  int32_t num_sc_per_device;
  int32_t num_scs;
  int32_t device_batch_size;     /* samples of the stack on this device */
  int32_t dim;                   /* floats per table row */
  int32_t max_ids_per_sample;    /* 1: at most one id per sample (enables the store-only forward); 0: unknown */
  int64_t rows_per_shard;
} sc_csr_t;

/* Forward: activations[s * B/S + sample] = sum gain * shard[g][embedding_id].
 * Replaces the custom call "SparseDenseMatmulOp" behind
 * tpu_sparse_dense_matmul_csr_primitive (lib/core/primitives/sparse_dense_matmul_csr.py:114-207).
 * `shard_tables_host[g]` is the device pointer of shard g ([rows_per_shard, dim] floats). */
size_t sc_sparse_dense_matmul_fwd_workspace_bytes(const sc_csr_t* csr);
int32_t sc_sparse_dense_matmul_fwd(const sc_csr_t* csr, const float* const* shard_tables_host, float* activations_device,
                                   void* workspace_device, size_t workspace_bytes, sc_stream_t stream);

/* Backward fused with the optimizer: G[row] = sum gain * activation_grad[sample] over every
 * entry of the row, then ONE update of the row and its slot variables, in place;
 * untouched rows keep their values.  Replaces "SparseDenseMatmulGradOpWithOptimizerUpdate"
 * behind the sgd / adagrad / adam primitives (lib/core/primitives/
 * sparse_dense_matmul_grad_with_sgd.py:98-238, ..._adagrad.py:119-292, ..._adam.py:144-405).
 * clip_min / clip_max clamp the table only (primitives/utils.py:24-59); pass NaN for "no bound". */
enum {
  SC_OPT_SGD = 0,              /* hyper {learning_rate}; no slot */
  SC_OPT_ADAGRAD = 1,          /* hyper {learning_rate}; slot0 accumulator */
  SC_OPT_ADAM = 2,             /* hyper {alpha_t, beta_1, beta_2, epsilon_hat}; slots momentum, velocity */
  /* The other fused optimizers of the reference (..._adagrad_momentum.py:262-308, ..._ftrl.py:275-334,
   * ..._laprop.py:294-335, ..._f2a.py:257-285); flags travel as 0.0 / 1.0. */
  SC_OPT_ADAGRAD_MOMENTUM = 3, /* hyper {lr, momentum, beta2, epsilon, exponent, use_nesterov}; slots accumulator, momentum */
  SC_OPT_FTRL = 4,             /* hyper {lr, lr_power, l1, l2, beta, multiply_linear_by_learning_rate}; slots accumulator, linear */
  SC_OPT_LAPROP = 5,           /* hyper {lr, b1, decay_rate, eps}; slots mu, nu */
  SC_OPT_F2A = 6               /* hyper {lr, rho, l1, l2, max_lr_multiplier, global_step}; slots accumulator, local_step */
};
typedef struct {
  int32_t optimizer;      /* SC_OPT_* */
  float hyper[8];
  float clip_min, clip_max;
} sc_optimizer_t;

size_t sc_sparse_dense_matmul_grad_workspace_bytes(const sc_csr_t* csr);
int32_t sc_sparse_dense_matmul_grad(const sc_csr_t* csr, const float* activation_grad_device,
                                    float* const* shard_tables_host, float* const* shard_slot0_host,
                                    float* const* shard_slot1_host, const sc_optimizer_t* optimizer,
                                    void* workspace_device, size_t workspace_bytes, sc_stream_t stream);

/* Grouped variants: ONE launch sequence serves every stacked table of a model (the loop over
 * stacked tables in lib/nn/embedding.py:1145-1172 and :1422-1527 of the reference issues one
 * custom call per table).  All tables of a group must have row lengths in the same class
 * (dim divisible by 4 and the same number of 128-float blocks, or the same scalar class). */
typedef struct {
  sc_csr_t csr;
  const float* const* shard_tables; /* host array [num_scs] of device pointers */
  float* activations;               /* device, [device_batch_size, dim] */
  /* One process per GPU with row-sharded tables: the shard this device holds in its own memory
   * (the other shard pointers are peer mappings).  Rows of the other shards are then fetched once
   * per distinct row into the workspace and gathered from there, so a row that many samples of
   * the batch look up crosses NVLink once.  -1: read every shard pointer directly. */
  int32_t local_shard;
  /* Optional forward plan emitted by sc_preprocess_grouped for the same buffers (both or neither;
   * device pointers): plan_bags[2 * r], plan_bags[2 * r + 1] delimit, inside plan_slots, the slots of
   * activation row r in ascending order.  The reference's operator signature carries only the id-major
   * arrays, so without a plan the sample-major view is rebuilt on every call (one scatter when
   * csr.max_ids_per_sample == 1, a counting sort otherwise). */
  const uint32_t* plan_slots;
  const uint32_t* plan_bags;
} sc_fwd_item_t;

/* Buffers of one source device as seen from the owner of a shard (peer-mapped device pointers). */
typedef struct {
  const int32_t* row_pointers;
  const int32_t* embedding_ids;
  const int32_t* sample_ids;
  const float* gains;
  const float* activation_grad;
} sc_pull_source_t;

typedef struct {
  sc_csr_t csr;
  const float* activation_grad;     /* device, [device_batch_size, dim] */
  float* const* shard_tables;       /* host arrays [num_scs] of device pointers */
  float* const* shard_slot0;
  float* const* shard_slot1;
  sc_optimizer_t optimizer;
  /* Row-sharded tables with one process per GPU ("pull" mode; replaces the cross-chip exchange
   * that the TPU custom call performs implicitly, sc/docs/parameters.rst:20-24).  When `sources`
   * is not NULL this device owns shard `shard` (its table is shard_tables[0]) and reduces the
   * entries that each of the `num_sources` == num_scs devices holds for that shard, reading the
   * peers' CSR buffers and gradient rows over NVLink; `csr` then describes the geometry of ONE
   * source buffer and `partition_capacity` bounds the entries per (source, shard), normally
   * max_ids_per_partition rounded up to 8.  The caller makes every source buffer complete and
   * visible (a stream-ordered barrier across the devices) before this call. */
  const sc_pull_source_t* sources;  /* host array [num_sources] or NULL */
  int32_t num_sources;
  int32_t shard;
  int32_t partition_capacity;
} sc_grad_item_t;

size_t sc_sparse_dense_matmul_fwd_grouped_workspace_bytes(const sc_fwd_item_t* items, int32_t count);
int32_t sc_sparse_dense_matmul_fwd_grouped(const sc_fwd_item_t* items, int32_t count, void* workspace_device,
                                           size_t workspace_bytes, sc_stream_t stream);
/* Pull mode only, before the barrier across the devices: publishes what this device holds for every
 * shard in its own exchange buffers (sources[shard]).  When dim % 4 == 0 the gradient rows of all
 * entries that hit one (shard, row) are summed here first (in slot order) and the exchange carries
 * one entry and one reduced gradient row per distinct row: sources[...].activation_grad must then
 * hold coo_buffer_size rows and must not alias the CSR operands.  Otherwise the CSR buffers and
 * the activation gradients are copied unchanged (activation_grad of device_batch_size rows).
 * Follow with a barrier across the devices, then the grouped update. */
size_t sc_sparse_dense_matmul_grad_stage_workspace_bytes(const sc_grad_item_t* items, int32_t count);
int32_t sc_sparse_dense_matmul_grad_stage(const sc_grad_item_t* items, int32_t count, void* workspace_device,
                                          size_t workspace_bytes, sc_stream_t stream);
size_t sc_sparse_dense_matmul_grad_grouped_workspace_bytes(const sc_grad_item_t* items, int32_t count);
int32_t sc_sparse_dense_matmul_grad_grouped(const sc_grad_item_t* items, int32_t count, void* workspace_device,
                                            size_t workspace_bytes, sc_stream_t stream);

/* ---------------------------------------------------------------- peer-visible memory
 * Row-sharded tables with one process per GPU: every process allocates its table shards and its
 * exchange buffers with sc_peer_alloc, exports a 64-byte CUDA IPC handle and imports the handles
 * of its peers (exchanged by the host program); the kernels then read remote memory with plain
 * loads over NVLink.  Replaces the implicit cross-chip addressing of the TPU custom calls
 * (sc/docs/parameters.rst:20-24).  These are the only entry points that allocate. */
int32_t sc_peer_alloc(size_t bytes, void** device_pointer_out);
int32_t sc_peer_free(void* device_pointer);
int32_t sc_ipc_export(void* device_pointer, char* handle64_out);
int32_t sc_ipc_import(const char* handle64, void** peer_pointer_out);
int32_t sc_ipc_release(void* peer_pointer);

/* Fused backward + optimizer update for callers that cannot allocate device memory at all:
 * an embedding server whose device memory was carved up completely at start-up, a plugin invoked
 * from inside another runtime's execution callback where cudaMalloc is forbidden, or a
 * latency-critical loop that must never wait on the driver's allocator lock - places where even
 * asking a framework for a workspace tensor may end in cudaMalloc.  (No counterpart in the
 * reference project: there the XLA runtime owns all buffers.)
 *
 * Same arithmetic and kernels as sc_sparse_dense_matmul_grad, but the scratch lives in a
 * SC_STATIC_SCRATCH_BYTES array built into the library image, so the call performs no
 * cudaMalloc / cudaFree and takes no workspace.  Limits: one shard and one SparseCore per buffer
 * (num_scs == num_sc_per_device == 1) and
 *   768 + chunks * (8 * dim + 1) + ceil(chunks / 32) * (4 * dim + 1)  <=  SC_STATIC_SCRATCH_BYTES
 * with chunks = ceil(coo_buffer_size / 32),
 * e.g. 65536 slots at dim 128; larger inputs are rejected with SC_WORKSPACE_TOO_SMALL.
 * The first call on each device resolves the address of the array (cudaGetSymbolAddress); make
 * that first call before any stream capture begins (a call on a capturing stream is rejected with
 * SC_UNSUPPORTED).  All calls on a device share the one array:
 * the call overwrites every scratch word it later reads, so nothing needs clearing, but two
 * calls that overlap on the GPU (different streams) race and must be serialised by the caller. */
#define SC_STATIC_SCRATCH_BYTES (2 * 1024 * 1024 + 64 * 1024)
int32_t sc_sparse_dense_matmul_grad_static(const sc_csr_t* csr, const float* activation_grad_device,
                                           float* const* shard_tables_host, float* const* shard_slot0_host,
                                           float* const* shard_slot1_host, const sc_optimizer_t* optimizer,
                                           sc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SC_B200_H_ */
