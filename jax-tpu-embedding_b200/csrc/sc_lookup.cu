// Forward gather-combine and backward segment-reduce fused with SGD / Adagrad / Adam.
//
// Data layout in HBM
//   * table shards: float32 [rows_per_shard, dim] row-major, one pointer per shard;
//   * CSR-wrapped COO input of one device: row_pointers / embedding_ids / sample_ids /
//     gains exactly as the reference's preprocessing emits them (id-major: ordered by
//     source SparseCore, destination shard, row of the shard, sample);
//   * activations and activation gradients: float32 [device_batch, dim].
//
// Every kernel works on a GROUP of stacked tables described by an array of TableDesc in
// device memory, so that one launch serves all tables of a model (26 tables of 65536
// single-hot lookups would otherwise be 26 launches of a few microseconds each).
//
// Forward: the COO is id-major, the output is per sample.  The valid slots of all tables
// are stably radix-sorted by global activation row; a warp then owns 32 consecutive
// activation rows, resolves their first entries lane-parallel and sums gain * table_row
// per row in slot order (ascending shard, row).  The result does not depend on scheduling
// and every activation row is written exactly once (no memset, no atomics).
//
// Backward: every table row is a contiguous run of the id-major entry list.  A warp owns
// 32 consecutive entries, finds the runs with one ballot, reduces each run in entry order
// and applies the optimizer with a single read-modify-write of the row and its slot
// variables.  Runs that cross a 32-entry boundary leave per-chunk partial sums in scratch;
// a second kernel adds them in chunk order and applies the update once.  No floating-point
// atomics anywhere: results are bitwise reproducible.
//
// All arithmetic is float32 with separately rounded multiply and add (the file is
// compiled with -fmad=false) so that sequential sums match a float32 CPU loop.
#include <math.h>

#include <mutex>
#include <vector>

#include "sc_common.cuh"
#include <stdlib.h>
#include <string.h>

#include "sc_sort.cuh"

namespace sc {
namespace {

constexpr int kBlock = 256;
constexpr int kWarpsPerBlock = kBlock / 32;
constexpr uint32_t kNoRow = 0xffffffffu;
constexpr int kReduceOnly = 100;  // OptParams::kind of the reduce-only mode
// Slot variables of an optimizer kind.
inline int optimizer_slots(int kind) { return kind == SC_OPT_SGD ? 0 : kind == SC_OPT_ADAGRAD ? 1 : 2; }

struct CsrView {
  const int32_t* row_pointers;
  const int32_t* ids;
  const int32_t* sids;
  const float* gains;
  int32_t coo;         // slots per device buffer
  int32_t coo_per_sc;  // slots per SparseCore slice
  int32_t S, P, R;     // SparseCores per device, shards, row pointers per SparseCore
  int32_t bdev, bsc;   // samples per device / per SparseCore
  int32_t dim;
  int64_t rows_per_shard;
};

struct OptParams {
  int kind;   // SC_OPT_* of sc_b200.h, or kReduceOnly
  int slots;  // slot variables the update reads and writes: 0, 1 or 2
  float h0, h1, h2, h3, h4, h5;
  float lo, hi;  // NaN = unbounded
};

// Buffers of one source device as seen from the owner of a shard (peer-mapped pointers).
struct PullSrc {
  const int32_t* row_pointers;
  const int32_t* ids;
  const int32_t* sids;
  const float* gains;
  const float* grad;
};

// One stacked table of a grouped launch.
struct TableDesc {
  CsrView v;
  float* const* table;  // device array of P shard pointers
  float* const* slot0;
  float* const* slot1;
  float* act;           // forward output [bdev, dim]
  const float* grad;    // backward input [bdev, dim]
  OptParams opt;
  uint32_t slot_base;   // first global slot of this table
  uint32_t act_base;    // first global activation row
  uint32_t chunk_base;  // first global 32-entry chunk (backward)
  // Backward entry list: direct (entry e = slot e, row = ids[e]) for one SparseCore and one
  // shard; otherwise entries sorted by global row (rows[e]) with their source slot (slots[e]).
  // All indirect tables of a call share ONE sorted list: rows[] holds row_base + global row,
  // slots[] holds ent_base + entry index, and range[0..1] delimits this table's part of the list.
  const uint32_t* rows;
  const uint32_t* slots;
  const uint32_t* range;
  uint32_t row_base;
  uint32_t ent_base;
  uint32_t n_ent;       // size of this table's entry index space (0 for direct tables)
  int32_t indirect;
  uint32_t total_rows;  // P * rows_per_shard
  // Pull mode (row-sharded tables, one process per GPU): this device owns shard `pull_shard` and
  // reduces the entries that EVERY device holds for that shard, reading them and the gradient
  // rows from the peers' memory.  Entry index = source * pull_cap + position inside the partition.
  const PullSrc* pull;
  int32_t* pull_begin;  // first slot of the shard's partition in every source buffer
  int32_t pull_cap;
  int32_t pull_shard;
  int32_t num_sources;
  int32_t pull_rows;    // rows of a source's gradient buffer (samples, or slots when it holds reduced runs)
  uint32_t tile_base;   // merge of the sources' partitions: first compaction tile of this table ...
  uint32_t tiles_per_list;  // ... and tiles per (table, source) partition
  // Reduce-only mode (opt.kind == kReduceOnly, indirect == 2): the entry list is this device's own
  // CSR buffer (entry e = slot e, rows[e] = shard * rows_per_shard + id or kNoRow) and the sum of
  // every run is stored at red[first slot of the run] instead of being applied to a table.
  float* red;
  // Forward with remote shards (one process per GPU): rows of every shard but `local_shard` are
  // first copied, once per run of equal ids, into `remote_rows`; run_ord[global slot] is the row's
  // index there.  local_shard < 0: every shard pointer is read directly.
  int32_t local_shard;
  const uint32_t* run_ord;
  float* remote_rows;
  // Forward plan: bags[2 * r] .. bags[2 * r + 1] delimit the entries of local activation row r inside
  // `plan`, whose values minus plan_bias are slots of this table's buffer in ascending order
  // (plan == nullptr: the position itself is the value).
  const uint32_t* plan;
  const uint32_t* bags;
  uint32_t plan_bias;
};

// Index of the table whose [base, next base) range contains x.
template <typename F>
__device__ __forceinline__ int find_table(int count, uint32_t x, F base_of) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (base_of(mid) <= x) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Same result as find_table for an ascending base_of, computed by the whole warp with one load
// per lane (all 32 lanes must call it).
template <typename F>
__device__ __forceinline__ int warp_find_table(int count, uint32_t x, int lane, F base_of) {
  int t = -1;
  for (int base = 0; base < count; base += 32) {
    const int i = base + lane;
    const uint32_t below = __ballot_sync(0xffffffffu, i < count && base_of(i) <= x);
    t += __popc(below);
    if (below != 0xffffffffu) break;
  }
  return t;
}

// Destination shard of slot `local` (relative to its SparseCore slice), or -1 for
// alignment padding / the unwritten tail.  Shard g owns [round_up(rp[g-1], 8), rp[g]).
__device__ __forceinline__ int slot_shard(const CsrView& v, int s, int local) {
  const int32_t* rp = v.row_pointers + s * v.R;
  if (local >= rp[v.P - 1]) return -1;
  int lo = 0, hi = v.P - 1;  // first g with rp[g] > local
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (rp[mid] > local) hi = mid; else lo = mid + 1;
  }
  const int begin = lo == 0 ? 0 : ((rp[lo - 1] + kAlign - 1) & ~(kAlign - 1));
  return local >= begin ? lo : -1;
}

// Like slot_shard, also returning the first slot of the partition.
__device__ __forceinline__ int slot_shard_begin(const CsrView& v, int s, int local, int* begin_out) {
  const int32_t* rp = v.row_pointers + s * v.R;
  if (local >= rp[v.P - 1]) return -1;
  int lo = 0, hi = v.P - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (rp[mid] > local) hi = mid; else lo = mid + 1;
  }
  const int begin = lo == 0 ? 0 : ((rp[lo - 1] + kAlign - 1) & ~(kAlign - 1));
  *begin_out = begin;
  return local >= begin ? lo : -1;
}

// ------------------------------------------------------------------------ forward

// The forward plan lists, for every activation row, the slots that feed it, in ascending slot
// order (the order of the reference's sum).  It is a counting sort by activation row:
//   1. fwd_count_kernel    key[slot] = activation row, rank[slot] = arrival number in that row
//   2. exclusive scan      offsets[row] = first list position of the row
//   3. fwd_place_kernel    list[offsets[key] + rank] = slot
//   4. fwd_rowsort_kernel  arrival order is arbitrary: put each row's slots in ascending order
//      (insertion sort by one thread for short rows, fwd_bigrow_kernel for the others)
// Slots are unique, so the sorted lists do not depend on the arrival order.

// key = global activation row of the slot (total_act for slots that hold no entry).
__global__ void fwd_count_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_slots, uint32_t total_act,
                                 uint32_t* __restrict__ keys, uint32_t* __restrict__ ranks, uint32_t* __restrict__ counts) {
  const uint32_t gq = blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= total_slots) return;
  const int t = find_table(count, gq, [&](int i) { return tabs[i].slot_base; });
  const CsrView& v = tabs[t].v;
  const int q = (int)(gq - tabs[t].slot_base);
  const int s = v.S == 1 ? 0 : q / v.coo_per_sc;
  const int local = q - s * v.coo_per_sc;
  uint32_t key = total_act;
  if (slot_shard(v, s, local) >= 0) {
    const int sid = v.sids[q];
    if (sid >= 0 && sid < v.bsc) key = tabs[t].act_base + (uint32_t)(s * v.bsc + sid);
  }
  keys[gq] = key;
  if (key < total_act) ranks[gq] = atomicAdd(&counts[key], 1u);
}

__global__ void fwd_place_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ ranks,
                                 const uint32_t* __restrict__ offsets, uint32_t total_slots, uint32_t total_act,
                                 uint32_t* __restrict__ list) {
  const uint32_t gq = blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= total_slots) return;
  const uint32_t key = keys[gq];
  if (key < total_act) list[offsets[key] + ranks[gq]] = gq;
}

constexpr uint32_t kSerialSortLimit = 64;

// Thread per activation row.  Rows longer than kSerialSortLimit go to big_rows.  With `bags` the
// row's (begin, end) pair is stored there as well.
__global__ void fwd_rowsort_kernel(const uint32_t* __restrict__ offsets, uint32_t total_act, uint32_t* __restrict__ list,
                                   uint32_t* __restrict__ big_rows, uint32_t* __restrict__ big_count,
                                   uint32_t* __restrict__ bags) {
  const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= total_act) return;
  const uint32_t begin = offsets[r], n = offsets[r + 1] - begin;
  if (bags != nullptr) { bags[2 * r] = begin; bags[2 * r + 1] = begin + n; }
  if (n < 2) return;
  if (n > kSerialSortLimit) {
    big_rows[atomicAdd(big_count, 1u)] = r;
    return;
  }
  uint32_t* a = list + begin;
  for (uint32_t i = 1; i < n; ++i) {  // arrival order is close to slot order: few moves
    const uint32_t x = a[i];
    uint32_t j = i;
    while (j > 0 && a[j - 1] > x) { a[j] = a[j - 1]; --j; }
    a[j] = x;
  }
}

// Warp per long row (grid-stride over big_rows): stable LSD radix sort of the row's slots, 8 bits
// per pass, between `list` and `scratch`.  Row r spans [offsets[r * stride], offsets[r * stride + 1]):
// stride 1 for an offsets array, 2 for (begin, end) pairs.
__global__ void __launch_bounds__(kBlock) fwd_bigrow_kernel(const uint32_t* __restrict__ offsets, uint32_t* __restrict__ list,
                                                            uint32_t* __restrict__ scratch, const uint32_t* __restrict__ big_rows,
                                                            const uint32_t* __restrict__ big_count, int key_bits, int stride) {
  __shared__ uint32_t bins[kWarpsPerBlock][256];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const uint32_t warps = gridDim.x * kWarpsPerBlock;
  const uint32_t lt = (1u << lane) - 1u;
  const uint32_t todo = *big_count;
  for (uint32_t w = blockIdx.x * kWarpsPerBlock + wib; w < todo; w += warps) {
    const uint32_t r = big_rows[w];
    const uint32_t begin = offsets[(size_t)r * stride], n = offsets[(size_t)r * stride + 1] - begin;
    uint32_t* src = list + begin;
    uint32_t* dst = scratch + begin;
    for (int shift = 0; shift < key_bits; shift += 8) {
      for (int i = lane; i < 256; i += 32) bins[wib][i] = 0;
      __syncwarp();
      for (uint32_t i = lane; i < n; i += 32) atomicAdd(&bins[wib][(src[i] >> shift) & 255u], 1u);
      __syncwarp();
      {  // exclusive scan of the 256 bins: 8 per lane
        uint32_t local[8], sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { local[i] = sum; sum += bins[wib][lane * 8 + i]; }
        uint32_t inc = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const uint32_t o = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += o;
        }
        const uint32_t base = inc - sum;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) bins[wib][lane * 8 + i] = base + local[i];
      }
      __syncwarp();
      for (uint32_t i0 = 0; i0 < n; i0 += 32) {  // 32 consecutive elements per step keeps the order stable
        const uint32_t i = i0 + lane;
        const bool in = i < n;
        const uint32_t x = in ? src[i] : 0u;
        const uint32_t d = (x >> shift) & 255u;
        const uint32_t peers = __match_any_sync(0xffffffffu, in ? d : (0x100u | (uint32_t)lane));
        const uint32_t pos = in ? bins[wib][d] + __popc(peers & lt) : 0u;
        __syncwarp();
        if (in && (peers & lt) == 0) bins[wib][d] += __popc(peers);
        if (in) dst[pos] = x;
        __syncwarp();
      }
      uint32_t* tmp = src; src = dst; dst = tmp;
    }
    if (src != list + begin) {  // odd number of passes: copy back
      __syncwarp();
      for (uint32_t i = lane; i < n; i += 32) dst[i] = src[i];
    }
    __syncwarp();
  }
}

template <int W>
struct Vec;
template <>
struct Vec<4> {
  using T = float4;
  static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ void axpy(T& a, float g, const T& x) {
    a.x = a.x + g * x.x; a.y = a.y + g * x.y; a.z = a.z + g * x.z; a.w = a.w + g * x.w;
  }
  static __device__ __forceinline__ void add(T& a, const T& x) { a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w; }
};
template <>
struct Vec<1> {
  using T = float;
  static __device__ __forceinline__ T zero() { return 0.f; }
  static __device__ __forceinline__ void axpy(T& a, float g, const T& x) { a = a + g * x; }
  static __device__ __forceinline__ void add(T& a, const T& x) { a += x; }
};

// flags[slot] = 1 where the slot starts a run of equal ids inside a partition of a REMOTE shard.
// Entries of a partition are ordered by id, so a run is all lookups of one remote row.
// The kernels of the remote-row fetch work on the slots [first, first + total_slots) of the tables `tabs`
// (a part of the call's tables); flags, before and run_ord are indexed by global slot.
__global__ void fwd_remote_heads_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t first, uint32_t total_slots,
                                        uint32_t* __restrict__ flags) {
  const uint32_t gq = first + blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= first + total_slots) return;
  const int t = find_table(count, gq, [&](int i) { return tabs[i].slot_base; });
  const TableDesc& td = tabs[t];
  const CsrView& v = td.v;
  uint32_t head = 0;
  if (td.local_shard >= 0) {
    const int q = (int)(gq - td.slot_base);
    const int s = v.S == 1 ? 0 : q / v.coo_per_sc;
    const int local = q - s * v.coo_per_sc;
    int begin;
    const int g = slot_shard_begin(v, s, local, &begin);
    if (g >= 0 && g != td.local_shard) head = (local == begin || v.ids[q - 1] != v.ids[q]) ? 1u : 0u;
  }
  flags[gq] = head;
}

// One distinct remote row to fetch.
struct FetchJob {
  const float* src;  // row in the (peer-mapped) shard
  float* dst;        // its place in remote_rows
  int32_t floats;
  int32_t pad;
};

// `before` = exclusive scan of the head flags.  Thread per slot: writes run_ord for every slot of
// a remote partition and, for run heads, the fetch job of the run's row.
__global__ void fwd_fetch_plan_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t first, uint32_t total_slots,
                                      const uint32_t* __restrict__ before, uint32_t* __restrict__ run_ord,
                                      FetchJob* __restrict__ jobs) {
  const uint32_t gq = first + blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= first + total_slots) return;
  const int t = find_table(count, gq, [&](int i) { return tabs[i].slot_base; });
  const TableDesc& td = tabs[t];
  const CsrView& v = td.v;
  if (td.local_shard < 0) return;
  const int q = (int)(gq - td.slot_base);
  const int s = v.S == 1 ? 0 : q / v.coo_per_sc;
  const int local = q - s * v.coo_per_sc;
  int begin;
  const int g = slot_shard_begin(v, s, local, &begin);
  if (g < 0 || g == td.local_shard) return;
  const int id = v.ids[q];
  const bool head = local == begin || v.ids[q - 1] != id;
  const uint32_t job = before[gq] + (head ? 1u : 0u) - 1u;  // index among all runs of the launch
  const uint32_t ord = job - before[td.slot_base];           // index among the runs of this table
  run_ord[gq] = ord;
  if (head) {
    FetchJob j;
    const bool ok = id >= 0 && (int64_t)id < v.rows_per_shard;
    j.src = ok ? td.table[g] + (int64_t)id * v.dim : nullptr;
    j.dst = td.remote_rows + (int64_t)ord * v.dim;
    j.floats = v.dim;
    j.pad = 0;
    jobs[job] = j;
  }
}

// Copies the rows of the fetch jobs.  A warp takes 8 consecutive jobs; the whole warp reads one
// row with 16 bytes per lane (one 512-byte request for a 128-float row) and issues the loads of
// all 8 rows before its first store.  total_jobs lives in device memory (the scan's total).
__global__ void __launch_bounds__(kBlock) fwd_fetch_kernel(const FetchJob* __restrict__ jobs, const uint32_t* __restrict__ total_jobs,
                                                           uint32_t max_jobs) {
  constexpr int kRows = 8;
  const int lane = threadIdx.x & 31;
  const uint32_t n = min(*total_jobs, max_jobs);
  const uint32_t warps = gridDim.x * kWarpsPerBlock;
  for (uint32_t j0 = (blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5)) * kRows; j0 < n; j0 += warps * kRows) {
    // Lane r < kRows reads job j0 + r; the fields are then broadcast.
    FetchJob mine;
    mine.src = nullptr; mine.dst = nullptr; mine.floats = 0; mine.pad = 0;
    if (lane < kRows && j0 + lane < n) mine = jobs[j0 + lane];
    const bool fast = __all_sync(0xffffffffu, mine.src == nullptr ||
                                                  ((mine.floats & 3) == 0 && mine.floats <= 128 &&
                                                   ((reinterpret_cast<uintptr_t>(mine.src) | reinterpret_cast<uintptr_t>(mine.dst)) & 15u) == 0));
    if (fast) {
      float4 x[kRows];
      bool on[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const float4* s4 = reinterpret_cast<const float4*>(__shfl_sync(0xffffffffu, (unsigned long long)mine.src, r));
        const int nv = __shfl_sync(0xffffffffu, mine.floats, r) >> 2;
        on[r] = s4 != nullptr && lane < nv;
        if (on[r]) x[r] = s4[lane];
      }
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        float4* d4 = reinterpret_cast<float4*>(__shfl_sync(0xffffffffu, (unsigned long long)mine.dst, r));
        if (on[r]) d4[lane] = x[r];
      }
    } else {
      for (int r = 0; r < kRows; ++r) {
        const float* rs = reinterpret_cast<const float*>(__shfl_sync(0xffffffffu, (unsigned long long)mine.src, r));
        float* rd = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, (unsigned long long)mine.dst, r));
        const int nf = __shfl_sync(0xffffffffu, mine.floats, r);
        if (rs == nullptr) continue;
        for (int c = lane; c < nf; c += 32) rd[c] = rs[c];
      }
    }
  }
}

// Resolves position `pos` of table `td`'s forward plan: the table row to read (in its shard, or
// its staged copy when the shard is remote; nullptr when the entry contributes nothing) and the gain.
__device__ __forceinline__ const float* resolve_entry(const TableDesc& td, uint32_t pos, float* gain) {
  const CsrView& v = td.v;
  const int q = (int)((td.plan != nullptr ? td.plan[pos] : pos) - td.plan_bias);
  int g = 0;
  if (v.P > 1) {
    const int s = q / v.coo_per_sc;
    g = slot_shard(v, s, q - s * v.coo_per_sc);
  }
  const int id = v.ids[q];
  *gain = v.gains[q];
  if (g < 0 || id < 0 || (int64_t)id >= v.rows_per_shard) return nullptr;
  if (td.local_shard >= 0 && g != td.local_shard) return td.remote_rows + (int64_t)td.run_ord[td.slot_base + (uint32_t)q] * v.dim;
  return td.table[g] + (int64_t)id * v.dim;
}

// Single-valent inputs (at most one entry per activation row): the plan is the identity and a bag
// is (slot, slot + 1), stored with one 8-byte write.  `bags` must be zero beforehand.
__global__ void fwd_single_bags_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_slots,
                                       uint2* __restrict__ bags) {
  const uint32_t gq = blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= total_slots) return;
  const int t = find_table(count, gq, [&](int i) { return tabs[i].slot_base; });
  const CsrView& v = tabs[t].v;
  const int q = (int)(gq - tabs[t].slot_base);
  const int s = v.S == 1 ? 0 : q / v.coo_per_sc;
  if (slot_shard(v, s, q - s * v.coo_per_sc) < 0) return;
  const int sid = v.sids[q];
  if (sid >= 0 && sid < v.bsc) bags[tabs[t].act_base + (uint32_t)(s * v.bsc + sid)] = make_uint2(gq, gq + 1u);
}

// Asks L2 for the `bytes` of a table row that a later instruction of this warp will load.  The
// request holds no register, so a lane can have the rows of many entries on their way while the
// warp is still summing earlier ones.
__device__ __forceinline__ void prefetch_row(const float* row, int bytes) {
  const char* p = reinterpret_cast<const char*>(row);
  for (int off = 0; off < bytes; off += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off));
}

// What a forward warp knows about one of its 32 activation rows.
struct RowMeta {
  const float* src;  // table row of the first entry, nullptr if it contributes nothing
  uint32_t begin, end;
  int32_t table;
  float gain;
};

// One warp per 32 consecutive global activation rows.  Lane l first reads the bag of row r0 + l,
// resolves its first entry and asks L2 for that table row, so the dependent index loads of 32 rows
// overlap and their rows are on their way before the first sum starts.  The warp is then split
// into 32 / G groups of G lanes; a group owns every (32 / G)-th row and covers one table row with
// K vectors of width W per lane.  The lanes of a group resolve G entries of the bag at a time -
// the next G (with an L2 prefetch of their rows) while these are summed - and the table rows of U
// entries are loaded before the first of them is added, in bag order.  Every activation row is
// written exactly once; the sum runs in ascending slot order.
// Rows of up to 64 floats (K <= 2): 4 blocks per SM and U = 4 / 2 rows in registers; measured against 3 blocks and
// U = 8 / 4 on the multi-hot benchmark configurations: 0.118 ms instead of 0.181 ms (dim 64, bags of ~20) and 0.94 ms
// instead of 1.11 ms (dim 32, bags of ~8.5).  Longer rows keep 3 blocks (4 were 12 % slower at dim 128).
#ifndef SC_GATHER_ROWS_SHORT
#define SC_GATHER_ROWS_SHORT 4
#endif
template <int W, int K, int G>
__global__ void __launch_bounds__(kBlock, K >= 8 ? 1 : K <= 2 ? 4 : 3) fwd_gather_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t first_act,
    uint32_t total_act, int rows_per_warp) {
  using VT = typename Vec<W>::T;
  constexpr int NG = 32 / G;
  constexpr int U = K >= 4 ? 2 : SC_GATHER_ROWS_SHORT / K;  // table rows held in registers per group
  __shared__ RowMeta s_meta[kWarpsPerBlock][32];
  __shared__ uint8_t s_order[kWarpsPerBlock][32];  // rows of the warp by descending bag length
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  // Rows [first_act, total_act) of `tabs`, rows_per_warp (a multiple of 32 / G, at most 32) to a warp.
  const uint32_t r0 = first_act + (blockIdx.x * kWarpsPerBlock + wib) * (uint32_t)rows_per_warp;
  if (r0 >= total_act) return;
  {
    RowMeta m;
    m.src = nullptr; m.begin = m.end = 0; m.table = 0; m.gain = 0.f;
    const uint32_t my_r = r0 + lane;
    if (lane < rows_per_warp && my_r < total_act) {
      m.table = find_table(count, my_r, [&](int i) { return tabs[i].act_base; });
      const TableDesc& td = tabs[m.table];
      const uint2 bag = reinterpret_cast<const uint2*>(td.bags)[my_r - td.act_base];
      m.begin = bag.x;
      m.end = bag.y;
      if (m.end > m.begin) {
        m.src = resolve_entry(td, m.begin, &m.gain);
        if (m.src != nullptr) prefetch_row(m.src, td.v.dim * 4);
      }
    }
    s_meta[wib][lane] = m;
    if (NG > 1) {
      // The groups of a warp walk their bags side by side and share the warp's instruction stream, so rows of
      // different lengths make them diverge.  Rows are therefore taken in order of descending bag length: the NG rows
      // of a turn have neighbouring lengths.  (Every row is summed by one group in bag order whatever the turn is,
      // so the result does not depend on this order.)
      const uint32_t len = m.end - m.begin;
      int rank = 0;
#pragma unroll 8
      for (int i = 0; i < 32; ++i) {
        const uint32_t other = __shfl_sync(0xffffffffu, len, i);
        rank += (other > len || (other == len && i < lane)) ? 1 : 0;
      }
      s_order[wib][rank] = (uint8_t)lane;
    }
  }
  __syncwarp();
  const int group = lane / G, gl = lane % G;
  const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (group * G));
  const int rows_here = (int)min((uint32_t)rows_per_warp, total_act - r0);
  int cached_t = -1, dim = 0, vec_per_row = 0;
  float* act = nullptr;
  uint32_t act_base = 0;
  for (int turn = group; turn < 32; turn += NG) {
    const int j = NG > 1 ? (int)s_order[wib][turn] : turn;
    if (j >= rows_here) break;  // lanes past the warp's rows have empty bags and sort after every row of the warp
    const RowMeta m = s_meta[wib][j];
    if (m.table != cached_t) {
      const TableDesc& td = tabs[m.table];
      dim = td.v.dim;
      vec_per_row = dim / W;
      act = td.act;
      act_base = td.act_base;
      cached_t = m.table;
    }
    VT acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[k] = Vec<W>::zero();
    if (m.end - m.begin == 1u) {
      if (m.src != nullptr) {
        const VT* src = reinterpret_cast<const VT*>(m.src);
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const int c = gl + k * G;
          if (c < vec_per_row) Vec<W>::axpy(acc[k], m.gain, __ldg(src + c));
        }
      }
    } else if (m.end > m.begin) {
      const TableDesc& td = tabs[m.table];
      uint32_t base = m.begin;
      const float* c_ptr = nullptr;
      float c_gain = 0.f;
      if (gl == 0) { c_ptr = m.src; c_gain = m.gain; }
      else if (base + gl < m.end) {
        c_ptr = resolve_entry(td, base + gl, &c_gain);
        if (c_ptr != nullptr) prefetch_row(c_ptr, dim * 4);
      }
      for (;;) {
        const uint32_t nbase = base + G;
        const float* n_ptr = nullptr;
        float n_gain = 0.f;
        if (nbase + gl < m.end) {
          n_ptr = resolve_entry(td, nbase + gl, &n_gain);
          if (n_ptr != nullptr) prefetch_row(n_ptr, dim * 4);
        }
        const int cnt = (int)min((uint32_t)G, m.end - base);
        for (int i0 = 0; i0 < cnt; i0 += U) {
          VT x[U][K];
          float gn[U];
          bool on[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int idx = i0 + u;
            const VT* src = reinterpret_cast<const VT*>(__shfl_sync(gmask, (unsigned long long)c_ptr, idx, G));
            gn[u] = __shfl_sync(gmask, c_gain, idx, G);
            on[u] = idx < cnt && src != nullptr;
#pragma unroll
            for (int k = 0; k < K; ++k) {
              const int c = gl + k * G;
              if (on[u] && c < vec_per_row) x[u][k] = __ldg(src + c);
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (!on[u]) continue;
#pragma unroll
            for (int k = 0; k < K; ++k) {
              const int c = gl + k * G;
              if (c < vec_per_row) Vec<W>::axpy(acc[k], gn[u], x[u][k]);
            }
          }
        }
        if (nbase >= m.end) break;
        base = nbase;
        c_ptr = n_ptr;
        c_gain = n_gain;
      }
    }
    VT* dst = reinterpret_cast<VT*>(act + (int64_t)(r0 + j - act_base) * dim);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = gl + k * G;
      if (c < vec_per_row) dst[c] = acc[k];
    }
  }
}

// Gather for bags of at most one entry (single-valent features): no entry walk, so the kernel needs
// few registers and more warps fit an SM.  Same warp / group layout as fwd_gather_kernel; a group
// keeps the table rows of two of its activation rows in flight.  Rows without an entry are zeroed.
template <int W, int K, int G>
__global__ void __launch_bounds__(kBlock) fwd_gather_single_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t first_act,
    uint32_t total_act) {
  using VT = typename Vec<W>::T;
  constexpr int NG = 32 / G;
  struct Meta {
    const float* src;
    float* dst;
    float gain;
    int32_t vec_per_row;
  };
  __shared__ Meta s_meta[kWarpsPerBlock][32];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const uint32_t r0 = first_act + (blockIdx.x * kWarpsPerBlock + wib) * 32u;  // rows [first_act, total_act) of `tabs`
  if (r0 >= total_act) return;
  {
    Meta m;
    m.src = nullptr; m.dst = nullptr; m.gain = 0.f; m.vec_per_row = 0;
    const uint32_t my_r = r0 + lane;
    if (my_r < total_act) {
      const int t = find_table(count, my_r, [&](int i) { return tabs[i].act_base; });
      const TableDesc& td = tabs[t];
      const uint32_t lr = my_r - td.act_base;
      const uint2 bag = reinterpret_cast<const uint2*>(td.bags)[lr];
      m.dst = td.act + (int64_t)lr * td.v.dim;
      m.vec_per_row = td.v.dim / W;
      if (bag.y > bag.x) {
        m.src = resolve_entry(td, bag.x, &m.gain);
        if (m.src != nullptr) prefetch_row(m.src, td.v.dim * 4);
      }
    }
    s_meta[wib][lane] = m;
  }
  __syncwarp();
  const int group = lane / G, gl = lane % G;
  const int rows_here = (int)min(32u, total_act - r0);
  for (int j = group; j < rows_here; j += 2 * NG) {
    const Meta a = s_meta[wib][j];
    const bool two = j + NG < rows_here;
    Meta b = a;
    if (two) b = s_meta[wib][j + NG];
    VT xa[K], xb[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = gl + k * G;
      xa[k] = (a.src != nullptr && c < a.vec_per_row) ? __ldg(reinterpret_cast<const VT*>(a.src) + c) : Vec<W>::zero();
      xb[k] = (two && b.src != nullptr && c < b.vec_per_row) ? __ldg(reinterpret_cast<const VT*>(b.src) + c) : Vec<W>::zero();
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = gl + k * G;
      VT ya = Vec<W>::zero(), yb = Vec<W>::zero();
      Vec<W>::axpy(ya, a.gain, xa[k]);
      Vec<W>::axpy(yb, b.gain, xb[k]);
      if (c < a.vec_per_row) reinterpret_cast<VT*>(a.dst)[c] = ya;
      if (two && c < b.vec_per_row) reinterpret_cast<VT*>(b.dst)[c] = yb;
    }
  }
}

// ---- cp.async pipeline variant of the gather

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(__cvta_generic_to_global(src)) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

constexpr int kFwdBlock = 128;
constexpr int kFwdWarps = kFwdBlock / 32;
constexpr int kFwdTile = 32;  // steps whose entries are resolved at a time
// Steps held in a warp's ring for K 16-byte vectors per lane (8 KiB, 16 KiB for the longest rows).
__host__ __device__ constexpr int fwd_ring_steps(int K) { return K <= 1 ? 16 : K == 2 ? 8 : 4; }
__host__ __device__ constexpr size_t fwd_ring_warp_bytes(int K, int NG) {
  return (size_t)fwd_ring_steps(K) * K * 512 + (size_t)2 * NG * kFwdTile * 16 + 32 * 24;
}

// One resolved entry of a consumer group's list.
struct FwdEntry {
  const float* src;  // table row (or its staged copy)
  float gain;
  uint32_t meta;     // bits 0..4: row of the warp that the entry belongs to; kEnt* flags
};
constexpr uint32_t kEntEnds = 0x80000000u;  // last entry of its activation row: store the sum
constexpr uint32_t kEntSkip = 0x40000000u;  // contributes nothing

// Forward for rows of `dim` floats with dim % 4 == 0 and 16-byte aligned tables and activations.
// A warp owns 32 consecutive global activation rows.  It is split into NG consumer groups of
// 32 / NG lanes (NG = 4, 2, 1 for rows of up to 32, 64, more floats); group g owns rows g, g + NG,
// ... and sums their entries one after the other, in bag order, so every group walks ONE list of
// entries (the concatenation of its rows' bags) and all groups advance in lockstep: in step t every
// group handles the t-th entry of its list.  The lists are resolved lane-parallel, kFwdTile steps
// at a time (plan -> slot -> id, gain -> address; the next tile while this one streams), and the
// table rows stream through a ring of R step slots in shared memory with cp.async (16 bytes per
// lane and vector, nothing held in registers while in flight, R / 2 steps in flight): bytes in
// flight do not depend on the bag lengths, and a step costs the same few instructions whether it
// moves one 512-byte row or four 128-byte rows.  Every activation row is written exactly once
// (rows without entries are zeroed by the warp); sums run in ascending slot order with separately
// rounded multiply and add, so the result equals a sequential float32 loop bit for bit.
template <int K, int NG>
__global__ void __launch_bounds__(kFwdBlock) fwd_ring_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t first_act,
    uint32_t total_act) {
  constexpr int Gc = 32 / NG;           // lanes of a consumer group
  constexpr int RPG = 32 / NG;          // rows of a consumer group
  constexpr int R = fwd_ring_steps(K);
  constexpr int A = R / 2;              // steps in flight while one is consumed
  constexpr int T = kFwdTile;
  constexpr uint32_t kStepBytes = (uint32_t)K * 512u;
  extern __shared__ __align__(128) unsigned char fwd_smem[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const uint32_t r0 = first_act + (blockIdx.x * kFwdWarps + wib) * 32u;  // rows [first_act, total_act) of `tabs`
  if (r0 >= total_act) return;
  unsigned char* mine = fwd_smem + (size_t)wib * fwd_ring_warp_bytes(K, NG);
  const uint32_t ring_base = smem_addr(mine);
  FwdEntry* list = reinterpret_cast<FwdEntry*>(mine + (size_t)R * kStepBytes);
  float** s_act = reinterpret_cast<float**>(mine + (size_t)R * kStepBytes + (size_t)2 * NG * T * 16);
  uint32_t* s_begin = reinterpret_cast<uint32_t*>(s_act + 32);
  uint32_t* s_pref = s_begin + 32;
  uint32_t* s_len = s_pref + 32;
  uint32_t* s_tv = s_len + 32;  // table index | vectors per row << 16

  // Lane l describes row r0 + l.
  uint32_t begin = 0, len = 0, tv = 0;
  float* actp = nullptr;
  const bool valid = r0 + lane < total_act;
  if (valid) {
    const uint32_t my_r = r0 + lane;
    const int t = find_table(count, my_r, [&](int i) { return tabs[i].act_base; });
    const TableDesc& td = tabs[t];
    const uint32_t lr = my_r - td.act_base;
    const uint2 bag = reinterpret_cast<const uint2*>(td.bags)[lr];
    begin = bag.x;
    len = bag.y > bag.x ? bag.y - bag.x : 0u;
    tv = (uint32_t)t | ((uint32_t)(td.v.dim >> 2) << 16);
    actp = td.act + (int64_t)lr * td.v.dim;
  }
  // Position of every row inside its group's list: inclusive scan over the lanes of equal l % NG.
  uint32_t inc = len;
#pragma unroll
  for (int d = NG; d < 32; d <<= 1) {
    const uint32_t o = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += o;
  }
  s_begin[lane] = begin; s_pref[lane] = inc - len; s_len[lane] = len; s_tv[lane] = tv; s_act[lane] = actp;
  uint32_t glen[NG];
  uint32_t max_len = 0;
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    glen[g] = __shfl_sync(0xffffffffu, inc, 32 - NG + g);
    max_len = max(max_len, glen[g]);
  }
  const int my_group = lane / Gc, gl = lane % Gc;
  uint32_t my_len = glen[0];
#pragma unroll
  for (int g = 1; g < NG; ++g)
    if (my_group == g) my_len = glen[g];
  uint32_t zero_rows = __ballot_sync(0xffffffffu, valid && len == 0);
  __syncwarp();
  while (zero_rows) {  // rows without entries: the warp writes the zeros
    const int i = __ffs(zero_rows) - 1;
    zero_rows &= zero_rows - 1;
    float4* dst = reinterpret_cast<float4*>(s_act[i]);
    const int v = (int)(s_tv[i] >> 16);
    for (int c = lane; c < v; c += 32) dst[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (max_len == 0) return;

  // Resolves the entries of steps [n * T, n * T + T) of every group; lane l takes step n * T + l.
  auto build_list = [&](uint32_t n) {
    FwdEntry* L = list + (size_t)(n & 1u) * NG * T;
    const uint32_t p = n * T + (uint32_t)lane;
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      FwdEntry e;
      e.src = nullptr; e.gain = 0.f; e.meta = kEntSkip;
      if (p < glen[g]) {
        int lo = 0, hi = RPG - 1;  // last row of the group whose list position is <= p
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (s_pref[mid * NG + g] <= p) lo = mid; else hi = mid - 1;
        }
        const int row = lo * NG + g;
        const uint32_t off = p - s_pref[row];
        e.src = resolve_entry(tabs[s_tv[row] & 0xffffu], s_begin[row] + off, &e.gain);
        e.meta = (uint32_t)row | (off + 1u == s_len[row] ? kEntEnds : 0u) | (e.src == nullptr ? kEntSkip : 0u);
      }
      L[g * T + lane] = e;
    }
  };
  auto entry_of = [&](uint32_t t) -> const FwdEntry& {
    return list[(size_t)((t / T) & 1u) * NG * T + my_group * T + (t % T)];
  };
  // Starts the copies of step t: the rows that the groups sum in that step.  Always one commit group.
  auto issue = [&](uint32_t t) {
    if (t < my_len) {
      const FwdEntry& e = entry_of(t);
      if (!(e.meta & kEntSkip)) {
        const int vpr = (int)(s_tv[e.meta & 31u] >> 16);
        const float4* src = reinterpret_cast<const float4*>(e.src);
        const uint32_t dst = ring_base + (t % R) * kStepBytes + (uint32_t)lane * 16u;
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const int c = gl + k * Gc;
          if (c < vpr) cp_async16(dst + k * 512, src + c);
        }
      }
    }
    cp_async_commit();
  };
  float4 acc[K];
#pragma unroll
  for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  auto consume = [&](uint32_t t) {
    if (t >= my_len) return;
    const FwdEntry e = entry_of(t);
    const int vpr = (int)(s_tv[e.meta & 31u] >> 16);
    if (!(e.meta & kEntSkip)) {
      const uint32_t slot = ring_base + (t % R) * kStepBytes + (uint32_t)lane * 16u;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (gl + k * Gc < vpr) {
          const float4 x = lds128(slot + k * 512);
          acc[k].x = acc[k].x + e.gain * x.x; acc[k].y = acc[k].y + e.gain * x.y;
          acc[k].z = acc[k].z + e.gain * x.z; acc[k].w = acc[k].w + e.gain * x.w;
        }
      }
    }
    if (e.meta & kEntEnds) {
      float4* dst = reinterpret_cast<float4*>(s_act[e.meta & 31u]);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = gl + k * Gc;
        if (c < vpr) dst[c] = acc[k];
        acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  };

  build_list(0);
  __syncwarp();
#pragma unroll
  for (int a = 0; a < A; ++a) issue((uint32_t)a);
  for (uint32_t t = 0; t < max_len; ++t) {
    // The list of the next tile is needed by the copies issued A steps ahead; its buffer was last
    // read in the previous tile.
    if (t % T == 0 && t + T < max_len) {
      __syncwarp();  // every lane is done with step t - 1, the last reader of that buffer
      build_list(t / T + 1);
      __syncwarp();
    }
    issue(t + A);
    cp_async_wait<A>();  // this lane's copies of step t have landed
    __syncwarp();        // ... and every other lane's
    consume(t);
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------ backward

__device__ __forceinline__ float clip(float x, float lo, float hi) {
  if (!isnan(lo)) x = fmaxf(x, lo);
  if (!isnan(hi)) x = fminf(x, hi);
  return x;
}

// The two-slot optimizers beyond Adam, one scalar; returns the new (unclipped) weight.
//  adagrad momentum (sparse_dense_matmul_grad_with_adagrad_momentum.py:262-308 of the reference):
//    hyper = {lr, momentum, beta2, epsilon, exponent, use_nesterov}; slots (accumulator, momentum)
//  ftrl (..._ftrl.py:275-334): hyper = {lr, lr_power, l1, l2, beta, multiply_linear_by_lr}; slots (accumulator, linear)
//  laprop (..._laprop.py:294-335): hyper = {lr, b1, decay_rate, eps}; slots (mu, nu)
//  f2a (..._f2a.py:257-285): hyper = {lr, rho, l1, l2, max_lr_multiplier, global_step}; slots (accumulator, local_step)
// Not inlined: the common optimizers must not pay for its registers.
__device__ __noinline__ float3 apply_opt_two_slots(const OptParams& o, float w, float g, float s0, float s1) {
  if (o.kind == SC_OPT_ADAGRAD_MOMENTUM) {
    const float g2 = g * g;
    s0 = o.h2 == 1.0f ? s0 + g2 : o.h2 * s0 + (1.0f - o.h2) * g2;
    const float scaled = powf(s0 + o.h3, -1.0f / o.h4) * g;
    s1 = o.h1 * s1 + scaled;
    const float update = o.h5 != 0.0f ? o.h1 * s1 + scaled : s1;
    return make_float3(w - o.h0 * update, s0, s1);
  }
  if (o.kind == SC_OPT_FTRL) {
    const float acc_new = s0 + g * g;
    const float p_new = powf(acc_new, -o.h1);
    const float delta_p = p_new - powf(s0, -o.h1);
    const bool by_lr = o.h5 != 0.0f;
    s0 = acc_new;
    s1 = by_lr ? (s1 + o.h0 * g) - delta_p * w : (s1 + g) - (delta_p / o.h0) * w;
    const float l1 = by_lr ? o.h2 * o.h0 : o.h2;
    const float numer = o.h2 == 0.0f ? -s1 : fminf(fmaxf(s1, -l1), l1) - s1;
    const float denom = by_lr ? (p_new + 2.0f * (o.h0 * o.h3)) + o.h4 : (p_new + o.h4) / o.h0 + 2.0f * o.h3;
    return make_float3(numer / denom, s0, s1);
  }
  if (o.kind == SC_OPT_LAPROP) {
    const float g2 = g * g + o.h3;
    s1 = s1 * o.h2 + (1.0f - o.h2) * g2;
    float update = g / sqrtf(s1);
    update = o.h1 * s0 + sqrtf(1.0f - o.h1 * o.h1) * update;
    s0 = update;
    return make_float3(w - o.h0 * update, s0, s1);
  }
  // SC_OPT_F2A
  s1 = s1 + 1.0f;
  const float fa = fminf(powf(fmaxf(o.h5, 1.0f) / s1, o.h1), o.h4);
  s0 = s0 + g * g;
  const float sign = w > 0.0f ? 1.0f : (w < 0.0f ? -1.0f : 0.0f);
  const float update = (g * fa) / sqrtf(s0) + (o.h2 * sign + o.h3 * w);
  return make_float3(w - o.h0 * update, s0, s1);
}

// One optimizer step on one scalar; slot values are updated in place.  NS < 0: any optimizer;
// otherwise only the optimizers with NS slot variables can occur.
template <int NS = -1, bool EXTRA = true>
__device__ __forceinline__ float apply_opt(const OptParams& o, float w, float g, float& s0, float& s1) {
  float nw;
  if (NS == 0 || (NS < 0 && o.kind == SC_OPT_SGD)) {
    nw = w - o.h0 * g;
  } else if (NS == 1 || (NS < 0 && o.kind == SC_OPT_ADAGRAD)) {
    s0 = s0 + g * g;
    nw = w - (o.h0 * g) / sqrtf(s0);
  } else if (!EXTRA || o.kind == SC_OPT_ADAM) {
    s0 = s0 + (1.0f - o.h1) * (g - s0);
    s1 = s1 + (1.0f - o.h2) * (g * g - s1);
    nw = w - (o.h0 * s0) / (sqrtf(s1) + o.h3);
  } else {
    const float3 r = apply_opt_two_slots(o, w, g, s0, s1);
    nw = r.x; s0 = r.y; s1 = r.z;
  }
  return clip(nw, o.lo, o.hi);
}

__device__ __forceinline__ int entry_count(const TableDesc& td) {
  if (td.indirect == 2) return td.v.coo;
  return td.indirect ? (int)(td.range[1] - td.range[0]) : min(td.v.row_pointers[0], td.v.coo_per_sc);
}

__device__ __forceinline__ uint32_t entry_row(const TableDesc& td, int e, int n) {
  if (e < 0 || e >= n) return kNoRow;
  if (td.indirect == 2) return td.rows[e];
  if (td.indirect) return td.rows[td.range[0] + (uint32_t)e] - td.row_base;  // every listed entry is valid
  const int id = td.v.ids[e];
  return (id >= 0 && (int64_t)id < td.v.rows_per_shard) ? (uint32_t)id : kNoRow;
}

// Descriptor fields a backward warp needs, copied to registers once (the descriptor itself
// lives in global memory).
struct RowCtx {
  OptParams o;
  int dim, P;
  int64_t rows_per_shard;
  float* w0;  // shard 0 pointers (the only shard when P == 1)
  float* a0;
  float* b0;
  const TableDesc* td;
};

__device__ __forceinline__ RowCtx make_ctx(const TableDesc& td) {
  RowCtx c;
  c.o = td.opt;
  c.dim = td.v.dim;
  c.P = td.v.P;
  c.rows_per_shard = td.v.rows_per_shard;
  c.w0 = td.table[0];
  c.a0 = c.o.slots >= 1 ? td.slot0[0] : nullptr;
  c.b0 = c.o.slots >= 2 ? td.slot1[0] : nullptr;
  c.td = &td;
  return c;
}

__device__ __forceinline__ void row_pointers_of(const RowCtx& c, int64_t grow, float** w, float** a, float** b) {
  if (c.P == 1) {
    const int64_t off = grow * c.dim;
    *w = c.w0 + off;
    *a = c.a0 ? c.a0 + off : nullptr;
    *b = c.b0 ? c.b0 + off : nullptr;
    return;
  }
  const int g = (int)(grow / c.rows_per_shard);
  const int64_t off = (grow - (int64_t)g * c.rows_per_shard) * c.dim;
  *w = c.td->table[g] + off;
  *a = c.o.slots >= 1 ? c.td->slot0[g] + off : nullptr;
  *b = c.o.slots >= 2 ? c.td->slot1[g] + off : nullptr;
}

// Loads the table row (and slot rows) of global row `grow` into registers.
template <int W, int K>
__device__ __forceinline__ void load_row(const RowCtx& ctx, int64_t grow, int lane, typename Vec<W>::T (&w)[K],
                                         typename Vec<W>::T (&x0)[K], typename Vec<W>::T (&x1)[K]) {
  using VT = typename Vec<W>::T;
  float *pw, *pa, *pb;
  row_pointers_of(ctx, grow, &pw, &pa, &pb);
  const int vec_per_row = ctx.dim / W;
  const VT* tw = reinterpret_cast<const VT*>(pw);
  const VT* t0 = reinterpret_cast<const VT*>(pa);
  const VT* t1 = reinterpret_cast<const VT*>(pb);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + k * 32;
    const bool in = c < vec_per_row;
    w[k] = in ? tw[c] : Vec<W>::zero();
    x0[k] = (in && t0) ? t0[c] : Vec<W>::zero();
    x1[k] = (in && t1) ? t1[c] : Vec<W>::zero();
  }
}

// Applies the optimizer to a row held in registers and stores it (single write per array).
// EXTRA = false: the optimizer is known to be sgd, adagrad or adam.
template <int W, int K, bool EXTRA>
__device__ __forceinline__ void store_row(const RowCtx& ctx, int64_t grow, int lane, const typename Vec<W>::T (&gsum)[K],
                                          typename Vec<W>::T (&w)[K], typename Vec<W>::T (&x0)[K],
                                          typename Vec<W>::T (&x1)[K]) {
  using VT = typename Vec<W>::T;
  float *pw, *pa, *pb;
  row_pointers_of(ctx, grow, &pw, &pa, &pb);
  const int vec_per_row = ctx.dim / W;
  VT* tw = reinterpret_cast<VT*>(pw);
  VT* t0 = reinterpret_cast<VT*>(pa);
  VT* t1 = reinterpret_cast<VT*>(pb);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + k * 32;
    if (c >= vec_per_row) continue;
    float* wf = reinterpret_cast<float*>(&w[k]);
    float* af = reinterpret_cast<float*>(&x0[k]);
    float* bf = reinterpret_cast<float*>(&x1[k]);
    const float* gf = reinterpret_cast<const float*>(&gsum[k]);
#pragma unroll
    for (int i = 0; i < W; ++i) wf[i] = apply_opt<-1, EXTRA>(ctx.o, wf[i], gf[i], af[i], bf[i]);
    tw[c] = w[k];
    if (t0) t0[c] = x0[k];
    if (t1) t1[c] = x1[k];
  }
}

// Flags a chunk leaves for the fix-up kernel.
constexpr uint8_t kChunkHeadContinues = 1;  // a run that starts in this chunk goes on in the next one
constexpr uint8_t kChunkAllContinues = 2;   // the whole chunk continues an earlier run and does not end it

// What a backward warp knows about one of its 32 entries.
struct EntMeta {
  const float* src;  // gradient row of the entry (nullptr: contributes nothing)
  uint32_t row;      // kNoRow for lanes past the end of the list
  float gain;
};

// Warp per 32 consecutive entries of one table.  partial[(2 * global_chunk + k) * pstride ...]
// (pstride = longest row of the group, so tables of different dims never share a scratch row):
// k = 0 holds the sum of a run that started in an earlier chunk, k = 1 of a run that continues
// into the next chunk.  After the lane-parallel metadata phase the warp splits into 32 / G groups
// of G lanes; each group owns every (32 / G)-th run of the chunk, issues the loads of the run's
// table row and slot rows (NS of them) before it sums the gradient rows, and finishes with a
// single store per array.  NS is the number of slot variables (0 sgd, 1 adagrad, 2 adam).
template <int W, int K, int G, int NS>
__global__ void __launch_bounds__(kBlock) bwd_main_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_chunks,
                                                          float* __restrict__ partial, uint8_t* __restrict__ chunk_flags,
                                                          int pstride) {
  using VT = typename Vec<W>::T;
  constexpr int NG = 32 / G;
  __shared__ EntMeta s_ent[kWarpsPerBlock][32];
  __shared__ uint8_t s_start[kWarpsPerBlock][33];  // lane at which the r-th run of the chunk starts
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const uint32_t gchunk = blockIdx.x * kWarpsPerBlock + wib;
  if (gchunk >= total_chunks) return;
  const int t = find_table(count, gchunk, [&](int i) { return tabs[i].chunk_base; });
  const TableDesc& td = tabs[t];
  const CsrView& v = td.v;
  const int n = entry_count(td);
  const int e0 = (int)(gchunk - td.chunk_base) * 32;
  if (e0 >= n) {
    if (lane == 0) chunk_flags[gchunk] = 0;
    return;
  }
  const RowCtx ctx = make_ctx(td);
  const int dim = ctx.dim;
  const int vec_per_row = dim / W;

  const int e = e0 + lane;
  const uint32_t my_row = entry_row(td, e, n);
  uint32_t prev_row = __shfl_up_sync(0xffffffffu, my_row, 1);
  if (lane == 0) prev_row = entry_row(td, e0 - 1, n);
  const uint32_t next_row = entry_row(td, e0 + 32, n);  // row after the chunk
  const bool valid = my_row != kNoRow;
  {
    EntMeta m;
    m.src = nullptr; m.row = my_row; m.gain = 0.f;
    if (valid) {
      const int q = td.indirect ? (int)(td.slots[td.range[0] + (uint32_t)e] - td.ent_base) : e;
      if (td.pull != nullptr) {
        const int s = q / td.pull_cap;
        const PullSrc& src = td.pull[s];
        const int slot = td.pull_begin[s] + (q - s * td.pull_cap);
        const int sid = src.sids[slot];
        m.gain = src.gains[slot];
        if (sid >= 0 && sid < v.bdev) m.src = src.grad + (int64_t)sid * dim;
      } else {
        const int s = q / v.coo_per_sc;
        const int sid = v.sids[q];
        m.gain = v.gains[q];
        if (sid >= 0 && sid < v.bsc) m.src = td.grad + (int64_t)(s * v.bsc + sid) * dim;
      }
    }
    s_ent[wib][lane] = m;
  }
  const uint32_t heads = __ballot_sync(0xffffffffu, valid && my_row != prev_row);
  const uint32_t valids = __ballot_sync(0xffffffffu, valid);
  // Runs start at lane 0 (a continuation when lane 0 is valid but not a head) and at every head.
  const uint32_t starts = heads | (valids & 1u);
  const int nruns = __popc(starts);
  if (lane == 31) {
    // What the fix-up kernel needs to know about the run that reaches the end of the chunk.
    uint8_t flag = 0;
    if (valid && next_row == my_row) flag = ((heads >> (31 - __clz(starts))) & 1u) ? kChunkHeadContinues : kChunkAllContinues;
    chunk_flags[gchunk] = flag;
  }
  if ((starts >> lane) & 1u) s_start[wib][__popc(starts & ((1u << lane) - 1u))] = (uint8_t)lane;
  if (lane == 0) s_start[wib][nruns] = 32;
  __syncwarp();

  const int group = lane / G, gl = lane % G;
  constexpr int K0 = NS >= 1 ? K : 1, K1 = NS >= 2 ? K : 1;  // unused slot arrays shrink to one dead element
  for (int r = group; r < nruns; r += NG) {
    const int a = s_start[wib][r], b = s_start[wib][r + 1];
    const uint32_t row = s_ent[wib][a].row;
    int last = a;
    while (last + 1 < b && s_ent[wib][last + 1].row == row) ++last;  // stops at lanes past the list
    const bool is_head = (heads >> a) & 1u;
    const bool whole = is_head && !(last == 31 && next_row == row);
    float *pw = nullptr, *pa = nullptr, *pb = nullptr;
    VT w[K], x0[K0], x1[K1];
    if (whole) {
      row_pointers_of(ctx, (int64_t)row, &pw, &pa, &pb);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = gl + k * G;
        const bool in = c < vec_per_row;
        w[k] = in ? reinterpret_cast<const VT*>(pw)[c] : Vec<W>::zero();
        if (NS >= 1) x0[NS >= 1 ? k : 0] = in ? reinterpret_cast<const VT*>(pa)[c] : Vec<W>::zero();
        if (NS >= 2) x1[NS >= 2 ? k : 0] = in ? reinterpret_cast<const VT*>(pb)[c] : Vec<W>::zero();
      }
    }
    VT acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[k] = Vec<W>::zero();
    for (int j = a; j <= last; ++j) {
      const EntMeta m = s_ent[wib][j];
      if (m.src == nullptr) continue;
      const VT* src = reinterpret_cast<const VT*>(m.src);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = gl + k * G;
        if (c < vec_per_row) Vec<W>::axpy(acc[k], m.gain, src[c]);
      }
    }
    if (whole) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = gl + k * G;
        if (c >= vec_per_row) continue;
        float* wf = reinterpret_cast<float*>(&w[k]);
        float* af = NS >= 1 ? reinterpret_cast<float*>(&x0[NS >= 1 ? k : 0]) : nullptr;
        float* bf = NS >= 2 ? reinterpret_cast<float*>(&x1[NS >= 2 ? k : 0]) : nullptr;
        const float* gf = reinterpret_cast<const float*>(&acc[k]);
        float dead0 = 0.f, dead1 = 0.f;
#pragma unroll
        for (int i = 0; i < W; ++i) wf[i] = apply_opt<NS>(ctx.o, wf[i], gf[i], NS >= 1 ? af[i] : dead0, NS >= 2 ? bf[i] : dead1);
        reinterpret_cast<VT*>(pw)[c] = w[k];
        if (NS >= 1) reinterpret_cast<VT*>(pa)[c] = x0[NS >= 1 ? k : 0];
        if (NS >= 2) reinterpret_cast<VT*>(pb)[c] = x1[NS >= 2 ? k : 0];
      }
    } else {
      VT* dst = reinterpret_cast<VT*>(partial + ((int64_t)2 * gchunk + (is_head ? 1 : 0)) * pstride);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = gl + k * G;
        if (c < vec_per_row) dst[c] = acc[k];
      }
    }
  }
}

// ---- cp.async pipeline variant of the update kernel

constexpr int kPipeBlock = 128;
constexpr int kPipeWarps = kPipeBlock / 32;
constexpr int kPipeAhead = 2;  // batches in flight while one is consumed
// Rows copied per batch for K float4 vectors per lane (about 2 KiB).
__host__ __device__ constexpr int pipe_batch_rows(int K) { return K == 1 ? 4 : K == 2 ? 2 : 1; }
// Rows in a warp's ring.  While batch b is consumed, batches b + 1 .. b + kPipeAhead are in
// flight and the update of batch b may still read the 1 + NS rows before it; rounded up to a
// power of two so that a row's slot is `row & (R - 1)`.
__host__ __device__ constexpr int pipe_ring_rows(int K, int NS) {
  const int need = (kPipeAhead + 1) * pipe_batch_rows(K) + 1 + NS;
  return need <= 4 ? 4 : need <= 8 ? 8 : 16;
}
// Rows of a warp's list: 32 entries, up to 31 entries taken over from the next chunk, 1 + NS rows per run end.
__host__ __device__ constexpr int pipe_list_rows(int K, int NS) { return 32 * (3 + NS) + pipe_batch_rows(K); }
// Per-warp shared memory besides the ring: row addresses (8 bytes), descriptors and gains (4 + 4).
__host__ __device__ constexpr int pipe_list_bytes(int K, int NS) { return pipe_list_rows(K, NS) * 16; }

// What the consumer does with a row of the list.
constexpr uint32_t kRowGrad = 1;     // a gradient row: acc += gain * row
constexpr uint32_t kRowZero = 2;     // ... after clearing acc (first entry of a run)
constexpr uint32_t kRowIgnore = 4;   // ... but the entry has no gradient row: add nothing
constexpr uint32_t kRowPartial = 8;  // ... and then store acc as the chunk's partial sum
constexpr uint32_t kRowHead = 16;    // ... in the slot of a run that started in this chunk
constexpr uint32_t kRowApply = 32;   // the last of the 1 + NS table / slot rows: apply the optimizer
constexpr uint32_t kRowReduce = 64;  // reduce-only mode: store acc at red[chunk start + bits 8..12]

__device__ __forceinline__ float fast_axpy(float a, float g, float x) { return __fmaf_rn(g, x, a); }
// Hardware square root (one special-function instruction, relative error about 1e-7) instead of the
// multi-instruction IEEE sequence.
__device__ __forceinline__ float fast_sqrt(float x) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Optimizer step of the pipelined kernel: fused multiply-adds and the hardware reciprocal square
// root (2 ulp) instead of IEEE sqrt + divide; within 1e-6 relative of apply_opt.
// EXTRA: the optimizer is one of the two-slot ones beyond Adam (only with NS == 2).
template <int NS, bool EXTRA>
__device__ __forceinline__ float apply_opt_fast(const OptParams& o, bool clipped, float w, float g, float& s0, float& s1) {
  float nw;
  if (NS == 0) {
    nw = __fmaf_rn(-o.h0, g, w);
  } else if (NS == 1) {
    s0 = __fmaf_rn(g, g, s0);
    nw = __fmaf_rn(-(o.h0 * g), rsqrtf(s0), w);
  } else if (!EXTRA) {
    s0 = __fmaf_rn(1.0f - o.h1, g - s0, s0);
    s1 = __fmaf_rn(1.0f - o.h2, g * g - s1, s1);
    nw = w - __fdividef(o.h0 * s0, fast_sqrt(s1) + o.h3);
  } else {
    const float3 r = apply_opt_two_slots(o, w, g, s0, s1);
    nw = r.x; s0 = r.y; s1 = r.z;
  }
  return clipped ? clip(nw, o.lo, o.hi) : nw;
}


// Position q of entry e of a table's ordered entry list (e < entry_count) in the entry space of the table.
__device__ __forceinline__ int entry_slot(const TableDesc& td, int e) {
  return td.indirect == 1 ? (int)(td.slots[td.range[0] + (uint32_t)e] - td.ent_base) : e;
}
// Gradient row and gain of the entry at position q: `src` stays nullptr when the entry's sample id is outside the
// batch; `any_grad` is a readable address of the same memory.
__device__ __forceinline__ void entry_source(const TableDesc& td, int q, int dim, const float*& src, float& gain,
                                             const float*& any_grad) {
  const CsrView& v = td.v;
  if (td.pull != nullptr) {
    const int s = q / td.pull_cap;
    const PullSrc& ps = td.pull[s];
    const int slot = td.pull_begin[s] + (q - s * td.pull_cap);
    const int sid = ps.sids[slot];
    gain = ps.gains[slot];
    any_grad = ps.grad;
    if (sid >= 0 && sid < td.pull_rows) src = ps.grad + (int64_t)sid * dim;
  } else {
    const int s = v.S == 1 ? 0 : q / v.coo_per_sc;
    const int sid = v.sids[q];
    gain = v.gains[q];
    if (sid >= 0 && sid < v.bsc) src = td.grad + (int64_t)(s * v.bsc + sid) * dim;
  }
}

// The rows around a chunk [e0, e0 + 32), loaded together with the chunk's own rows so that no later decision waits
// for memory again.
struct ChunkRows {
  uint32_t mine;    // row of entry e0 + lane (kNoRow past the list)
  uint32_t ahead;   // row of entry e0 + 32 + lane
  uint32_t before;  // row of entry e0 - 1
  uint32_t back;    // row of entry e0 - 33
};
__device__ __forceinline__ ChunkRows load_chunk_rows(const TableDesc& td, int e0, int n, int lane) {
  ChunkRows r;
  r.mine = entry_row(td, e0 + lane, n);
  r.ahead = entry_row(td, e0 + 32 + lane, n);
  const uint32_t behind = lane < 2 ? entry_row(td, e0 - 1 - 32 * lane, n) : kNoRow;
  r.before = __shfl_sync(0xffffffffu, behind, 0);
  r.back = __shfl_sync(0xffffffffu, behind, 1);
  return r;
}

// Which runs that cross a border of the chunk the chunk's warp handles alone.  A run whose head lies in chunk c
// and which ends inside chunk c + 1 without filling it belongs to c entirely: c also reads the run's `ext` entries
// of c + 1, and c + 1 skips its first `skip` entries.  Every other crossing run goes through the chunks' partial
// sums.  Both chunks evaluate the same conditions on the same rows, so they agree.
struct ChunkBorders {
  int skip;  // leading entries of this chunk that the previous chunk handles
  int ext;   // entries of the next chunk that this chunk handles (they continue its last run)
};
__device__ __forceinline__ ChunkBorders chunk_borders(const ChunkRows& r, bool last_run_head_continues) {
  ChunkBorders b{0, 0};
  const uint32_t lead = __ballot_sync(0xffffffffu, r.mine != kNoRow && r.mine == r.before);
  if (lead != 0 && lead != 0xffffffffu && r.back != r.before) b.skip = __popc(lead);
  const uint32_t last_row = __shfl_sync(0xffffffffu, r.mine, 31);
  const uint32_t same = __ballot_sync(0xffffffffu, r.ahead == last_row);
  if (last_run_head_continues && same != 0xffffffffu) b.ext = __ffs(~same) - 1;
  return b;
}

// Same contract as bwd_main_kernel, for rows of `dim` floats with dim % 4 == 0 and 16-byte aligned
// tables, slot variables and gradients.  A warp owns 32 consecutive entries.  Lane j describes
// entry j and appends its rows to a per-warp list in shared memory, in entry order: the
// gradient row and, when a run that this warp owns entirely ends at j, the table row and the NS
// slot rows to update -- each with its address, a descriptor (kRow* flags) and the gain.  The
// warp then streams the list through a ring of R row slots with cp.async (16 bytes per lane,
// nothing held in registers while in flight): B rows per commit group, kPipeAhead groups in
// flight, and executes the descriptors of a batch as soon as it has landed -- K float4 per lane
// from shared memory.  The pipeline is as deep for a chunk of 32 single-entry rows as for one
// long run, and the bytes in flight per warp do not depend on the optimizer.
template <int K, int NS, bool REDUCE, bool EXTRA>
__global__ void __launch_bounds__(kPipeBlock) bwd_pipe_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_chunks,
                                                             float* __restrict__ partial, uint8_t* __restrict__ chunk_flags,
                                                             int ring_floats, int pstride) {
  constexpr int B = pipe_batch_rows(K);
  constexpr int R = pipe_ring_rows(K, NS);
  constexpr int kListRows = pipe_list_rows(K, NS);
  constexpr int kLanesPerRow = 32 / B;        // lanes that copy one row of a batch
  constexpr int kPieces = K * B;              // 16-byte pieces per lane and row
  extern __shared__ __align__(128) unsigned char pipe_smem[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const uint32_t gchunk = blockIdx.x * kPipeWarps + wib;
  if (gchunk >= total_chunks) return;
  const int t = warp_find_table(count, gchunk, lane, [&](int i) { return tabs[i].chunk_base; });
  const TableDesc& td = tabs[t];
  const int n = entry_count(td);
  const int e0 = (int)(gchunk - td.chunk_base) * 32;
  if (e0 >= n) {
    if (lane == 0) chunk_flags[gchunk] = 0;
    return;
  }
  const RowCtx ctx = make_ctx(td);
  const int dim = ctx.dim;
  const int vec_per_row = dim >> 2;
  const uint32_t rowbytes = (uint32_t)dim * 4u;
  // Shared memory: [rings of all warps | lists of all warps]; a list is addresses, descriptors, gains.
  const uint32_t ring_base = smem_addr(pipe_smem) + (uint32_t)wib * (uint32_t)ring_floats * 4u;
  unsigned char* list = pipe_smem + (size_t)kPipeWarps * ring_floats * 4 + (size_t)wib * pipe_list_bytes(K, NS);
  const float** rowaddr = reinterpret_cast<const float**>(list);
  uint32_t* rowdesc = reinterpret_cast<uint32_t*>(list + kListRows * 8);
  float* rowgain = reinterpret_cast<float*>(list + kListRows * 12);

  const int e = e0 + lane;
  const ChunkRows cr = load_chunk_rows(td, e0, n, lane);
  const uint32_t my_row = cr.mine;
  uint32_t prev_row = __shfl_up_sync(0xffffffffu, my_row, 1);
  if (lane == 0) prev_row = cr.before;
  const uint32_t next_row = __shfl_sync(0xffffffffu, cr.ahead, 0);  // row after the chunk
  const bool valid = my_row != kNoRow;
  const uint32_t lt = (1u << lane) - 1u;
  const uint32_t heads = __ballot_sync(0xffffffffu, valid && my_row != prev_row);
  const uint32_t valids = __ballot_sync(0xffffffffu, valid);
  if (valids == 0) {
    if (lane == 0) chunk_flags[gchunk] = 0;
    return;
  }
  const uint32_t starts = heads | (valids & 1u);
  // The run of lane j starts at the highest start bit at or below j.
  const int run_start = 31 - __clz(starts & (lt | (1u << lane)));
  const bool head_run = valid && ((heads >> run_start) & 1u);
  const bool is_end = valid && (lane == 31 || (((starts | ~valids) >> (lane + 1)) & 1u));
  const bool crosses = lane == 31 && valid && next_row == my_row;  // the last run continues in the next chunk
  const ChunkBorders border = chunk_borders(cr, __shfl_sync(0xffffffffu, crosses && head_run, 31));
  const bool goes_on = crosses && border.ext == 0;    // ... and is summed through the partial sums
  const bool w_end = is_end && head_run && !goes_on;  // a run that this chunk owns ends here: apply the optimizer
  const bool listed = valid && lane >= border.skip;   // the first `skip` entries are the previous chunk's
  const uint32_t wendmask = __ballot_sync(0xffffffffu, w_end);
  const uint32_t listedmask = __ballot_sync(0xffffffffu, listed);
  if (lane == 31)
    chunk_flags[gchunk] = goes_on ? (head_run ? kChunkHeadContinues : (run_start == 0 ? kChunkAllContinues : 0)) : 0;
  // Sources of this lane's entry and of the entry it describes among those taken over from the next chunk (x_*):
  // the two chains of loads run side by side.
  const float *my_src = nullptr, *x_src = nullptr;
  float my_gain = 0.f, x_gain = 0.f;
  const float* any_grad = td.grad;  // a readable address for entries without a gradient row
  {
    const int q = listed ? entry_slot(td, e) : -1;
    const int xq = lane < border.ext ? entry_slot(td, e + 32) : -1;
    if (q >= 0) entry_source(td, q, dim, my_src, my_gain, any_grad);
    if (xq >= 0) entry_source(td, xq, dim, x_src, x_gain, any_grad);
  }
  constexpr int kExtra = REDUCE ? 0 : 1 + NS;  // table and slot rows of an entry that applies the optimizer
  const int total = __popc(listedmask) + border.ext + kExtra * __popc(wendmask);  // rows to stream
  if (listed) {
    int o = __popc(listedmask & lt) + kExtra * __popc(wendmask & lt);
    const bool more = lane == 31 && border.ext > 0;  // the run goes on with the entries taken from the next chunk
    rowaddr[o] = my_src != nullptr ? my_src : any_grad;
    rowdesc[o] = kRowGrad | (((starts >> lane) & 1u) ? kRowZero : 0u) | (my_src == nullptr ? kRowIgnore : 0u) |
                 ((is_end && !w_end) ? kRowPartial : 0u) | (head_run ? kRowHead : 0u) |
                 ((REDUCE && w_end && !more) ? (kRowReduce | ((uint32_t)run_start << 8)) : 0u);
    rowgain[o] = my_gain;
    if (more) o += border.ext;
    if (!REDUCE && w_end) {
      float *pw, *pa, *pb;
      row_pointers_of(ctx, (int64_t)my_row, &pw, &pa, &pb);
      rowaddr[++o] = pw;
      rowdesc[o] = NS == 0 ? kRowApply : 0u;
      if (NS >= 1) { rowaddr[++o] = pa; rowdesc[o] = NS == 1 ? kRowApply : 0u; }
      if (NS >= 2) { rowaddr[++o] = pb; rowdesc[o] = kRowApply; }
    }
  }
  const int last_run_start = __shfl_sync(0xffffffffu, run_start, 31);
  if (lane < border.ext) {
    // Entry lane of the next chunk: it follows entry 31 in the list (which is listed: its run has its head here).
    const int o = __popc(listedmask) + kExtra * __popc(wendmask & 0x7fffffffu) + lane;
    rowaddr[o] = x_src != nullptr ? x_src : any_grad;
    rowdesc[o] = kRowGrad | (x_src == nullptr ? kRowIgnore : 0u) |
                 ((REDUCE && lane == border.ext - 1) ? (kRowReduce | ((uint32_t)last_run_start << 8)) : 0u);
    rowgain[o] = x_gain;
  }
  if (lane < B) rowdesc[total + lane] = 0;  // the tail of the last batch does nothing
  __syncwarp();

  // Copies the next B rows of the list into their ring slots, kLanesPerRow lanes per row;
  // always exactly one commit group.
  int issue_row = 0;
  const int my_sub = lane / kLanesPerRow, my_piece = lane % kLanesPerRow;
  auto issue_batch = [&]() {
    const int r = issue_row + my_sub;
    if (r < total) {
      const char* src = reinterpret_cast<const char*>(rowaddr[r]) + my_piece * 16;
      const uint32_t dst = ring_base + (uint32_t)(r & (R - 1)) * rowbytes + (uint32_t)my_piece * 16u;
#pragma unroll
      for (int k = 0; k < kPieces; ++k)
        if (my_piece + k * kLanesPerRow < vec_per_row) cp_async16(dst + k * kLanesPerRow * 16, src + k * kLanesPerRow * 16);
    }
    issue_row += B;
    cp_async_commit();
  };

  const bool clipped = !isnan(ctx.o.lo) || !isnan(ctx.o.hi);
  float4 acc[K];
#pragma unroll
  for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  // Executes the descriptor of list row r.
  auto consume_row = [&](int r) {
    const uint32_t d = rowdesc[r];
    const uint32_t slot_addr = ring_base + (uint32_t)(r & (R - 1)) * rowbytes + (uint32_t)lane * 16u;
    if (d & kRowGrad) {
      if (d & kRowZero) {
#pragma unroll
        for (int k = 0; k < K; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (!(d & kRowIgnore)) {
        const float gain = rowgain[r];
#pragma unroll
        for (int k = 0; k < K; ++k) {
          if (lane + k * 32 < vec_per_row) {
            const float4 x = lds128(slot_addr + k * 512);
            acc[k].x = fast_axpy(acc[k].x, gain, x.x); acc[k].y = fast_axpy(acc[k].y, gain, x.y);
            acc[k].z = fast_axpy(acc[k].z, gain, x.z); acc[k].w = fast_axpy(acc[k].w, gain, x.w);
          }
        }
      }
      if (REDUCE && (d & kRowReduce)) {
        float4* dst = reinterpret_cast<float4*>(td.red + (int64_t)(e0 + (int)((d >> 8) & 31u)) * dim);
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const int c = lane + k * 32;
          if (c < vec_per_row) dst[c] = acc[k];
        }
      }
      if (d & kRowPartial) {
        float4* dst = reinterpret_cast<float4*>(partial + ((int64_t)2 * gchunk + ((d & kRowHead) ? 1 : 0)) * pstride);
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const int c = lane + k * 32;
          if (c < vec_per_row) dst[c] = acc[k];
        }
      }
    } else if (!REDUCE && (d & kRowApply)) {
      // Rows r - NS .. r hold the table row and the slot rows.
      float* pw = const_cast<float*>(rowaddr[r - NS]);
      float* pa = NS >= 1 ? const_cast<float*>(rowaddr[r - NS + (NS >= 1 ? 1 : 0)]) : nullptr;
      float* pb = NS >= 2 ? const_cast<float*>(rowaddr[r]) : nullptr;
      const uint32_t lane_off = (uint32_t)lane * 16u;
      const uint32_t aw = ring_base + (uint32_t)((r - NS) & (R - 1)) * rowbytes + lane_off;
      const uint32_t aa = ring_base + (uint32_t)((r - NS + 1) & (R - 1)) * rowbytes + lane_off;
      const uint32_t ab = ring_base + (uint32_t)(r & (R - 1)) * rowbytes + lane_off;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = lane + k * 32;
        if (c >= vec_per_row) continue;
        float4 w = lds128(aw + k * 512);
        float4 x0 = NS >= 1 ? lds128(aa + k * 512) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 x1 = NS >= 2 ? lds128(ab + k * 512) : make_float4(0.f, 0.f, 0.f, 0.f);
        float* wf = reinterpret_cast<float*>(&w);
        float* af = reinterpret_cast<float*>(&x0);
        float* bf = reinterpret_cast<float*>(&x1);
        const float* gf = reinterpret_cast<const float*>(&acc[k]);
#pragma unroll
        for (int i = 0; i < 4; ++i) wf[i] = apply_opt_fast<NS, EXTRA>(ctx.o, clipped, wf[i], gf[i], af[i], bf[i]);
        reinterpret_cast<float4*>(pw)[c] = w;
        if (NS >= 1) reinterpret_cast<float4*>(pa)[c] = x0;
        if (NS >= 2) reinterpret_cast<float4*>(pb)[c] = x1;
      }
    }
  };

  const int batches = (total + B - 1) / B;
#pragma unroll
  for (int b = 0; b < kPipeAhead; ++b) issue_batch();
  for (int b = 0; b < batches; ++b) {
    // The slots that the next batch overwrites held rows of batch b - 2 or older, which no
    // descriptor of batch b or later reads (see pipe_ring_rows).
    issue_batch();
    cp_async_wait<kPipeAhead>();  // this lane's copies of batch b have landed
    __syncwarp();                 // ... and every other lane's
#pragma unroll
    for (int i = 0; i < B; ++i) consume_row(b * B + i);
    __syncwarp();                 // all lanes are done with the slots that the next batch recycles
  }
  cp_async_wait<0>();
}

// ---- rows of at most 128 floats: lane groups, several rows per warp instruction, rows through registers
constexpr int kGroupWindow = 8;  // entries of a window = gradient rows a lane holds in registers at a time
// Per warp: per entry the gradient row address and the gain | per run end a descriptor | table / slot row addresses
// of the runs to apply | segment sums: one pass's segments, the carry, the groups' shares of taken-over entries.
__host__ __device__ constexpr size_t lane_groups_warp_bytes(int NG, int PASSES, bool reduce_only) {
  return 32 * 12 + 34 * 4 + 8 + (reduce_only ? 0 : 32 * 3 * 8) + (size_t)(32 / PASSES + 1 + NG) * (32 / NG) * 16;
}

__device__ __forceinline__ float4 ld_row16(const float4* p) { return *p; }
__device__ __forceinline__ uint32_t lanes_below(int j) { return j >= 32 ? 0xffffffffu : (1u << j) - 1u; }

// Same contract as bwd_pipe_kernel, for rows of at most 128 / NG floats.  The warp's 32 lanes form NG groups of
// 32 / NG lanes (one float4 per lane and row), so one warp instruction moves, sums or updates NG rows.  A chunk is
// processed in PASSES passes of 32 / PASSES entries; a pass has phases whose steps are uniform across the groups:
//   reduce   group g owns the WINDOW of kGroupWindow entries [g * 8, g * 8 + 8) of the pass, whatever the runs
//            are: it loads the window's gradient rows into registers and adds them up; a SEGMENT ends where a run
//            ends or the window ends, and its sum goes to shared memory.  (The entries taken over from the next
//            chunk are split evenly among the groups in the last pass.)
//   combine  the sum of a run is the carry (the run's segments of earlier passes), its at most NG segments of the
//            pass in window order, and the groups' shares of the taken-over entries;
//   apply    the runs that the chunk owns and that end in the pass are dealt round-robin to the groups, which load
//            the table row and the slot rows, apply the optimizer and store.  Runs that cross the chunk store their
//            sum as the chunk's partial sum; in reduce-only mode the sums go to the exchange buffer.
// A hot row that fills the chunk is spread over all groups, nothing waits in a ring, and a warp needs about 6 KiB of
// shared memory and at most 64 registers per thread, so that half of the SM's warp slots are filled and hide the
// latency of a chunk's dependent metadata loads.  Inside a segment the sum runs in entry order.
template <int NG, int PASSES, int NS, bool REDUCE, bool EXTRA>
__global__ void __launch_bounds__(kPipeBlock, 8) bwd_lane_groups_kernel(const TableDesc* __restrict__ tabs, int count,
                                                                       uint32_t total_chunks, float* __restrict__ partial,
                                                                       uint8_t* __restrict__ chunk_flags, int pstride) {
  constexpr int Gc = 32 / NG;     // lanes of a group
  constexpr int S = 32 / PASSES;  // entries of a pass
  constexpr int Wd = S / NG;      // entries of a window
  static_assert(Wd == kGroupWindow, "a window is one batch of register loads");
  constexpr int kCarry = S, kTaken = S + 1;  // segment slots after the pass's own
  extern __shared__ __align__(128) unsigned char pipe_smem[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const uint32_t gchunk = blockIdx.x * kPipeWarps + wib;
  if (gchunk >= total_chunks) return;
  const int t = warp_find_table(count, gchunk, lane, [&](int i) { return tabs[i].chunk_base; });
  const TableDesc& td = tabs[t];
  const int n = entry_count(td);
  const int e0 = (int)(gchunk - td.chunk_base) * 32;
  if (e0 >= n) {
    if (lane == 0) chunk_flags[gchunk] = 0;
    return;
  }
  const RowCtx ctx = make_ctx(td);
  const int dim = ctx.dim;
  const int vec_per_row = dim >> 2;
  unsigned char* aux = pipe_smem + (size_t)wib * lane_groups_warp_bytes(NG, PASSES, REDUCE);
  const float** ent_addr = reinterpret_cast<const float**>(aux);              // [32]
  float* ent_gain = reinterpret_cast<float*>(aux + 32 * 8);                   // [32]
  uint32_t* item_desc = reinterpret_cast<uint32_t*>(aux + 32 * 12);           // [32] runs to apply, [2] runs that cross
  float** applyaddr = reinterpret_cast<float**>(aux + 32 * 12 + 34 * 4 + 8);  // [run][table, slot 0, slot 1]
  const uint32_t segs_base = smem_addr(aux + 32 * 12 + 34 * 4 + 8 + (REDUCE ? 0 : 32 * 3 * 8));  // [slot][Gc float4]

  const int e = e0 + lane;
  const ChunkRows cr = load_chunk_rows(td, e0, n, lane);
  const uint32_t my_row = cr.mine;
  uint32_t prev_row = __shfl_up_sync(0xffffffffu, my_row, 1);
  if (lane == 0) prev_row = cr.before;
  const uint32_t next_row = __shfl_sync(0xffffffffu, cr.ahead, 0);  // row after the chunk
  const bool valid = my_row != kNoRow;
  const uint32_t lt = (1u << lane) - 1u;
  const uint32_t heads = __ballot_sync(0xffffffffu, valid && my_row != prev_row);
  const uint32_t valids = __ballot_sync(0xffffffffu, valid);
  if (valids == 0) {
    if (lane == 0) chunk_flags[gchunk] = 0;
    return;
  }
  const uint32_t starts = heads | (valids & 1u);
  // The run of lane j starts at the highest start bit at or below j.
  const int run_start = 31 - __clz(starts & (lt | (1u << lane)));
  const bool head_run = valid && ((heads >> run_start) & 1u);
  const bool is_end = valid && (lane == 31 || (((starts | ~valids) >> (lane + 1)) & 1u));
  const bool crosses = lane == 31 && valid && next_row == my_row;  // the last run continues in the next chunk
  const ChunkBorders border = chunk_borders(cr, __shfl_sync(0xffffffffu, crosses && head_run, 31));
  const bool goes_on = crosses && border.ext == 0;    // ... and is summed through the partial sums
  const bool w_end = is_end && head_run && !goes_on;  // a run that this chunk owns ends here: apply the optimizer
  const bool listed = valid && lane >= border.skip;   // the first `skip` entries are the previous chunk's
  const uint32_t wendmask = __ballot_sync(0xffffffffu, w_end);
  const uint32_t listedmask = __ballot_sync(0xffffffffu, listed);
  const uint32_t endmask = __ballot_sync(0xffffffffu, listed && is_end);
  const uint32_t crossmask = endmask & ~wendmask;  // runs that cross the chunk, at most 2: the first and the last
  if (lane == 31)
    chunk_flags[gchunk] = goes_on ? (head_run ? kChunkHeadContinues : (run_start == 0 ? kChunkAllContinues : 0)) : 0;
  // Sources of this lane's entry and of the entry it describes among those taken over from the next chunk (x_*):
  // the two chains of loads run side by side.
  const float *my_src = nullptr, *x_src = nullptr;
  float my_gain = 0.f, x_gain = 0.f;
  const float* any_grad = td.grad;  // a readable address for entries without a gradient row
  {
    const int q = listed ? entry_slot(td, e) : -1;
    const int xq = lane < border.ext ? entry_slot(td, e + 32) : -1;
    if (q >= 0) entry_source(td, q, dim, my_src, my_gain, any_grad);
    if (xq >= 0) entry_source(td, xq, dim, x_src, x_gain, any_grad);
  }
  // Every address of the chunk is known now: ask L2 for the rows of this GPU's own memory (a prefetch of a peer
  // address - the gradient rows in pull mode - is not a hint but a slow remote access).
  if (td.pull == nullptr) {
    if (my_src != nullptr) prefetch_row(my_src, dim * 4);
    if (x_src != nullptr) prefetch_row(x_src, dim * 4);
  }
  // Segments: a new one starts with every run and with every window.
  const uint32_t segfirst_mask = __ballot_sync(0xffffffffu, listed && (((starts >> lane) & 1u) || lane % Wd == 0));
  const uint32_t seglast_mask = __ballot_sync(0xffffffffu, listed && (is_end || lane % Wd == Wd - 1));
  const uint32_t src_mask = __ballot_sync(0xffffffffu, listed && my_src != nullptr);
  const int my_group = lane / Gc, gl = lane % Gc;
  const bool in_row = gl < vec_per_row;
  const uint32_t seg_off = (uint32_t)gl * 16u;
  if (listed) {
    ent_addr[lane] = my_src != nullptr ? my_src : any_grad;
    ent_gain[lane] = my_gain;
    if (is_end) {
      // First and last segment of the run (numbered over the chunk), its first entry, and what to do with the sum.
      const uint32_t item = (uint32_t)__popc(seglast_mask & ((1u << run_start) - 1u)) | ((uint32_t)__popc(seglast_mask & lt) << 8) |
                            ((uint32_t)run_start << 16) | (head_run ? 1u << 24 : 0u) |
                            ((lane == 31 && border.ext > 0) ? 1u << 25 : 0u) | ((uint32_t)lane << 26);
      if (w_end) {
        const int a = __popc(wendmask & lt);
        item_desc[a] = item;
        if (!REDUCE) {
          float *pw, *pa, *pb;
          row_pointers_of(ctx, (int64_t)my_row, &pw, &pa, &pb);
          applyaddr[a * 3 + 0] = pw;
          applyaddr[a * 3 + 1] = pa;
          applyaddr[a * 3 + 2] = pb;
          prefetch_row(pw, dim * 4);
          if (NS >= 1) prefetch_row(pa, dim * 4);
          if (NS >= 2) prefetch_row(pb, dim * 4);
        }
      } else {
        item_desc[32 + __popc(crossmask & lt)] = item;
      }
    }
  }
  __syncwarp();

  auto store_slot = [&](int slot, const float4& acc) {
    const uint32_t dst = segs_base + (uint32_t)slot * (uint32_t)(Gc * 16) + seg_off;
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
  };
  auto load_slot = [&](int slot) { return lds128(segs_base + (uint32_t)slot * (uint32_t)(Gc * 16) + seg_off); };
  const bool clipped = !isnan(ctx.o.lo) || !isnan(ctx.o.hi);
  const int ncross = __popc(crossmask);

#pragma unroll
  for (int h = 0; h < PASSES; ++h) {
    const int lane0 = h * S;                                         // first entry of the pass
    const int segbase = __popc(seglast_mask & lanes_below(lane0));   // segments of earlier passes
    if (h > 0 && (listedmask >> lane0) == 0) break;                  // no entries left
    // ---- reduce: this lane's vector of the window's gradient rows, summed segment by segment
    {
      const int first = lane0 + my_group * Wd;
      float4 x[Wd];
#pragma unroll
      for (int u = 0; u < Wd; ++u) {
        x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (((src_mask >> (first + u)) & 1u) && in_row) x[u] = ld_row16(reinterpret_cast<const float4*>(ent_addr[first + u]) + gl);
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < Wd; ++u) {
        const int j = first + u;
        if (!((listedmask >> j) & 1u)) continue;
        if ((segfirst_mask >> j) & 1u) acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((src_mask >> j) & 1u) {  // (the gain of an entry without a gradient row may be anything)
          const float gain = ent_gain[j];
          acc.x = fast_axpy(acc.x, gain, x[u].x); acc.y = fast_axpy(acc.y, gain, x[u].y);
          acc.z = fast_axpy(acc.z, gain, x[u].z); acc.w = fast_axpy(acc.w, gain, x[u].w);
        }
        if (((seglast_mask >> j) & 1u) && in_row) store_slot(__popc(seglast_mask & lanes_below(j)) - segbase, acc);
      }
    }
    // ---- the entries taken over from the next chunk (they continue the chunk's last run): a contiguous share per group
    if (h == PASSES - 1 && border.ext > 0) {
      const int per = (border.ext + NG - 1) / NG;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int i = 0; i < per; i += 2) {
        float4 x[2];
        float gain[2];
        bool on[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int j = my_group * per + i + u;
          const float* src = reinterpret_cast<const float*>(__shfl_sync(0xffffffffu, (unsigned long long)x_src, j & 31));
          gain[u] = __shfl_sync(0xffffffffu, x_gain, j & 31);
          on[u] = i + u < per && j < border.ext && src != nullptr && in_row;
          x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (on[u]) x[u] = ld_row16(reinterpret_cast<const float4*>(src) + gl);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (!on[u]) continue;
          acc.x = fast_axpy(acc.x, gain[u], x[u].x); acc.y = fast_axpy(acc.y, gain[u], x[u].y);
          acc.z = fast_axpy(acc.z, gain[u], x[u].z); acc.w = fast_axpy(acc.w, gain[u], x[u].w);
        }
      }
      if (in_row) store_slot(kTaken + my_group, acc);
    }
    __syncwarp();  // the pass's segment sums are in shared memory
    // Sum of a run whose segments up to `last` lie in this pass or earlier ones (this lane's vector).
    auto run_sum = [&](int first, int last, bool taken) {
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
      if (PASSES > 1 && first < segbase) {
        g = load_slot(kCarry);
        first = segbase;
      }
#pragma unroll
      for (int k = 0; k < NG; ++k) {
        if (first + k <= last) {
          const float4 x = load_slot(first + k - segbase);
          g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
        }
      }
      if (taken) {
#pragma unroll
        for (int k = 0; k < NG; ++k) {
          const float4 x = load_slot(kTaken + k);
          g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
        }
      }
      return g;
    };
    auto item_sum = [&](uint32_t item) { return run_sum((int)(item & 31u), (int)((item >> 8) & 31u), (item >> 25) & 1u); };
    // ---- runs that cross the chunk and end in this pass: their sums are the chunk's partial sums
    for (int k = 0; k < ncross; ++k) {
      const uint32_t item = item_desc[32 + k];
      const int end_lane = (int)(item >> 26);
      if (end_lane >= lane0 && end_lane < lane0 + S && my_group == k % NG && in_row)
        reinterpret_cast<float4*>(partial + ((int64_t)2 * gchunk + ((item >> 24) & 1u)) * pstride)[gl] = item_sum(item);
    }
    // ---- the owned runs that end in this pass
    const int a_begin = __popc(wendmask & lanes_below(lane0)), a_end = __popc(wendmask & lanes_below(lane0 + S));
    if (REDUCE) {
      // reduce-only: the sums go to the exchange buffer
      for (int a = a_begin + my_group; a < a_end; a += NG) {
        if (!in_row) break;
        const uint32_t item = item_desc[a];
        reinterpret_cast<float4*>(td.red + (int64_t)(e0 + (int)((item >> 16) & 31u)) * dim)[gl] = item_sum(item);
      }
    } else {
      // dealt round-robin to the groups, two runs in registers at a time
      for (int a0 = a_begin + my_group; a0 < a_end; a0 += 2 * NG) {
        if (!in_row) break;
        float4 w[2], x0[2], x1[2];
        bool on[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int a = a0 + u * NG;
          on[u] = a < a_end;
          w[u] = x0[u] = x1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (on[u]) {
            w[u] = reinterpret_cast<const float4*>(applyaddr[a * 3 + 0])[gl];
            if (NS >= 1) x0[u] = reinterpret_cast<const float4*>(applyaddr[a * 3 + 1])[gl];
            if (NS >= 2) x1[u] = reinterpret_cast<const float4*>(applyaddr[a * 3 + 2])[gl];
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int a = a0 + u * NG;
          if (!on[u]) continue;
          const float4 g = item_sum(item_desc[a]);
          float* wf = reinterpret_cast<float*>(&w[u]);
          float* af = reinterpret_cast<float*>(&x0[u]);
          float* bf = reinterpret_cast<float*>(&x1[u]);
          const float* gf = reinterpret_cast<const float*>(&g);
#pragma unroll
          for (int i = 0; i < 4; ++i) wf[i] = apply_opt_fast<NS, EXTRA>(ctx.o, clipped, wf[i], gf[i], af[i], bf[i]);
          reinterpret_cast<float4*>(applyaddr[a * 3 + 0])[gl] = w[u];
          if (NS >= 1) reinterpret_cast<float4*>(applyaddr[a * 3 + 1])[gl] = x0[u];
          if (NS >= 2) reinterpret_cast<float4*>(applyaddr[a * 3 + 2])[gl] = x1[u];
        }
      }
    }
    if (h + 1 < PASSES) {
      // ---- a run that goes on in the next pass: its sum so far becomes the carry
      __syncwarp();  // every group has read the old carry and the pass's segments
      const int jl = lane0 + S - 1;
      if (((listedmask >> jl) & 1u) && !((endmask >> jl) & 1u)) {  // warp-uniform
        const int rs = __shfl_sync(0xffffffffu, run_start, jl);
        const float4 g = run_sum(__popc(seglast_mask & lanes_below(rs)), __popc(seglast_mask & lanes_below(jl)), false);
        __syncwarp();
        if (my_group == 0 && in_row) store_slot(kCarry, g);
      }
      __syncwarp();  // the next pass overwrites the segment slots
    }
  }
}

// Second level of the partial sums, for rows hit by thousands of entries.  Warp per group of 32
// consecutive chunks: if all of them are flagged kChunkAllContinues (they continue one and the
// same run), their 32 partial sums are added in chunk order into group_partial[group] and the
// group is flagged, so that the fix-up of that run reads one row instead of 32.
template <int W, int K>
__global__ void __launch_bounds__(kBlock) bwd_group_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_chunks,
                                                           const float* __restrict__ partial,
                                                           const uint8_t* __restrict__ chunk_flags,
                                                           float* __restrict__ group_partial, uint8_t* __restrict__ group_flags,
                                                           int pstride) {
  using VT = typename Vec<W>::T;
  const int lane = threadIdx.x & 31;
  const uint32_t group = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const uint32_t c0 = group * 32u;
  if (c0 >= total_chunks) return;
  const uint32_t c = c0 + lane;
  const bool on = c < total_chunks && (chunk_flags[c] & kChunkAllContinues);
  const bool all = __ballot_sync(0xffffffffu, on) == 0xffffffffu;
  if (lane == 0) group_flags[group] = all ? 1 : 0;
  if (!all) return;
  const int t = find_table(count, c0, [&](int i) { return tabs[i].chunk_base; });
  const int dim = tabs[t].v.dim;
  const int vec_per_row = dim / W;
  VT acc[K];
#pragma unroll
  for (int k = 0; k < K; ++k) acc[k] = Vec<W>::zero();
  constexpr int U = K == 1 ? 16 : K == 2 ? 8 : K == 4 ? 4 : 2;  // partial rows in flight
  for (int i = 0; i < 32; i += U) {
    VT p[U][K];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const VT* src = reinterpret_cast<const VT*>(partial + (int64_t)2 * (c0 + i + u) * pstride);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int cc = lane + k * 32;
        p[u][k] = cc < vec_per_row ? src[cc] : Vec<W>::zero();
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < K; ++k) Vec<W>::add(acc[k], p[u][k]);
  }
  VT* dst = reinterpret_cast<VT*>(group_partial + (int64_t)group * pstride);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int cc = lane + k * 32;
    if (cc < vec_per_row) dst[cc] = acc[k];
  }
}

// For a chunk that is flagged kChunkHeadContinues: adds the partial sums of the run that
// starts in this chunk and goes on through the following ones -- chunk by chunk up to the next
// group boundary, then whole flagged groups, then chunk by chunk to the run's end -- and
// applies the optimizer once.  Executed by a whole warp.
template <int W, int K, bool EXTRA>
__device__ __forceinline__ void fixup_chunk(const TableDesc* __restrict__ tabs, int count, uint32_t total_chunks,
                                            const float* __restrict__ partial, const uint8_t* __restrict__ chunk_flags,
                                            const float* __restrict__ group_partial, const uint8_t* __restrict__ group_flags,
                                            int pstride, uint32_t gchunk, int lane) {
  using VT = typename Vec<W>::T;
  const int t = warp_find_table(count, gchunk, lane, [&](int i) { return tabs[i].chunk_base; });
  const TableDesc& td = tabs[t];
  // The flag says that entry 31 of the chunk exists and holds a valid row.
  const uint32_t e31 = (gchunk - td.chunk_base) * 32u + 31u;
  const uint32_t row = td.indirect == 2 ? td.rows[e31]
                       : td.indirect  ? td.rows[td.range[0] + e31] - td.row_base
                                      : (uint32_t)td.v.ids[e31];
  const int dim = td.v.dim;
  const int vec_per_row = dim / W;
  // The run covers chunk gchunk + 1, every following chunk flagged kChunkAllContinues and the
  // chunk after those (where it ends).  The last chunk of a table never carries a flag.
  // Segment 1: chunks [s1, s1 + n1), none of them past the next group boundary.
  const uint32_t s1 = gchunk + 1;
  const uint32_t boundary = (s1 + 31u) & ~31u;
  uint32_t n1, ng = 0, s3, n3 = 0;
  bool ended;
  {
    const uint32_t c = s1 + lane;
    const bool on = c < boundary && c < total_chunks && (chunk_flags[c] & kChunkAllContinues);
    const uint32_t stop = __ballot_sync(0xffffffffu, !on);  // lanes at or past the boundary stop too
    const uint32_t first = (uint32_t)__ffs(stop) - 1u;      // stop != 0 unless s1 is aligned and all 32 are on
    if (stop == 0) { n1 = 32; ended = false; }
    else if (s1 + first < boundary) { n1 = first + 1; ended = true; }  // the chunk that ends the run is included
    else { n1 = first; ended = false; }
  }
  s3 = s1 + n1;
  if (!ended) {
    // Segment 2: whole groups starting at s3 (group aligned).
    for (;;) {
      const uint32_t g = s3 / 32u + ng + lane;
      const bool on = (uint64_t)(g + 1) * 32u <= total_chunks && group_flags[g];
      const uint32_t stop = __ballot_sync(0xffffffffu, !on);
      if (stop != 0) { ng += (uint32_t)__ffs(stop) - 1u; break; }
      ng += 32;
    }
    // Segment 3: chunks after the groups, up to and including the one that ends the run.
    s3 += ng * 32u;
    const uint32_t c = s3 + lane;
    const bool on = c < total_chunks && (chunk_flags[c] & kChunkAllContinues);
    const uint32_t stop = __ballot_sync(0xffffffffu, !on);  // never 0: the next group is not all on
    n3 = (uint32_t)__ffs(stop);
  }
  const float* g0 = group_partial + (int64_t)((s1 + n1) / 32u) * pstride;
  const uint32_t total = n1 + ng + n3;
  auto row_ptr = [&](uint32_t i) -> const VT* {
    if (i < n1) return reinterpret_cast<const VT*>(partial + (int64_t)2 * (s1 + i) * pstride);
    if (i < n1 + ng) return reinterpret_cast<const VT*>(g0 + (int64_t)(i - n1) * pstride);
    return reinterpret_cast<const VT*>(partial + (int64_t)2 * (s3 + (i - n1 - ng)) * pstride);
  };
  VT acc[K];
  {
    const VT* src = reinterpret_cast<const VT*>(partial + ((int64_t)2 * gchunk + 1) * pstride);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      acc[k] = c < vec_per_row ? src[c] : Vec<W>::zero();
    }
  }
  constexpr int U = K == 1 ? 8 : K == 2 ? 4 : 2;  // partial rows in flight
  uint32_t i = 0;
  for (; i + U <= total; i += U) {
    VT p[U][K];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const VT* src = row_ptr(i + u);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = lane + k * 32;
        p[u][k] = c < vec_per_row ? src[c] : Vec<W>::zero();
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < K; ++k) Vec<W>::add(acc[k], p[u][k]);
  }
  for (; i < total; ++i) {
    const VT* src = row_ptr(i);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      if (c < vec_per_row) Vec<W>::add(acc[k], src[c]);
    }
  }
  if (td.opt.kind == kReduceOnly) {
    // The run starts at the first entry of this chunk that holds `row` (entries are ordered by row).
    const uint32_t same = __ballot_sync(0xffffffffu, td.rows[e31 - 31u + (uint32_t)lane] == row);
    VT* dst = reinterpret_cast<VT*>(td.red + (int64_t)(e31 - 31u + (uint32_t)(__ffs(same) - 1)) * dim);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      if (c < vec_per_row) dst[c] = acc[k];
    }
    return;
  }
  {
    const RowCtx ctx = make_ctx(td);
    VT w[K], x0[K], x1[K];
    load_row<W, K>(ctx, (int64_t)row, lane, w, x0, x1);
    store_row<W, K, EXTRA>(ctx, (int64_t)row, lane, acc, w, x0, x1);
  }
}

// Flagged chunks are few once short crossing runs are handled by the chunk that holds their head: a warp looks at
// kFixupSpan consecutive flags and fixes up the flagged chunks one after the other.
constexpr int kFixupSpan = 8;
template <int W, int K, bool EXTRA>
__global__ void __launch_bounds__(kBlock, K <= 2 ? 4 : 1) bwd_fixup_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_chunks,
                                                           const float* __restrict__ partial,
                                                           const uint8_t* __restrict__ chunk_flags,
                                                           const float* __restrict__ group_partial,
                                                           const uint8_t* __restrict__ group_flags, int pstride) {
  const int lane = threadIdx.x & 31;
  const uint32_t c0 = (blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5)) * (uint32_t)kFixupSpan;
  if (c0 >= total_chunks) return;
  const uint32_t c = c0 + lane;
  uint32_t todo = __ballot_sync(0xffffffffu, lane < kFixupSpan && c < total_chunks && (chunk_flags[c] & kChunkHeadContinues));
  while (todo != 0) {
    const uint32_t i = (uint32_t)__ffs(todo) - 1u;
    todo &= todo - 1u;
    fixup_chunk<W, K, EXTRA>(tabs, count, total_chunks, partial, chunk_flags, group_partial, group_flags, pstride, c0 + i, lane);
  }
}


// Entry index space of all indirect tables -> sort key (row_base + global row; `invalid` for
// indices that hold no entry).  Virtual-device tables: entry index = slot of the concatenated
// buffer.  Pull tables: entry index = source * cap + position inside the source's partition.
// With `counts` != nullptr the kernel also starts a counting sort: ranks[entry] = arrival number
// among the entries of its row.
__global__ void bwd_keys_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_ent, uint32_t invalid,
                                uint32_t* __restrict__ keys, uint32_t* __restrict__ counts, uint32_t* __restrict__ ranks) {
  const uint32_t ge = blockIdx.x * blockDim.x + threadIdx.x;
  if (ge >= total_ent) return;
  // Tables with an empty entry space share their base with the next one: pick the last match.
  const int t = find_table(count, ge, [&](int i) { return tabs[i].ent_base; });
  const TableDesc& td = tabs[t];
  const CsrView& v = td.v;
  const int q = (int)(ge - td.ent_base);
  uint32_t key = invalid;
  if (td.pull != nullptr) {
    const int s = q / td.pull_cap, j = q - s * td.pull_cap;
    const PullSrc& src = td.pull[s];
    const int g = td.pull_shard;
    const int begin = g == 0 ? 0 : ((src.row_pointers[g - 1] + kAlign - 1) & ~(kAlign - 1));
    const int end = src.row_pointers[g];
    if (j == 0) td.pull_begin[s] = begin;
    if (begin + j < end) {
      const int id = src.ids[begin + j];
      if (id >= 0 && (int64_t)id < v.rows_per_shard) key = td.row_base + (uint32_t)id;
    }
  } else {
    const int s = q / v.coo_per_sc, local = q - s * v.coo_per_sc;
    const int g = slot_shard(v, s, local);
    if (g >= 0) {
      const int id = v.ids[q];
      if (id >= 0 && (int64_t)id < v.rows_per_shard) key = td.row_base + (uint32_t)((int64_t)g * v.rows_per_shard + id);
    }
  }
  keys[ge] = key;
  if (counts != nullptr && key != invalid) ranks[ge] = atomicAdd(&counts[key], 1u);
}

// ---- pull mode: the sources' partitions are already ordered by row, so the entry list is a MERGE
//
// The valid entries of a source's partition (run heads when the sources exchange reduced runs, with
// padding slots between them) are first compacted, in order, tile by tile:
//   pull_tile_count_kernel    valid entries per tile of kPullTile partition slots
//   exclusive scan            over all tiles (ordered by table, source, position): offsets of the tiles,
//                             and with them the length of every compact list and the range of every table
//   pull_tile_scatter_kernel  ckeys = row inside the shard, cidx = position inside the partition
// and then merged:
//   pull_merge_kernel         position of compact entry c of source s = c + sum over the other sources o of
//                             the number of their keys that sort before it (smaller row; equal row and o < s),
//                             by binary search.  Equal rows keep source order, then position: the order of a
//                             stable sort by row, without counters or sorting passes.
constexpr int kPullItems = 8;
constexpr int kPullTile = kScanThreads * kPullItems;  // 2048

// The partition slots [first, last) of the tile and where its source's partition starts.
struct PullTile {
  int t, s;
  int begin;        // first slot of the partition in the source buffer
  int first, last;  // positions inside the partition
};

__device__ __forceinline__ PullTile pull_tile_of(const TableDesc* __restrict__ tabs, int count, uint32_t tile) {
  PullTile p;
  p.t = find_table(count, tile, [&](int i) { return tabs[i].tile_base; });
  const TableDesc& td = tabs[p.t];
  const uint32_t local = tile - td.tile_base;
  p.s = (int)(local / td.tiles_per_list);
  const int k = (int)(local - (uint32_t)p.s * td.tiles_per_list);
  const int32_t* rp = td.pull[p.s].row_pointers;
  const int g = td.pull_shard;
  p.begin = g == 0 ? 0 : ((rp[g - 1] + kAlign - 1) & ~(kAlign - 1));
  const int len = min(max(rp[g] - p.begin, 0), td.pull_cap);
  p.first = min(k * kPullTile, len);
  p.last = min(p.first + kPullTile, len);
  return p;
}

__global__ void __launch_bounds__(kScanThreads) pull_tile_count_kernel(const TableDesc* __restrict__ tabs, int count,
                                                                       uint32_t* __restrict__ tile_counts) {
  const PullTile p = pull_tile_of(tabs, count, blockIdx.x);
  const TableDesc& td = tabs[p.t];
  const int32_t* ids = td.pull[p.s].ids + p.begin;
  uint32_t mine = 0;
  for (int j = p.first + (int)threadIdx.x; j < p.last; j += kScanThreads) {
    const int id = ids[j];
    mine += (id >= 0 && (int64_t)id < td.v.rows_per_shard) ? 1u : 0u;
  }
  uint32_t total;
  block_exclusive_scan<uint32_t>(mine, &total);
  if (threadIdx.x == 0) {
    tile_counts[blockIdx.x] = total;
    if (p.first == 0) td.pull_begin[p.s] = p.begin;
  }
}

// offs = exclusive scan of the tile counts, offs[total_tiles] = grand total.
__global__ void __launch_bounds__(kScanThreads) pull_tile_scatter_kernel(const TableDesc* __restrict__ tabs, int count,
                                                                         uint32_t total_tiles, const uint32_t* __restrict__ offs,
                                                                         uint32_t* __restrict__ ckeys, uint32_t* __restrict__ cidx,
                                                                         uint32_t* __restrict__ ranges) {
  const PullTile p = pull_tile_of(tabs, count, blockIdx.x);
  const TableDesc& td = tabs[p.t];
  const uint32_t list_first = td.tile_base + (uint32_t)p.s * td.tiles_per_list;
  if (threadIdx.x == 0 && blockIdx.x == td.tile_base) {
    ranges[p.t] = offs[blockIdx.x];
    if (p.t == count - 1) ranges[count] = offs[total_tiles];
  }
  const int32_t* ids = td.pull[p.s].ids + p.begin;
  // Thread i takes kPullItems consecutive slots, so the compact order is the slot order.
  const int j0 = p.first + (int)threadIdx.x * kPullItems;
  int id[kPullItems];
  uint32_t mine = 0;
#pragma unroll
  for (int i = 0; i < kPullItems; ++i) {
    id[i] = j0 + i < p.last ? ids[j0 + i] : -1;
    if (id[i] >= 0 && (int64_t)id[i] >= td.v.rows_per_shard) id[i] = -1;
    mine += id[i] >= 0 ? 1u : 0u;
  }
  uint32_t total;
  uint32_t c = block_exclusive_scan<uint32_t>(mine, &total) + (offs[blockIdx.x] - offs[list_first]);
  uint32_t* out_k = ckeys + td.ent_base + (uint32_t)p.s * (uint32_t)td.pull_cap;
  uint32_t* out_i = cidx + td.ent_base + (uint32_t)p.s * (uint32_t)td.pull_cap;
#pragma unroll
  for (int i = 0; i < kPullItems; ++i) {
    if (id[i] >= 0) {
      out_k[c] = (uint32_t)id[i];
      out_i[c] = (uint32_t)(j0 + i);
      ++c;
    }
  }
}

__global__ void pull_merge_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_ent,
                                  const uint32_t* __restrict__ ckeys, const uint32_t* __restrict__ cidx,
                                  const uint32_t* __restrict__ offs, uint32_t* __restrict__ rows_sorted,
                                  uint32_t* __restrict__ list) {
  const uint32_t ge = blockIdx.x * blockDim.x + threadIdx.x;
  if (ge >= total_ent) return;
  const int t = find_table(count, ge, [&](int i) { return tabs[i].ent_base; });
  const TableDesc& td = tabs[t];
  const uint32_t cap = (uint32_t)td.pull_cap, tpl = td.tiles_per_list;
  const uint32_t q = ge - td.ent_base;
  const uint32_t s = q / cap, c = q - s * cap;
  const uint32_t* list_offs = offs + td.tile_base;  // compact list o holds offs[(o + 1) * tpl] - offs[o * tpl] keys
  if (c >= list_offs[(s + 1) * tpl] - list_offs[s * tpl]) return;
  const uint32_t key = ckeys[ge];
  uint32_t pos = c;
  for (uint32_t o = 0; o < (uint32_t)td.num_sources; ++o) {
    if (o == s) continue;
    const uint32_t* other = ckeys + td.ent_base + o * cap;
    // Keys of source o that sort before this entry: row < key, and row == key when o < s.
    const uint32_t bound = o < s ? key + 1u : key;
    uint32_t lo = 0, hi = list_offs[(o + 1) * tpl] - list_offs[o * tpl];
    while (lo < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      if (other[mid] < bound) lo = mid + 1; else hi = mid;
    }
    pos += lo;
  }
  const uint32_t at = list_offs[0] + pos;
  rows_sorted[at] = td.row_base + key;
  list[at] = td.ent_base + s * cap + cidx[ge];
}

// ranges[t] = first sorted position whose key is >= row_base of table t; ranges[count] = number of
// valid entries.  Table t's entries are [ranges[t], ranges[t + 1]).
__global__ void bwd_ranges_kernel(const TableDesc* __restrict__ tabs, int count, const uint32_t* __restrict__ keys, uint32_t n,
                                  uint32_t invalid, uint32_t* __restrict__ ranges) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t > count) return;
  const uint32_t target = t < count ? tabs[t].row_base : invalid;
  uint32_t lo = 0, hi = n;
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    if (keys[mid] < target) lo = mid + 1; else hi = mid;
  }
  ranges[t] = lo;
}

// Counting sort of the entries by row, second half: offsets = exclusive scan of the counts.
// rows_sorted[position] = key and list[position] = entry for every entry with a valid key; the
// entries of one row are then put in ascending entry order by fwd_rowsort_kernel /
// fwd_bigrow_kernel, which makes the list identical to a stable sort by row.
__global__ void bwd_place_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ ranks,
                                 const uint32_t* __restrict__ offsets, uint32_t total_ent, uint32_t invalid,
                                 uint32_t* __restrict__ rows_sorted, uint32_t* __restrict__ list) {
  const uint32_t ge = blockIdx.x * blockDim.x + threadIdx.x;
  if (ge >= total_ent) return;
  const uint32_t key = keys[ge];
  if (key == invalid) return;
  const uint32_t pos = offsets[key] + ranks[ge];
  rows_sorted[pos] = key;
  list[pos] = ge;
}

// ranges[t] = first list position of table t (its rows start at row_base); ranges[count] = number
// of valid entries.
__global__ void bwd_ranges_from_offsets_kernel(const TableDesc* __restrict__ tabs, int count,
                                               const uint32_t* __restrict__ offsets, uint32_t invalid,
                                               uint32_t* __restrict__ ranges) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t > count) return;
  ranges[t] = offsets[t < count ? tabs[t].row_base : invalid];
}

// Reduce-only staging, step 1.  keys[slot] = shard * rows_per_shard + id for slots that hold an
// entry, kNoRow for alignment padding and the unwritten tail.
__global__ void stage_keys_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_slots,
                                  uint32_t* __restrict__ keys) {
  const uint32_t gq = blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= total_slots) return;
  const int t = find_table(count, gq, [&](int i) { return tabs[i].slot_base; });
  const CsrView& v = tabs[t].v;
  const int q = (int)(gq - tabs[t].slot_base);
  const int g = slot_shard(v, 0, q);
  uint32_t key = kNoRow;
  if (g >= 0) {
    const int id = v.ids[q];
    if (id >= 0 && (int64_t)id < v.rows_per_shard) key = (uint32_t)((int64_t)g * v.rows_per_shard + id);
  }
  keys[gq] = key;
}

// Reduce-only staging, step 2.  Writes the CSR buffers that the owners of the shards will read:
// one entry per run (at the run's first slot, gain 1, sample id = the slot, i.e. the row of the
// reduced-gradient buffer), padding everywhere else; row pointers are copied.
__global__ void stage_meta_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_slots,
                                  const uint32_t* __restrict__ keys, const PullSrc* __restrict__ outs) {
  const uint32_t gq = blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= total_slots) return;
  const int t = find_table(count, gq, [&](int i) { return tabs[i].slot_base; });
  const TableDesc& td = tabs[t];
  const int q = (int)(gq - td.slot_base);
  const PullSrc& out = outs[t];
  const uint32_t key = keys[gq];
  const bool head = key != kNoRow && (q == 0 || keys[gq - 1] != key);
  const_cast<int32_t*>(out.ids)[q] = head ? td.v.ids[q] : INT_MAX;
  const_cast<int32_t*>(out.sids)[q] = head ? q : INT_MAX;
  const_cast<float*>(out.gains)[q] = head ? 1.0f : nanf("");
  if (q < td.v.R) const_cast<int32_t*>(out.row_pointers)[q] = td.v.row_pointers[q];
}

// ------------------------------------------------------------------------ host side

int make_view(const sc_csr_t* c, CsrView* v) {
  if (c == nullptr) SC_FAIL(SC_INVALID_ARGUMENT, "csr descriptor is null");
  if (c->num_sc_per_device <= 0 || c->num_scs <= 0 || c->num_scs % c->num_sc_per_device != 0 ||
      (c->num_scs & (c->num_scs - 1)) != 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "num_scs (%d) must be a power of two and a multiple of num_sc_per_device (%d)", c->num_scs,
            c->num_sc_per_device);
  if (c->num_scs > SC_MAX_SHARDS) SC_FAIL(SC_UNSUPPORTED, "num_scs %d exceeds SC_MAX_SHARDS", c->num_scs);
  if (c->coo_buffer_size <= 0 || c->coo_buffer_size % c->num_sc_per_device != 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "coo_buffer_size (%d) must be positive and divisible by num_sc_per_device", c->coo_buffer_size);
  if (c->device_batch_size <= 0 || c->device_batch_size % c->num_sc_per_device != 0)
    SC_FAIL(SC_INVALID_ARGUMENT, "device_batch_size (%d) must be positive and divisible by num_sc_per_device", c->device_batch_size);
  if (c->dim <= 0 || c->rows_per_shard <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "dim and rows_per_shard must be positive");
  if ((int64_t)c->num_scs * c->rows_per_shard >= 0xffffffffLL) SC_FAIL(SC_UNSUPPORTED, "stacked table has too many rows");
  if (!c->row_pointers || !c->embedding_ids || !c->sample_ids || !c->gains) SC_FAIL(SC_INVALID_ARGUMENT, "null CSR array");
  v->row_pointers = c->row_pointers; v->ids = c->embedding_ids; v->sids = c->sample_ids; v->gains = c->gains;
  v->coo = c->coo_buffer_size; v->S = c->num_sc_per_device; v->P = c->num_scs;
  v->coo_per_sc = v->coo / v->S; v->R = v->P > kAlign ? v->P : kAlign;
  v->bdev = c->device_batch_size; v->bsc = v->bdev / v->S; v->dim = c->dim; v->rows_per_shard = c->rows_per_shard;
  return SC_OK;
}

struct SortScratch {
  SortBuffers b;
};

void carve_sort(Workspace& ws, size_t n, SortBuffers* b) {
  b->keys[0] = ws.take<uint32_t>(n); b->keys[1] = ws.take<uint32_t>(n);
  b->vals[0] = ws.take<uint32_t>(n); b->vals[1] = ws.take<uint32_t>(n);
  b->hist = ws.take<uint32_t>(sort_hist_elems(n));
  b->scan_temp = ws.take<uint32_t>(scan_temp_elems(sort_hist_elems(n)));
}

// Host image of the descriptors of one grouped call: TableDesc array followed by the shard
// pointer pool; uploaded with one cudaMemcpyAsync.
struct GroupImage {
  std::vector<TableDesc> tabs;
  std::vector<float*> pool;
  size_t bytes() const { return align_up(tabs.size() * sizeof(TableDesc), 256) + pool.size() * sizeof(float*); }
  size_t pool_offset() const { return align_up(tabs.size() * sizeof(TableDesc), 256); }
};

// Copies the image to `dst` (device) after pointing every table at its slice of the pool.
cudaError_t upload(GroupImage& g, char* dst, const std::vector<int>& pool_index, cudaStream_t cs) {
  {  // the copy below reads host memory that does not outlive this call
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(cs, &status) == cudaSuccess && status != cudaStreamCaptureStatusNone)
      return cudaErrorStreamCaptureUnsupported;
  }
  float** pool_dev = reinterpret_cast<float**>(dst + g.pool_offset());
  for (size_t i = 0; i < g.tabs.size(); ++i) {
    const int P = g.tabs[i].v.P;
    g.tabs[i].table = pool_dev + pool_index[3 * i + 0];
    g.tabs[i].slot0 = pool_index[3 * i + 1] >= 0 ? pool_dev + pool_index[3 * i + 1] : nullptr;
    g.tabs[i].slot1 = pool_index[3 * i + 2] >= 0 ? pool_dev + pool_index[3 * i + 2] : nullptr;
    (void)P;
  }
  std::vector<char> blob(g.bytes());
  memcpy(blob.data(), g.tabs.data(), g.tabs.size() * sizeof(TableDesc));
  memcpy(blob.data() + g.pool_offset(), g.pool.data(), g.pool.size() * sizeof(float*));
  // Pageable source: the call returns after the bytes were staged, so `blob` may be freed.
  return cudaMemcpyAsync(dst, blob.data(), blob.size(), cudaMemcpyHostToDevice, cs);
}

size_t image_bytes(int count, int total_shards) {
  return align_up((size_t)count * sizeof(TableDesc), 256) + (size_t)3 * total_shards * sizeof(float*);
}

// Lanes per row (G) and vectors per lane (K) for a row of `dim` floats; W is the vector width.
bool pick_group_shape(int dim, int* w, int* k, int* g) {
  *w = (dim % 4 == 0) ? 4 : 1;
  const int vecs = dim / *w;
  if (vecs <= 4) { *g = 4; *k = 1; }
  else if (vecs <= 8) { *g = 8; *k = 1; }
  else if (vecs <= 16) { *g = 8; *k = 2; }
  else if (vecs <= 32) { *g = 8; *k = 4; }
  else if (vecs <= 64) { *g = 16; *k = 4; }
  else if (vecs <= 128) { *g = 32; *k = 4; }
  else if (vecs <= 256) { *g = 32; *k = 8; }
  else return false;
  // Tuning knob: SC_GROUP_LANES=16|32 widens the groups of rows that would use 8 lanes.
  static const int forced = [] { const char* e = getenv("SC_GROUP_LANES"); return e ? atoi(e) : 0; }();
  if (*g == 8 && (forced == 16 || forced == 32)) {
    const int lanes = forced;
    *k = (vecs + lanes - 1) / lanes;
    *k = *k <= 1 ? 1 : *k <= 2 ? 2 : 4;
    *g = lanes;
  }
  return true;
}

// Lets `Kernel` use `smem` bytes of dynamic shared memory.  The driver calls are repeated only when a
// launch needs more than any earlier launch of the same kernel on the same device.
template <auto Kernel>
int configure_smem(size_t smem) {
  static size_t configured[64] = {};
  int dev = 0;
  SC_CUDA_OK(cudaGetDevice(&dev));
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && configured[dev] >= smem) return SC_OK;
  SC_CUDA_OK(cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  SC_CUDA_OK(cudaFuncSetAttribute(Kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
  if (tracked) configured[dev] = smem;
  return SC_OK;
}

template <int K, int NG>
int launch_fwd_ring(const TableDesc* tabs, int count, uint32_t first_act, uint32_t end_act, cudaStream_t st) {
  const size_t smem = (size_t)kFwdWarps * fwd_ring_warp_bytes(K, NG);
  if (int rc = configure_smem<fwd_ring_kernel<K, NG>>(smem)) return rc;
  const unsigned warps = (unsigned)ceil_div(end_act - first_act, 32);
  fwd_ring_kernel<K, NG><<<(unsigned)ceil_div(warps, kFwdWarps), kFwdBlock, smem, st>>>(tabs, count, first_act, end_act);
  SC_LAUNCH_OK("fwd_ring_kernel");
  return SC_OK;
}

// Gather with the cp.async ring; the longest row of the group picks the shape.
inline int dispatch_fwd_ring(const TableDesc* tabs, int count, uint32_t first_act, uint32_t end_act, int max_dim, cudaStream_t st) {
  const int vecs = max_dim / 4;
  if (vecs <= 8) return launch_fwd_ring<1, 4>(tabs, count, first_act, end_act, st);
  if (vecs <= 16) return launch_fwd_ring<1, 2>(tabs, count, first_act, end_act, st);
  if (vecs <= 32) return launch_fwd_ring<1, 1>(tabs, count, first_act, end_act, st);
  if (vecs <= 64) return launch_fwd_ring<2, 1>(tabs, count, first_act, end_act, st);
  if (vecs <= 128) return launch_fwd_ring<4, 1>(tabs, count, first_act, end_act, st);
  return launch_fwd_ring<8, 1>(tabs, count, first_act, end_act, st);
}

// The register kernel with L2 prefetch is the default gather; SC_FWD_KERNEL=ring selects the cp.async ring.
inline bool fwd_ring_enabled() {
  static const bool on = [] { const char* e = getenv("SC_FWD_KERNEL"); return e && strcmp(e, "ring") == 0; }();
  return on;
}

template <int W, int K, int G>
int launch_fwd_single(const TableDesc* tabs, int count, uint32_t first_act, uint32_t end_act, cudaStream_t st) {
  const unsigned warps = (unsigned)ceil_div(end_act - first_act, 32);
  fwd_gather_single_kernel<W, K, G><<<(unsigned)ceil_div(warps, kWarpsPerBlock), kBlock, 0, st>>>(tabs, count, first_act, end_act);
  SC_LAUNCH_OK("fwd_gather_single_kernel");
  return SC_OK;
}

// Activation rows per warp of the multi-hot gather.  A warp works through its rows 32 / G at a time and every step
// waits for dependent loads, so a launch too small to fill the SMs is split into more and shorter warps: the largest
// of 32, 16, 8, ... 32 / G rows that gives every SM at least 16 warps.  Launches that fill the GPU keep 32 rows (the
// first entries of 32 bags are then resolved side by side): on 8 tables x 16384 bags of ~20 ids, dim 64, 32 and 16
// rows per warp took 0.114 ms, 8 rows 0.121 ms, 4 rows 0.136 ms; on 16384 bags of one 1e8-row table, dim 128, 4 rows
// per warp took 0.052 ms instead of 0.097 ms.  SC_FWD_ROWS_PER_WARP overrides the choice.
inline int gather_rows_per_warp(uint32_t rows, int groups) {
  static const int forced = [] { const char* e = getenv("SC_FWD_ROWS_PER_WARP"); return e ? atoi(e) : 0; }();
  if (forced >= groups && forced <= 32 && forced % groups == 0) return forced;
  const uint64_t want = (uint64_t)sm_count() * 16;  // warps
  int r = 32;
  while (r > groups && ceil_div(rows, r) < (int64_t)want) r /= 2;
  return r;
}

template <int W, int K, int G>
int launch_fwd(const TableDesc* tabs, int count, uint32_t first_act, uint32_t end_act, cudaStream_t st) {
  const int rows_per_warp = gather_rows_per_warp(end_act - first_act, 32 / G);
  const unsigned warps = (unsigned)ceil_div(end_act - first_act, rows_per_warp);
  fwd_gather_kernel<W, K, G><<<(unsigned)ceil_div(warps, kWarpsPerBlock), kBlock, 0, st>>>(tabs, count, first_act, end_act, rows_per_warp);
  SC_LAUNCH_OK("fwd_gather_kernel");
  return SC_OK;
}

// Scratch that the update kernel hands to the fix-up kernels.
struct UpdateScratch {
  float* partial;        // [2 * chunks][dim]: per chunk, sum of the run continued from before / continuing after
  uint8_t* flags;        // [chunks] kChunk* flags
  float* group_partial;  // [ceil(chunks / 32)][dim]
  uint8_t* group_flags;  // [ceil(chunks / 32)]
  int pstride;           // floats between consecutive rows of partial / group_partial: the group's longest row
};
inline size_t update_groups(size_t chunks) { return (chunks + 31) / 32; }

template <int W, int K32>
int launch_fixup(const TableDesc* tabs, int count, uint32_t total_chunks, const UpdateScratch& u, bool extra, cudaStream_t st) {
  const unsigned groups = (unsigned)ceil_div(total_chunks, 32);
  bwd_group_kernel<W, K32><<<(unsigned)ceil_div(groups, kWarpsPerBlock), kBlock, 0, st>>>(tabs, count, total_chunks, u.partial,
                                                                                        u.flags, u.group_partial, u.group_flags, u.pstride);
  SC_LAUNCH_OK("bwd_group_kernel");
  const unsigned blocks = (unsigned)ceil_div(ceil_div(total_chunks, kFixupSpan), kWarpsPerBlock);
  if (extra)
    bwd_fixup_kernel<W, K32, true><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, u.partial, u.flags, u.group_partial,
                                                             u.group_flags, u.pstride);
  else
    bwd_fixup_kernel<W, K32, false><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, u.partial, u.flags, u.group_partial,
                                                              u.group_flags, u.pstride);
  SC_LAUNCH_OK("bwd_fixup_kernel");
  return SC_OK;
}

template <int K, int NS, bool REDUCE = false, bool EXTRA = false>
int launch_pipe_ns(const TableDesc* tabs, int count, uint32_t total_chunks, const UpdateScratch& u, int max_dim,
                   cudaStream_t st) {
  const int ring_floats = pipe_ring_rows(K, NS) * max_dim;
  const size_t smem = (size_t)kPipeWarps * ((size_t)ring_floats * 4 + pipe_list_bytes(K, NS));
  if (int rc = configure_smem<bwd_pipe_kernel<K, NS, REDUCE, EXTRA>>(smem)) return rc;
  const unsigned blocks = (unsigned)ceil_div(total_chunks, kPipeWarps);
  bwd_pipe_kernel<K, NS, REDUCE, EXTRA><<<blocks, kPipeBlock, smem, st>>>(tabs, count, total_chunks, u.partial, u.flags, ring_floats,
                                                                          u.pstride);
  SC_LAUNCH_OK("bwd_pipe_kernel");
  return SC_OK;
}

// Update with the cp.async pipeline kernel; K32 = float4 vectors per lane of a full warp.
template <int K32>
int launch_bwd_pipe(const TableDesc* tabs, int count, uint32_t total_chunks, const UpdateScratch& u, int num_slots,
                    bool extra, int max_dim, cudaStream_t st) {
  int rc;
  if (num_slots == kReduceOnly) rc = launch_pipe_ns<K32, 0, true>(tabs, count, total_chunks, u, max_dim, st);
  else if (num_slots == 0) rc = launch_pipe_ns<K32, 0>(tabs, count, total_chunks, u, max_dim, st);
  else if (num_slots == 1) rc = launch_pipe_ns<K32, 1>(tabs, count, total_chunks, u, max_dim, st);
  else if (!extra) rc = launch_pipe_ns<K32, 2>(tabs, count, total_chunks, u, max_dim, st);
  else rc = launch_pipe_ns<K32, 2, false, true>(tabs, count, total_chunks, u, max_dim, st);
  if (rc != SC_OK) return rc;
  return launch_fixup<4, K32>(tabs, count, total_chunks, u, extra, st);
}

template <int NG, int PASSES, int NS, bool REDUCE = false, bool EXTRA = false>
int launch_lane_groups_ns(const TableDesc* tabs, int count, uint32_t total_chunks, const UpdateScratch& u, cudaStream_t st) {
  const size_t smem = (size_t)kPipeWarps * lane_groups_warp_bytes(NG, PASSES, REDUCE);
  if (int rc = configure_smem<bwd_lane_groups_kernel<NG, PASSES, NS, REDUCE, EXTRA>>(smem)) return rc;
  const unsigned blocks = (unsigned)ceil_div(total_chunks, kPipeWarps);
  bwd_lane_groups_kernel<NG, PASSES, NS, REDUCE, EXTRA><<<blocks, kPipeBlock, smem, st>>>(tabs, count, total_chunks, u.partial, u.flags, u.pstride);
  SC_LAUNCH_OK("bwd_lane_groups_kernel");
  return SC_OK;
}

// Rows of at most 128 / NG floats: NG rows per warp instruction.
template <int NG>
int launch_bwd_lane_groups(const TableDesc* tabs, int count, uint32_t total_chunks, const UpdateScratch& u, int num_slots,
                           bool extra, cudaStream_t st) {
  constexpr int PASSES = 4 / NG;
  int rc;
  if (num_slots == kReduceOnly) rc = launch_lane_groups_ns<NG, PASSES, 0, true>(tabs, count, total_chunks, u, st);
  else if (num_slots == 0) rc = launch_lane_groups_ns<NG, PASSES, 0>(tabs, count, total_chunks, u, st);
  else if (num_slots == 1) rc = launch_lane_groups_ns<NG, PASSES, 1>(tabs, count, total_chunks, u, st);
  else if (!extra) rc = launch_lane_groups_ns<NG, PASSES, 2>(tabs, count, total_chunks, u, st);
  else rc = launch_lane_groups_ns<NG, PASSES, 2, false, true>(tabs, count, total_chunks, u, st);
  if (rc != SC_OK) return rc;
  return launch_fixup<4, 1>(tabs, count, total_chunks, u, extra, st);
}

// SC_BWD_GROUPS=off keeps short rows on the cp.async pipeline; SC_BWD_GROUPS=<dim> sends rows of up to <dim> floats
// (at most 128) to the lane-group kernel instead of the default 64.
inline int lane_groups_max_dim() {
  static const int v = [] {
    const char* e = getenv("SC_BWD_GROUPS");
    if (e == nullptr) return 64;
    if (strcmp(e, "off") == 0) return 0;
    const int d = atoi(e);
    return d < 0 ? 0 : d > 128 ? 128 : d;
  }();
  return v;
}

inline int dispatch_bwd_pipe(const TableDesc* tabs, int count, uint32_t total_chunks, const UpdateScratch& u,
                             int num_slots, bool extra, int max_dim, cudaStream_t st) {
  if (max_dim <= lane_groups_max_dim()) {
    if (max_dim <= 32) return launch_bwd_lane_groups<4>(tabs, count, total_chunks, u, num_slots, extra, st);
    if (max_dim <= 64) return launch_bwd_lane_groups<2>(tabs, count, total_chunks, u, num_slots, extra, st);
    return launch_bwd_lane_groups<1>(tabs, count, total_chunks, u, num_slots, extra, st);
  }
  const int vecs = (max_dim / 4 + 31) / 32;
  if (vecs <= 1) return launch_bwd_pipe<1>(tabs, count, total_chunks, u, num_slots, extra, max_dim, st);
  if (vecs <= 2) return launch_bwd_pipe<2>(tabs, count, total_chunks, u, num_slots, extra, max_dim, st);
  if (vecs <= 4) return launch_bwd_pipe<4>(tabs, count, total_chunks, u, num_slots, extra, max_dim, st);
  return launch_bwd_pipe<8>(tabs, count, total_chunks, u, num_slots, extra, max_dim, st);
}

// SC_BWD_SORT=radix forces the radix sort of the indirect entry list.
inline bool counting_sort_enabled() {
  static const bool on = [] { const char* e = getenv("SC_BWD_SORT"); return !(e && strcmp(e, "radix") == 0); }();
  return on;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool pipe_enabled();
// A pull item exchanges reduced runs (one gradient row per distinct table row and source) when its
// rows can go through the 16-byte asynchronous copies; otherwise the raw entries and gradients.
inline bool exchanges_reduced_runs(const CsrView& v) { return v.dim % 4 == 0 && pipe_enabled(); }

// The cp.async pipeline is the default; SC_BWD_KERNEL=groups selects the register-only kernel.
inline bool pipe_enabled() {
  static const bool on = [] { const char* e = getenv("SC_BWD_KERNEL"); return !(e && strcmp(e, "groups") == 0); }();
  return on;
}

template <int W, int K, int G>
int launch_bwd(const TableDesc* tabs, int count, uint32_t total_chunks, const UpdateScratch& u, int num_slots,
               cudaStream_t st) {
  const unsigned blocks = (unsigned)ceil_div(total_chunks, kWarpsPerBlock);
  if (num_slots == 0) bwd_main_kernel<W, K, G, 0><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, u.partial, u.flags, u.pstride);
  else if (num_slots == 1) bwd_main_kernel<W, K, G, 1><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, u.partial, u.flags, u.pstride);
  else bwd_main_kernel<W, K, G, 2><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, u.partial, u.flags, u.pstride);
  SC_LAUNCH_OK("bwd_main_kernel");
  // The fix-up kernel keeps the full warp per row: K32 vectors per lane.
  constexpr int K32 = (K * G + 31) / 32;
  return launch_fixup<W, K32>(tabs, count, total_chunks, u, true, st);
}

#define SC_SHAPE_SWITCH_W(W, k, g, CALL)             \
  do {                                               \
    if (g == 4) return CALL(W, 1, 4);                \
    if (g == 8 && k == 1) return CALL(W, 1, 8);      \
    if (g == 8 && k == 2) return CALL(W, 2, 8);      \
    if (g == 8) return CALL(W, 4, 8);                \
    if (g == 16 && k == 1) return CALL(W, 1, 16);    \
    if (g == 16 && k == 2) return CALL(W, 2, 16);    \
    if (g == 16) return CALL(W, 4, 16);              \
    if (k == 1) return CALL(W, 1, 32);               \
    if (k == 2) return CALL(W, 2, 32);               \
    if (k == 4) return CALL(W, 4, 32);               \
    return CALL(W, 8, 32);                           \
  } while (0)
#define SC_SHAPE_SWITCH(w, k, g, CALL)               \
  do {                                               \
    if (w == 4) SC_SHAPE_SWITCH_W(4, k, g, CALL);    \
    SC_SHAPE_SWITCH_W(1, k, g, CALL);                \
  } while (0)

// ---- forward group -----------------------------------------------------------------------

// A second stream per device for work that may overlap the caller's stream, with the two
// events that fork it from and join it to that stream.  Created on first use, never destroyed.
constexpr int kMaxFwdParts = 4;
struct SideStream {
  cudaStream_t stream;
  cudaEvent_t fork, join;
  cudaEvent_t part[kMaxFwdParts];  // the remote rows of part k of a forward call have arrived
};

SideStream* side_stream() {
  static SideStream streams[64];
  static bool ready[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ready[dev]) {
    if (cudaStreamCreateWithFlags(&streams[dev].stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&streams[dev].fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&streams[dev].join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int k = 0; k < kMaxFwdParts; ++k)
      if (cudaEventCreateWithFlags(&streams[dev].part[k], cudaEventDisableTiming) != cudaSuccess) return nullptr;
    ready[dev] = true;
  }
  return &streams[dev];
}

// Where the forward's plan (per activation row, its slots in ascending order) comes from.
enum FwdPlanMode {
  kPlanGiven = 0,   // every item brings the plan that preprocessing emitted
  kPlanSingle = 1,  // every item promises at most one id per sample: bags by one scatter, no list
  kPlanBuild = 2,   // counting sort of the slots by activation row, here
};

struct FwdPlan {
  std::vector<CsrView> views;
  int mode = kPlanBuild;
  bool single_valent = false;  // every item promises at most one id per sample
  uint64_t total_slots = 0, total_act = 0;
  uint64_t remote_floats = 0;  // staging space for rows of remote shards (tables with local_shard >= 0)
  int total_shards = 0;
  int w = 0, k = 0, g = 0, max_dim = 0;
};

int plan_fwd(const sc_fwd_item_t* items, int count, FwdPlan* p) {
  if (!items || count <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "empty forward group");
  p->views.resize(count);
  bool given = true, single = true;
  for (int i = 0; i < count; ++i) {
    int st = make_view(&items[i].csr, &p->views[i]);
    if (st != SC_OK) return st;
    if ((items[i].plan_slots == nullptr) != (items[i].plan_bags == nullptr))
      SC_FAIL(SC_INVALID_ARGUMENT, "plan_slots and plan_bags must be given together");
    given = given && items[i].plan_bags != nullptr;
    single = single && items[i].csr.max_ids_per_sample == 1;
    int w, k, g;
    if (!pick_group_shape(p->views[i].dim, &w, &k, &g)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the gather kernel", p->views[i].dim);
    if (i == 0) { p->w = w; p->k = k; p->g = g; }
    if (w != p->w || k != p->k || g != p->g) SC_FAIL(SC_INVALID_ARGUMENT, "tables of one group must share the row length class (dim %d vs %d)",
                                       p->views[i].dim, p->views[0].dim);
    p->max_dim = p->views[i].dim > p->max_dim ? p->views[i].dim : p->max_dim;
    p->total_slots += (uint64_t)p->views[i].coo;
    p->total_act += (uint64_t)p->views[i].bdev;
    p->total_shards += p->views[i].P;
    if (items[i].local_shard >= p->views[i].P) SC_FAIL(SC_INVALID_ARGUMENT, "local_shard %d out of range", items[i].local_shard);
    if (items[i].local_shard >= 0 && p->views[i].P > 1) p->remote_floats += (uint64_t)p->views[i].coo * (uint64_t)p->views[i].dim;
  }
  if (p->total_slots >= 0xffffffffull || p->total_act >= 0xffffffffull) SC_FAIL(SC_UNSUPPORTED, "group too large for 32-bit indices");
  p->mode = given ? kPlanGiven : single ? kPlanSingle : kPlanBuild;
  p->single_valent = single;
  return SC_OK;
}

struct FwdScratch {
  char* image;
  uint32_t* keys;       // [slots] activation row of every slot
  uint32_t* ranks;      // [slots] arrival number inside the row
  uint32_t* list;       // [slots] slots ordered by (activation row, slot)
  uint32_t* scratch;    // [slots] second buffer of the long-row sort
  uint32_t* offsets;    // [act + 2] counts, then their exclusive scan; the last word counts the long rows
  uint32_t* bags;       // [2 * act] (begin, end) of every activation row inside `list`
  uint32_t* scan_temp;
  uint32_t* big_rows;   // [slots / kSerialSortLimit + 1]
  uint32_t* run_ord;    // [slots] index of a remote slot's row in remote_rows (remote shards only)
  uint32_t* heads;      // [slots] run-head flags, then their exclusive scan
  uint32_t* heads_temp; // scan scratch of the run heads, then one word: number of runs
  FetchJob* fetch_jobs; // [slots]
  float* remote_rows;
};

bool carve_fwd(Workspace& ws, const FwdPlan& p, int count, FwdScratch* s) {
  const size_t slots = (size_t)p.total_slots, act = (size_t)p.total_act;
  s->image = ws.take<char>(image_bytes(count, p.total_shards));
  const bool build = p.mode == kPlanBuild;
  s->keys = ws.take<uint32_t>(build ? slots : 0);
  s->ranks = ws.take<uint32_t>(build ? slots : 0);
  s->list = ws.take<uint32_t>(build ? slots : 0);
  s->scratch = ws.take<uint32_t>(build ? slots : 0);
  s->offsets = ws.take<uint32_t>(build ? act + 2 : 0);
  s->bags = ws.take<uint32_t>(p.mode == kPlanGiven ? 0 : 2 * act);
  s->scan_temp = ws.take<uint32_t>(build ? scan_temp_elems(act + 1) : 0);
  s->big_rows = ws.take<uint32_t>(build ? slots / kSerialSortLimit + 1 : 0);
  s->run_ord = ws.take<uint32_t>(p.remote_floats ? slots : 0);
  s->heads = ws.take<uint32_t>(p.remote_floats ? slots : 0);
  s->heads_temp = ws.take<uint32_t>(p.remote_floats ? scan_temp_elems(slots) + kMaxFwdParts : 0);
  s->fetch_jobs = ws.take<FetchJob>(p.remote_floats ? slots : 0);
  s->remote_rows = ws.take<float>((size_t)p.remote_floats);
  return ws.ok();
}

// ---- backward group ----------------------------------------------------------------------

struct BwdPlan {
  std::vector<CsrView> views;
  std::vector<int> indirect;
  std::vector<uint32_t> n_ent;  // entry index space per table (0 for direct tables)
  uint64_t total_chunks = 0, total_ent = 0, total_rows = 0, total_tiles = 0;
  int total_shards = 0, total_sources = 0;
  int w = 0, k = 0, g = 0, max_dim = 0, kind = 0, max_slots = 0;
  bool counting = false;  // order the indirect entries by a counting sort on the row instead of a radix sort
  bool merge = false;     // every indirect table is a pull table: merge the sources' sorted partitions instead
};

int plan_bwd(const sc_grad_item_t* items, int count, BwdPlan* p) {
  if (!items || count <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "empty backward group");
  p->views.resize(count);
  p->indirect.resize(count);
  p->n_ent.resize(count);
  for (int i = 0; i < count; ++i) {
    int st = make_view(&items[i].csr, &p->views[i]);
    if (st != SC_OK) return st;
    CsrView& v = p->views[i];
    int w, k, g;
    if (!pick_group_shape(v.dim, &w, &k, &g)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the update kernel", v.dim);
    if (i == 0) { p->w = w; p->k = k; p->g = g; }
    if (w != p->w || k != p->k || g != p->g) SC_FAIL(SC_INVALID_ARGUMENT, "tables of one group must share the row length class (dim %d vs %d)",
                                       v.dim, p->views[0].dim);
    const bool pull = items[i].sources != nullptr;
    if (pull) {
      if (v.S != 1) SC_FAIL(SC_INVALID_ARGUMENT, "pull mode needs one SparseCore per device");
      if (items[i].num_sources != v.P) SC_FAIL(SC_INVALID_ARGUMENT, "pull mode needs one source per shard (%d vs %d)", items[i].num_sources, v.P);
      if (items[i].shard < 0 || items[i].shard >= v.P) SC_FAIL(SC_INVALID_ARGUMENT, "shard %d out of range", items[i].shard);
      if (items[i].partition_capacity <= 0 || items[i].partition_capacity > v.coo)
        SC_FAIL(SC_INVALID_ARGUMENT, "partition_capacity must be in (0, coo_buffer_size]");
      for (int sidx = 0; sidx < v.P; ++sidx) {
        const sc_pull_source_t& src = items[i].sources[sidx];
        if (!src.row_pointers || !src.embedding_ids || !src.sample_ids || !src.gains || !src.activation_grad)
          SC_FAIL(SC_INVALID_ARGUMENT, "source %d has a null buffer", sidx);
      }
      p->n_ent[i] = (uint32_t)((int64_t)v.P * items[i].partition_capacity);
      p->total_sources += v.P;
      p->total_tiles += (uint64_t)v.P * (uint64_t)ceil_div(items[i].partition_capacity, kPullTile);
    } else {
      p->n_ent[i] = (v.S == 1 && v.P == 1) ? 0u : (uint32_t)v.coo;
    }
    p->indirect[i] = p->n_ent[i] != 0;
    if (p->indirect[i]) {
      p->total_ent += p->n_ent[i];
      p->total_rows += pull ? (uint64_t)v.rows_per_shard : (uint64_t)v.P * (uint64_t)v.rows_per_shard;
    }
    const int64_t space = p->indirect[i] ? (int64_t)p->n_ent[i] : (int64_t)v.coo;
    p->total_chunks += (uint64_t)ceil_div(space, 32);
    p->total_shards += v.P;
    p->max_dim = v.dim > p->max_dim ? v.dim : p->max_dim;
    const sc_optimizer_t& o = items[i].optimizer;
    if (o.optimizer < 0 || o.optimizer > SC_OPT_F2A) SC_FAIL(SC_INVALID_ARGUMENT, "unknown optimizer");
    if (i == 0) { p->kind = o.optimizer; p->max_slots = optimizer_slots(o.optimizer); }
    if (o.optimizer != p->kind) SC_FAIL(SC_INVALID_ARGUMENT, "tables of one group must share the optimizer kind");
    if ((!pull && !items[i].activation_grad) || !items[i].shard_tables) SC_FAIL(SC_INVALID_ARGUMENT, "null gradient or table pointer");
    if (p->max_slots >= 1 && !items[i].shard_slot0) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 0");
    if (p->max_slots >= 2 && !items[i].shard_slot1) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 1");
    if (!isnan(o.clip_min) && !isnan(o.clip_max) && o.clip_min > o.clip_max)
      SC_FAIL(SC_INVALID_ARGUMENT, "min_value must be less than or equal to max_value");
  }
  if (p->total_chunks >= 0x7fffffffull || p->total_ent >= 0xffffffffull || p->total_rows >= 0xfffffffeull)
    SC_FAIL(SC_UNSUPPORTED, "group too large for 32-bit indices");
  // One counter per row pays off while the rows are not much more numerous than the entries
  // (measured on 26 tables, 1.9 M entries: 30 M rows lose to the radix sort, 7 M rows win).
  bool all_pull = p->total_ent > 0;
  for (int i = 0; i < count; ++i) all_pull = all_pull && items[i].sources != nullptr;
  static const bool merge_enabled = [] { const char* e = getenv("SC_BWD_SORT"); return e == nullptr || strcmp(e, "merge") == 0; }();
  p->merge = all_pull && merge_enabled;
  p->counting = !p->merge && p->total_ent > 0 && p->total_rows <= 4 * p->total_ent && counting_sort_enabled();
  return SC_OK;
}

struct BwdScratch {
  char* image;
  SortBuffers sort;  // one sorted list for all indirect tables
  // Counting sort: sort.keys[0] keys, sort.keys[1] ranks, sort.vals[0] list, sort.vals[1] scratch.
  uint32_t* rows_sorted;  // [entries]
  uint32_t* counts;       // [rows + 2] counts, then offsets; the last word counts the long rows
  uint32_t* count_temp;
  uint32_t* big_rows;
  uint32_t* ranges;
  PullSrc* pull;
  int32_t* pull_begin;
  UpdateScratch update;
};

bool carve_bwd(Workspace& ws, const BwdPlan& p, int count, BwdScratch* s) {
  s->image = ws.take<char>(image_bytes(count, p.total_shards));
  if (p.total_ent > 0 && !p.merge) carve_sort(ws, (size_t)p.total_ent, &s->sort);
  if (p.merge) {
    s->sort.keys[0] = ws.take<uint32_t>((size_t)p.total_ent);  // compact keys per (table, source)
    s->sort.keys[1] = ws.take<uint32_t>((size_t)p.total_ent);  // their positions inside the partition
    s->sort.vals[0] = ws.take<uint32_t>((size_t)p.total_ent);  // merged entry list
    s->rows_sorted = ws.take<uint32_t>((size_t)p.total_ent);
    s->counts = ws.take<uint32_t>((size_t)p.total_tiles + 1);  // valid keys per tile, then their exclusive scan
    s->count_temp = ws.take<uint32_t>(scan_temp_elems((size_t)p.total_tiles));
  }
  if (p.counting) {
    s->rows_sorted = ws.take<uint32_t>((size_t)p.total_ent);
    s->counts = ws.take<uint32_t>((size_t)p.total_rows + 2);
    s->count_temp = ws.take<uint32_t>(scan_temp_elems((size_t)p.total_rows + 1));
    s->big_rows = ws.take<uint32_t>((size_t)p.total_ent / kSerialSortLimit + 1);
  }
  s->ranges = ws.take<uint32_t>((size_t)count + 1);
  s->pull = ws.take<PullSrc>((size_t)p.total_sources + 1);
  s->pull_begin = ws.take<int32_t>((size_t)p.total_sources + 1);
  s->update.partial = ws.take<float>((size_t)2 * (size_t)p.total_chunks * (size_t)p.max_dim);
  s->update.flags = ws.take<uint8_t>((size_t)p.total_chunks + 1);
  s->update.group_partial = ws.take<float>(update_groups(p.total_chunks) * (size_t)p.max_dim + 1);
  s->update.group_flags = ws.take<uint8_t>(update_groups(p.total_chunks) + 1);
  s->update.pstride = p.max_dim;
  return ws.ok();
}

}  // namespace
}  // namespace sc

using namespace sc;

extern "C" size_t sc_sparse_dense_matmul_fwd_grouped_workspace_bytes(const sc_fwd_item_t* items, int32_t count) {
  FwdPlan p;
  if (plan_fwd(items, count, &p) != SC_OK) return 0;
  Workspace ws(nullptr, 0);
  FwdScratch s;
  carve_fwd(ws, p, count, &s);
  return ws.used();
}

extern "C" int32_t sc_sparse_dense_matmul_fwd_grouped(const sc_fwd_item_t* items, int32_t count, void* workspace,
                                                      size_t workspace_bytes, sc_stream_t stream) {
  FwdPlan p;
  int st = plan_fwd(items, count, &p);
  if (st != SC_OK) return st;
  Workspace ws(workspace, workspace_bytes);
  FwdScratch s;
  if (!carve_fwd(ws, p, count, &s)) SC_FAIL(SC_WORKSPACE_TOO_SMALL, "forward needs %zu workspace bytes, got %zu", ws.used(), workspace_bytes);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  GroupImage img;
  std::vector<int> pool_index;
  uint32_t slot_base = 0, act_base = 0;
  size_t remote_base = 0;
  bool ring = p.w == 4 && fwd_ring_enabled();  // 16-byte asynchronous copies need aligned rows
  for (int i = 0; i < count; ++i) {
    if (!items[i].shard_tables || !items[i].activations) SC_FAIL(SC_INVALID_ARGUMENT, "null table or activation pointer");
    ring = ring && aligned16(items[i].activations);
    TableDesc td;
    memset(&td, 0, sizeof td);
    td.v = p.views[i];
    td.act = items[i].activations;
    td.slot_base = slot_base; td.act_base = act_base;
    td.local_shard = (items[i].local_shard >= 0 && td.v.P > 1) ? items[i].local_shard : -1;
    if (td.local_shard >= 0) {
      td.run_ord = s.run_ord;
      td.remote_rows = s.remote_rows + remote_base;
      remote_base += (size_t)td.v.coo * (size_t)td.v.dim;
    }
    if (p.mode == kPlanGiven) {
      td.plan = items[i].plan_slots;
      td.bags = items[i].plan_bags;
      td.plan_bias = 0;
    } else {
      td.plan = p.mode == kPlanBuild ? s.list : nullptr;
      td.bags = s.bags + 2 * (size_t)act_base;
      td.plan_bias = slot_base;
    }
    slot_base += (uint32_t)td.v.coo; act_base += (uint32_t)td.v.bdev;
    pool_index.push_back((int)img.pool.size()); pool_index.push_back(-1); pool_index.push_back(-1);
    for (int g = 0; g < td.v.P; ++g) {
      if (!items[i].shard_tables[g]) SC_FAIL(SC_INVALID_ARGUMENT, "shard %d has no table pointer", g);
      ring = ring && aligned16(items[i].shard_tables[g]);
      img.pool.push_back(const_cast<float*>(items[i].shard_tables[g]));
    }
    img.tabs.push_back(td);
  }
  SC_CUDA_OK(upload(img, s.image, pool_index, cs));
  const TableDesc* tabs = reinterpret_cast<const TableDesc*>(s.image);
  const uint32_t total_slots = (uint32_t)p.total_slots, total_act = (uint32_t)p.total_act;

  PhaseScope whole("tpu_sparse_dense_matmul", cs);
  // With remote shards the tables can be handled in up to kMaxFwdParts parts of about equal size, the remote
  // rows of part k + 1 being fetched (side stream) while part k is gathered (this stream).  Measured on 2 GPUs
  // (26 tables, 65536 single-hot lookups each) the parts LOSE, 0.54 ms against 0.44 ms: the gather fills every
  // SM, so the fetch of the next part only runs in its tail, and every part pays the small planning kernels
  // again.  One part is the default; SC_FWD_PARTS=2..4 selects the split.
  static const int wanted_parts = [] {
    const char* e = getenv("SC_FWD_PARTS");
    const int v = e ? atoi(e) : 1;
    return v < 1 ? 1 : v > kMaxFwdParts ? kMaxFwdParts : v;
  }();
  int part_begin[kMaxFwdParts + 1];
  int parts = 1;
  part_begin[0] = 0;
  if (p.remote_floats > 0 && p.mode == kPlanGiven && wanted_parts > 1) {
    const uint64_t per_part = (p.total_slots + wanted_parts - 1) / wanted_parts;
    for (int i = 1; i < count && parts < wanted_parts; ++i)
      if ((uint64_t)img.tabs[i].slot_base >= per_part * (uint64_t)parts) part_begin[parts++] = i;
  }
  part_begin[parts] = count;
  auto slot_end = [&](int i) { return i < count ? img.tabs[i].slot_base : total_slots; };
  auto act_end = [&](int i) { return i < count ? img.tabs[i].act_base : total_act; };
  SideStream* side = nullptr;
  if (p.remote_floats > 0) {
    // Rows of remote shards: fetch each distinct row once, then gather from the local copies.
    side = side_stream();
    if (side == nullptr) SC_FAIL(SC_CUDA_ERROR, "cannot create the side stream of the forward");
    SC_CUDA_OK(cudaEventRecord(side->fork, cs));
    SC_CUDA_OK(cudaStreamWaitEvent(side->stream, side->fork, 0));
    cudaStream_t fs = side->stream;
    PhaseScope phase("FetchRemoteRows", fs);
    for (int k = 0; k < parts; ++k) {
      const int a = part_begin[k], n = part_begin[k + 1] - a;
      const uint32_t first = slot_end(a), slots = slot_end(a + n) - first;
      if (slots > 0) {
        const unsigned blocks = (unsigned)ceil_div(slots, kBlock);
        fwd_remote_heads_kernel<<<blocks, kBlock, 0, fs>>>(tabs + a, n, first, slots, s.heads);
        SC_LAUNCH_OK("fwd_remote_heads_kernel");
        uint32_t* total_jobs = s.heads_temp + scan_temp_elems((size_t)total_slots) + k;
        SC_CUDA_OK(exclusive_scan<uint32_t>(s.heads + first, s.heads + first, (size_t)slots, s.heads_temp, total_jobs, fs));
        fwd_fetch_plan_kernel<<<blocks, kBlock, 0, fs>>>(tabs + a, n, first, slots, s.heads, s.run_ord, s.fetch_jobs + first);
        SC_LAUNCH_OK("fwd_fetch_plan_kernel");
        fwd_fetch_kernel<<<(unsigned)sm_count() * 8, kBlock, 0, fs>>>(s.fetch_jobs + first, total_jobs, slots);
        SC_LAUNCH_OK("fwd_fetch_kernel");
      }
      SC_CUDA_OK(cudaEventRecord(side->part[k], fs));
    }
  }
  if (p.mode == kPlanSingle) {
    PhaseScope phase("ForwardPlan", cs);
    SC_CUDA_OK(cudaMemsetAsync(s.bags, 0, (size_t)total_act * 2 * sizeof(uint32_t), cs));
    fwd_single_bags_kernel<<<(unsigned)ceil_div(total_slots, kBlock), kBlock, 0, cs>>>(tabs, count, total_slots,
                                                                                      reinterpret_cast<uint2*>(s.bags));
    SC_LAUNCH_OK("fwd_single_bags_kernel");
  } else if (p.mode == kPlanBuild) {
    PhaseScope phase("ForwardPlan", cs);
    uint32_t* big_count = s.offsets + total_act + 1;
    SC_CUDA_OK(cudaMemsetAsync(s.offsets, 0, ((size_t)total_act + 2) * sizeof(uint32_t), cs));
    const unsigned slot_blocks = (unsigned)ceil_div(total_slots, kBlock);
    fwd_count_kernel<<<slot_blocks, kBlock, 0, cs>>>(tabs, count, total_slots, total_act, s.keys, s.ranks, s.offsets);
    SC_LAUNCH_OK("fwd_count_kernel");
    SC_CUDA_OK(exclusive_scan<uint32_t>(s.offsets, s.offsets, (size_t)total_act + 1, s.scan_temp, nullptr, cs));
    fwd_place_kernel<<<slot_blocks, kBlock, 0, cs>>>(s.keys, s.ranks, s.offsets, total_slots, total_act, s.list);
    SC_LAUNCH_OK("fwd_place_kernel");
    fwd_rowsort_kernel<<<(unsigned)ceil_div(total_act, kBlock), kBlock, 0, cs>>>(s.offsets, total_act, s.list, s.big_rows, big_count,
                                                                                s.bags);
    SC_LAUNCH_OK("fwd_rowsort_kernel");
    fwd_bigrow_kernel<<<(unsigned)sm_count(), kBlock, 0, cs>>>(s.offsets, s.list, s.scratch, s.big_rows, big_count,
                                                               bit_width_u32(total_slots), 1);
    SC_LAUNCH_OK("fwd_bigrow_kernel");
  }
  PhaseScope phase("GatherCombine", cs);
  for (int k = 0; k < parts; ++k) {
    const int a = part_begin[k], n = part_begin[k + 1] - a;
    const uint32_t first = act_end(a), end = act_end(a + n);
    if (side != nullptr) SC_CUDA_OK(cudaStreamWaitEvent(cs, side->part[k], 0));  // this part's remote rows have arrived
    if (end == first) continue;
    int rc = SC_OK;
    if (ring) {
      rc = dispatch_fwd_ring(tabs + a, n, first, end, p.max_dim, cs);
    } else if (p.single_valent) {
#define SC_FWD_SINGLE_CALL(W, K, G) launch_fwd_single<W, K, G>(tabs + a, n, first, end, cs)
      rc = [&]() -> int { SC_SHAPE_SWITCH(p.w, p.k, p.g, SC_FWD_SINGLE_CALL); }();
#undef SC_FWD_SINGLE_CALL
    } else {
#define SC_FWD_CALL(W, K, G) launch_fwd<W, K, G>(tabs + a, n, first, end, cs)
      // Rows of 65 .. 128 floats: 16 lanes with two vectors each instead of 8 lanes with four.  The kernel then fits
      // 4 blocks per SM (64 registers) and a warp keeps as many rows in flight; measured on bags of 1 .. 32 ids over
      // one 1e8-row table: 0.276 -> 0.177 ms at batch 131072, 0.052 -> 0.044 ms at batch 16384.  (Shorter rows lose
      // with wider groups: 64 floats 0.104 -> 0.107 ms, 32 floats 0.82 -> 1.16 ms.)
      const bool wide = p.w == 4 && p.k == 4 && p.g == 8;
      const int fk = wide ? 2 : p.k, fg = wide ? 16 : p.g;
      rc = [&]() -> int { SC_SHAPE_SWITCH(p.w, fk, fg, SC_FWD_CALL); }();
#undef SC_FWD_CALL
    }
    if (rc != SC_OK) return rc;
  }
  return SC_OK;
}

extern "C" size_t sc_sparse_dense_matmul_grad_grouped_workspace_bytes(const sc_grad_item_t* items, int32_t count) {
  BwdPlan p;
  if (plan_bwd(items, count, &p) != SC_OK) return 0;
  Workspace ws(nullptr, 0);
  BwdScratch s;
  carve_bwd(ws, p, count, &s);
  return ws.used();
}

extern "C" int32_t sc_sparse_dense_matmul_grad_grouped(const sc_grad_item_t* items, int32_t count, void* workspace,
                                                       size_t workspace_bytes, sc_stream_t stream) {
  BwdPlan p;
  int st = plan_bwd(items, count, &p);
  if (st != SC_OK) return st;
  Workspace ws(workspace, workspace_bytes);
  BwdScratch s;
  if (!carve_bwd(ws, p, count, &s)) SC_FAIL(SC_WORKSPACE_TOO_SMALL, "backward needs %zu workspace bytes, got %zu", ws.used(), workspace_bytes);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  GroupImage img;
  std::vector<int> pool_index;
  std::vector<PullSrc> pull_host;
  uint32_t chunk_base = 0, ent_base = 0, row_base = 0, tile_base = 0;
  int source_base = 0;
  bool ring = p.w == 4 && pipe_enabled();  // 16-byte asynchronous copies need aligned rows
  for (int i = 0; i < count; ++i) {
    const sc_optimizer_t& o = items[i].optimizer;
    const bool pull = items[i].sources != nullptr;
    ring = ring && aligned16(items[i].activation_grad);
    TableDesc td;
    memset(&td, 0, sizeof td);
    td.v = p.views[i];
    td.grad = items[i].activation_grad;
    td.opt.kind = o.optimizer;
    td.opt.slots = p.max_slots;
    td.opt.h0 = o.hyper[0]; td.opt.h1 = o.hyper[1]; td.opt.h2 = o.hyper[2]; td.opt.h3 = o.hyper[3];
    td.opt.h4 = o.hyper[4]; td.opt.h5 = o.hyper[5];
    td.opt.lo = o.clip_min; td.opt.hi = o.clip_max;
    td.chunk_base = chunk_base;
    td.indirect = p.indirect[i];
    td.n_ent = p.n_ent[i];
    td.ent_base = ent_base;
    td.row_base = row_base;
    td.range = s.ranges + i;
    const int table_shards = pull ? 1 : td.v.P;  // a pull table updates only the shard it owns
    td.total_rows = (uint32_t)((int64_t)table_shards * td.v.rows_per_shard);
    chunk_base += (uint32_t)ceil_div(td.indirect ? (int64_t)td.n_ent : (int64_t)td.v.coo, 32);
    if (td.indirect) {
      ent_base += td.n_ent;
      row_base += td.total_rows;
    }
    if (pull) {
      td.pull = s.pull + source_base;
      td.tiles_per_list = (uint32_t)ceil_div(items[i].partition_capacity, kPullTile);
      td.tile_base = tile_base;
      tile_base += (uint32_t)items[i].num_sources * td.tiles_per_list;
      td.pull_begin = s.pull_begin + source_base;
      td.pull_cap = items[i].partition_capacity;
      td.pull_shard = items[i].shard;
      td.num_sources = items[i].num_sources;
      td.pull_rows = exchanges_reduced_runs(td.v) ? td.v.coo : td.v.bdev;
      for (int sidx = 0; sidx < items[i].num_sources; ++sidx) {
        const sc_pull_source_t& src = items[i].sources[sidx];
        pull_host.push_back(PullSrc{src.row_pointers, src.embedding_ids, src.sample_ids, src.gains, src.activation_grad});
        ring = ring && aligned16(src.activation_grad);
      }
      source_base += items[i].num_sources;
      td.v.P = 1;  // row -> pointer arithmetic of the update sees the owned shard only
    }
    float* const* srcs[3] = {items[i].shard_tables, p.max_slots >= 1 ? items[i].shard_slot0 : nullptr,
                             p.max_slots >= 2 ? items[i].shard_slot1 : nullptr};
    for (int a = 0; a < 3; ++a) {
      if (!srcs[a]) { pool_index.push_back(-1); continue; }
      pool_index.push_back((int)img.pool.size());
      for (int g = 0; g < table_shards; ++g) {
        if (!srcs[a][g]) SC_FAIL(SC_INVALID_ARGUMENT, "shard %d misses a table or slot pointer", g);
        ring = ring && aligned16(srcs[a][g]);
        img.pool.push_back(srcs[a][g]);
      }
    }
    img.tabs.push_back(td);
  }
  PhaseScope whole("tpu_sparse_dense_matmul_grad", cs);
  const uint32_t total_ent = (uint32_t)p.total_ent, invalid = (uint32_t)p.total_rows;
  if (total_ent > 0) {
    // The sorted list lives in one of the two sort buffers; which one is known before launching.
    const int passes = (bit_width_u32(invalid) + kRadixBits - 1) / kRadixBits;
    const int res_index = passes & 1;
    for (auto& td : img.tabs) {
      td.rows = (p.counting || p.merge) ? s.rows_sorted : s.sort.keys[res_index];
      td.slots = (p.counting || p.merge) ? s.sort.vals[0] : s.sort.vals[res_index];
    }
  }
  if (!pull_host.empty())
    SC_CUDA_OK(cudaMemcpyAsync(s.pull, pull_host.data(), pull_host.size() * sizeof(PullSrc), cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(upload(img, s.image, pool_index, cs));
  const TableDesc* tabs = reinterpret_cast<const TableDesc*>(s.image);
  {
  PhaseScope order_phase("OrderEntries", cs);
  if (total_ent > 0 && p.merge) {
    // Row-sharded tables: every source's partition is ordered by row already; merge them.
    const uint32_t total_tiles = (uint32_t)p.total_tiles;
    pull_tile_count_kernel<<<total_tiles, kScanThreads, 0, cs>>>(tabs, count, s.counts);
    SC_LAUNCH_OK("pull_tile_count_kernel");
    SC_CUDA_OK(exclusive_scan<uint32_t>(s.counts, s.counts, (size_t)total_tiles, s.count_temp, s.counts + total_tiles, cs));
    pull_tile_scatter_kernel<<<total_tiles, kScanThreads, 0, cs>>>(tabs, count, total_tiles, s.counts, s.sort.keys[0], s.sort.keys[1],
                                                                  s.ranges);
    SC_LAUNCH_OK("pull_tile_scatter_kernel");
    pull_merge_kernel<<<(unsigned)ceil_div(total_ent, kBlock), kBlock, 0, cs>>>(tabs, count, total_ent, s.sort.keys[0], s.sort.keys[1],
                                                                               s.counts, s.rows_sorted, s.sort.vals[0]);
    SC_LAUNCH_OK("pull_merge_kernel");
  } else if (total_ent > 0 && p.counting) {
    // Entries of several SparseCores / shards / devices: order them by global row first, entries of
    // one row in entry order (source, sample): counting sort on the row, one for all tables.
    const uint32_t total_rows = invalid;
    uint32_t* big_count = s.counts + total_rows + 1;
    SC_CUDA_OK(cudaMemsetAsync(s.counts, 0, ((size_t)total_rows + 2) * sizeof(uint32_t), cs));
    const unsigned ent_blocks = (unsigned)ceil_div(total_ent, kBlock);
    bwd_keys_kernel<<<ent_blocks, kBlock, 0, cs>>>(tabs, count, total_ent, invalid, s.sort.keys[0], s.counts, s.sort.keys[1]);
    SC_LAUNCH_OK("bwd_keys_kernel");
    SC_CUDA_OK(exclusive_scan<uint32_t>(s.counts, s.counts, (size_t)total_rows + 1, s.count_temp, nullptr, cs));
    bwd_place_kernel<<<ent_blocks, kBlock, 0, cs>>>(s.sort.keys[0], s.sort.keys[1], s.counts, total_ent, invalid, s.rows_sorted,
                                                   s.sort.vals[0]);
    SC_LAUNCH_OK("bwd_place_kernel");
    fwd_rowsort_kernel<<<(unsigned)ceil_div(total_rows, kBlock), kBlock, 0, cs>>>(s.counts, total_rows, s.sort.vals[0], s.big_rows,
                                                                                big_count, nullptr);
    SC_LAUNCH_OK("fwd_rowsort_kernel");
    fwd_bigrow_kernel<<<(unsigned)sm_count(), kBlock, 0, cs>>>(s.counts, s.sort.vals[0], s.sort.vals[1], s.big_rows, big_count,
                                                               bit_width_u32(total_ent), 1);
    SC_LAUNCH_OK("fwd_bigrow_kernel");
    bwd_ranges_from_offsets_kernel<<<(unsigned)ceil_div(count + 1, kBlock), kBlock, 0, cs>>>(tabs, count, s.counts, invalid,
                                                                                           s.ranges);
    SC_LAUNCH_OK("bwd_ranges_from_offsets_kernel");
  } else if (total_ent > 0) {
    // The same order by a stable radix sort (rows far more numerous than entries).
    bwd_keys_kernel<<<(unsigned)ceil_div(total_ent, kBlock), kBlock, 0, cs>>>(tabs, count, total_ent, invalid, s.sort.keys[0],
                                                                             nullptr, nullptr);
    SC_LAUNCH_OK("bwd_keys_kernel");
    int res = 0;
    SC_CUDA_OK(radix_sort_pairs(s.sort, (size_t)total_ent, bit_width_u32(invalid), true, &res, cs));
    const int passes = (bit_width_u32(invalid) + kRadixBits - 1) / kRadixBits;
    if (res != (passes & 1)) SC_FAIL(SC_CUDA_ERROR, "internal: unexpected sort buffer parity");
    bwd_ranges_kernel<<<(unsigned)ceil_div(count + 1, kBlock), kBlock, 0, cs>>>(tabs, count, s.sort.keys[res], total_ent, invalid,
                                                                              s.ranges);
    SC_LAUNCH_OK("bwd_ranges_kernel");
  }
  }
  PhaseScope update_phase("ReduceAndUpdate", cs);
  const uint32_t total_chunks = (uint32_t)p.total_chunks;
  if (ring) return dispatch_bwd_pipe(tabs, count, total_chunks, s.update, p.max_slots, p.kind >= SC_OPT_ADAGRAD_MOMENTUM, p.max_dim, cs);
#define SC_BWD_CALL(W, K, G) launch_bwd<W, K, G>(tabs, count, total_chunks, s.update, p.max_slots, cs)
  SC_SHAPE_SWITCH(p.w, p.k, p.g, SC_BWD_CALL);
#undef SC_BWD_CALL
}

// One (source, destination, bytes) triple of the grouped staging copy; all multiples of 4 bytes.
struct CopyJob {
  const uint32_t* src;
  uint32_t* dst;
  uint64_t words;
};

// blockIdx.y = job; the blocks of a row stride over the job's words (16-byte vectors when aligned).
__global__ void stage_copy_kernel(const CopyJob* __restrict__ jobs) {
  const CopyJob j = jobs[blockIdx.y];
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if ((((uintptr_t)j.src | (uintptr_t)j.dst) & 15) == 0) {
    const uint64_t vecs = j.words / 4;
    const uint4* s4 = reinterpret_cast<const uint4*>(j.src);
    uint4* d4 = reinterpret_cast<uint4*>(j.dst);
    for (uint64_t i = tid; i < vecs; i += stride) d4[i] = s4[i];
    for (uint64_t i = vecs * 4 + tid; i < j.words; i += stride) j.dst[i] = j.src[i];
  } else {
    for (uint64_t i = tid; i < j.words; i += stride) j.dst[i] = j.src[i];
  }
}

struct StagePlan {
  std::vector<CsrView> views;
  std::vector<int> reduced;  // per item
  uint64_t slots = 0, chunks = 0;
  int reduced_count = 0, max_dim = 0;
  size_t copy_jobs = 0;
};

int plan_stage(const sc_grad_item_t* items, int count, StagePlan* p) {
  if (!items || count <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "empty backward group");
  p->views.resize(count);
  p->reduced.assign(count, 0);
  for (int i = 0; i < count; ++i) {
    const sc_grad_item_t& it = items[i];
    if (!it.sources) continue;
    int st = make_view(&it.csr, &p->views[i]);
    if (st != SC_OK) return st;
    const CsrView& v = p->views[i];
    if (it.shard < 0 || it.shard >= it.num_sources || !it.activation_grad) SC_FAIL(SC_INVALID_ARGUMENT, "bad pull item");
    if (v.S != 1) SC_FAIL(SC_UNSUPPORTED, "pull mode needs one SparseCore per device");
    if (exchanges_reduced_runs(v)) {
      p->reduced[i] = 1;
      p->reduced_count += 1;
      p->slots += (uint64_t)v.coo;
      p->chunks += (uint64_t)ceil_div(v.coo, 32);
      p->max_dim = v.dim > p->max_dim ? v.dim : p->max_dim;
    } else {
      p->copy_jobs += 5;
    }
  }
  if (p->slots >= 0xffffffffull || p->chunks >= 0x7fffffffull) SC_FAIL(SC_UNSUPPORTED, "group too large for 32-bit indices");
  return SC_OK;
}

struct StageScratch {
  CopyJob* jobs;
  char* image;
  PullSrc* outs;
  uint32_t* keys;
  UpdateScratch update;
};

bool carve_stage(Workspace& ws, const StagePlan& p, StageScratch* s) {
  s->jobs = ws.take<CopyJob>(p.copy_jobs + 1);
  s->image = ws.take<char>(image_bytes(p.reduced_count + 1, p.reduced_count + 1));
  s->outs = ws.take<PullSrc>((size_t)p.reduced_count + 1);
  s->keys = ws.take<uint32_t>((size_t)p.slots + 1);
  s->update.partial = ws.take<float>((size_t)2 * (size_t)p.chunks * (size_t)p.max_dim + 1);
  s->update.flags = ws.take<uint8_t>((size_t)p.chunks + 1);
  s->update.group_partial = ws.take<float>(update_groups(p.chunks) * (size_t)p.max_dim + 1);
  s->update.group_flags = ws.take<uint8_t>(update_groups(p.chunks) + 1);
  s->update.pstride = p.max_dim;
  return ws.ok();
}

extern "C" size_t sc_sparse_dense_matmul_grad_stage_workspace_bytes(const sc_grad_item_t* items, int32_t count) {
  StagePlan p;
  if (plan_stage(items, count, &p) != SC_OK) return 0;
  Workspace ws(nullptr, 0);
  StageScratch s;
  carve_stage(ws, p, &s);
  return ws.used();
}

// Pull mode, before the barrier: publishes what this device holds for every shard in its own
// peer-visible exchange buffers (sources[shard]).  Items whose rows allow it publish reduced runs:
// the gradient rows of all entries of one (shard, row) run are summed here, in slot order, into
// activation_grad[first slot of the run] of the exchange buffers (which must hold coo_buffer_size
// rows), and the exchanged CSR lists one entry per run.  A row that many samples of the batch hit
// then crosses NVLink once per source instead of once per sample.  Other items copy their CSR
// buffers and activation gradients unchanged.
extern "C" int32_t sc_sparse_dense_matmul_grad_stage(const sc_grad_item_t* items, int32_t count, void* workspace,
                                                     size_t workspace_bytes, sc_stream_t stream) {
  StagePlan p;
  int st = plan_stage(items, count, &p);
  if (st != SC_OK) return st;
  Workspace ws(workspace, workspace_bytes);
  StageScratch s;
  if (!carve_stage(ws, p, &s)) SC_FAIL(SC_WORKSPACE_TOO_SMALL, "staging needs %zu workspace bytes, got %zu", ws.used(), workspace_bytes);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  PhaseScope whole("StageGradients", cs);

  std::vector<CopyJob> jobs;
  GroupImage img;
  std::vector<int> pool_index;
  std::vector<PullSrc> outs;
  uint32_t slot_base = 0, chunk_base = 0;
  for (int i = 0; i < count; ++i) {
    const sc_grad_item_t& it = items[i];
    if (!it.sources) continue;
    const CsrView& v = p.views[i];
    const sc_pull_source_t& own = it.sources[it.shard];
    if (!own.row_pointers || !own.embedding_ids || !own.sample_ids || !own.gains || !own.activation_grad)
      SC_FAIL(SC_INVALID_ARGUMENT, "this device's exchange buffers are missing");
    if (!p.reduced[i]) {
      const void* srcs[5] = {v.row_pointers, v.ids, v.sids, v.gains, it.activation_grad};
      const void* dsts[5] = {own.row_pointers, own.embedding_ids, own.sample_ids, own.gains, own.activation_grad};
      const uint64_t words[5] = {(uint64_t)v.R * v.S, (uint64_t)v.coo, (uint64_t)v.coo, (uint64_t)v.coo,
                                 (uint64_t)v.bdev * v.dim};
      for (int a = 0; a < 5; ++a) {
        if (srcs[a] == dsts[a] || words[a] == 0) continue;
        jobs.push_back(CopyJob{static_cast<const uint32_t*>(srcs[a]),
                               const_cast<uint32_t*>(static_cast<const uint32_t*>(dsts[a])), words[a]});
      }
      continue;
    }
    if (!aligned16(it.activation_grad) || !aligned16(own.activation_grad))
      SC_FAIL(SC_UNSUPPORTED, "activation gradients of a row-sharded table must be 16-byte aligned");
    if (own.embedding_ids == v.ids || own.sample_ids == v.sids || own.gains == v.gains || own.activation_grad == it.activation_grad)
      SC_FAIL(SC_INVALID_ARGUMENT, "the exchange buffers must not alias the CSR operands or the activation gradients");
    TableDesc td;
    memset(&td, 0, sizeof td);
    td.v = v;
    td.grad = it.activation_grad;
    td.opt.kind = kReduceOnly;
    td.opt.lo = td.opt.hi = nanf("");
    td.indirect = 2;
    td.rows = s.keys + slot_base;
    td.red = const_cast<float*>(own.activation_grad);
    td.slot_base = slot_base;
    td.chunk_base = chunk_base;
    td.local_shard = -1;
    slot_base += (uint32_t)v.coo;
    chunk_base += (uint32_t)ceil_div(v.coo, 32);
    pool_index.push_back((int)img.pool.size()); pool_index.push_back(-1); pool_index.push_back(-1);
    img.pool.push_back(td.red);  // make_ctx reads table[0]; never dereferenced in this mode
    img.tabs.push_back(td);
    outs.push_back(PullSrc{own.row_pointers, own.embedding_ids, own.sample_ids, own.gains, own.activation_grad});
  }
  if (!jobs.empty()) {
    SC_CUDA_OK(cudaMemcpyAsync(s.jobs, jobs.data(), jobs.size() * sizeof(CopyJob), cudaMemcpyHostToDevice, cs));
    dim3 grid(32, (unsigned)jobs.size());
    stage_copy_kernel<<<grid, kBlock, 0, cs>>>(s.jobs);
    SC_LAUNCH_OK("stage_copy_kernel");
  }
  if (img.tabs.empty()) return SC_OK;
  const int n = (int)img.tabs.size();
  SC_CUDA_OK(cudaMemcpyAsync(s.outs, outs.data(), outs.size() * sizeof(PullSrc), cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(upload(img, s.image, pool_index, cs));
  const TableDesc* tabs = reinterpret_cast<const TableDesc*>(s.image);
  const uint32_t total_slots = (uint32_t)p.slots;
  const unsigned slot_blocks = (unsigned)ceil_div(total_slots, kBlock);
  stage_keys_kernel<<<slot_blocks, kBlock, 0, cs>>>(tabs, n, total_slots, s.keys);
  SC_LAUNCH_OK("stage_keys_kernel");
  stage_meta_kernel<<<slot_blocks, kBlock, 0, cs>>>(tabs, n, total_slots, s.keys, s.outs);
  SC_LAUNCH_OK("stage_meta_kernel");
  return dispatch_bwd_pipe(tabs, n, (uint32_t)p.chunks, s.update, kReduceOnly, false, p.max_dim, cs);
}

// ---- single-table entry points: groups of one ---------------------------------------------

extern "C" size_t sc_sparse_dense_matmul_fwd_workspace_bytes(const sc_csr_t* csr) {
  if (!csr) return 0;
  float* dummy_ptrs[SC_MAX_SHARDS];
  for (int i = 0; i < SC_MAX_SHARDS; ++i) dummy_ptrs[i] = reinterpret_cast<float*>(256);
  sc_fwd_item_t item = {*csr, dummy_ptrs, reinterpret_cast<float*>(256), -1, nullptr, nullptr};
  return sc_sparse_dense_matmul_fwd_grouped_workspace_bytes(&item, 1);
}

extern "C" int32_t sc_sparse_dense_matmul_fwd(const sc_csr_t* csr, const float* const* shard_tables, float* activations,
                                              void* workspace, size_t workspace_bytes, sc_stream_t stream) {
  if (!csr) SC_FAIL(SC_INVALID_ARGUMENT, "csr descriptor is null");
  sc_fwd_item_t item = {*csr, shard_tables, activations, -1, nullptr, nullptr};
  return sc_sparse_dense_matmul_fwd_grouped(&item, 1, workspace, workspace_bytes, stream);
}

extern "C" size_t sc_sparse_dense_matmul_grad_workspace_bytes(const sc_csr_t* csr) {
  if (!csr) return 0;
  float* dummy_ptrs[SC_MAX_SHARDS];
  for (int i = 0; i < SC_MAX_SHARDS; ++i) dummy_ptrs[i] = reinterpret_cast<float*>(256);
  sc_grad_item_t item;
  memset(&item, 0, sizeof item);
  item.csr = *csr;
  item.activation_grad = reinterpret_cast<const float*>(256);
  item.shard_tables = dummy_ptrs;
  item.optimizer.clip_min = item.optimizer.clip_max = nanf("");
  return sc_sparse_dense_matmul_grad_grouped_workspace_bytes(&item, 1);
}

extern "C" int32_t sc_sparse_dense_matmul_grad(const sc_csr_t* csr, const float* activation_grad, float* const* shard_tables,
                                               float* const* shard_slot0, float* const* shard_slot1,
                                               const sc_optimizer_t* optimizer, void* workspace, size_t workspace_bytes,
                                               sc_stream_t stream) {
  if (!csr || !optimizer) SC_FAIL(SC_INVALID_ARGUMENT, "null descriptor");
  sc_grad_item_t item = {*csr, activation_grad, shard_tables, shard_slot0, shard_slot1, *optimizer};
  return sc_sparse_dense_matmul_grad_grouped(&item, 1, workspace, workspace_bytes, stream);
}

// ---- update without any allocation -----------------------------------------------------------
// Scratch of sc_sparse_dense_matmul_grad_static: one descriptor block followed by the per-chunk
// partial sums.  Every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[SC_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_static_scratch per device ordinal, resolved on first use.
void* g_static_scratch_ptr[64] = {nullptr};
std::mutex g_static_scratch_mutex;
// The documented size limit counts 512 bytes for the descriptor and 256 for the three pointers.
static_assert(sizeof(TableDesc) <= 512, "update the limit documented for sc_sparse_dense_matmul_grad_static");
constexpr size_t kStaticImageBytes = 512 + 256;

// True while `stream` records into a CUDA graph.  The descriptors of a call travel by copies from
// host memory that is gone when a graph replays, so such calls are refused.
bool stream_is_capturing(cudaStream_t stream) {
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &status) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return status != cudaStreamCaptureStatusNone;
}
}  // namespace

extern "C" int32_t sc_sparse_dense_matmul_grad_static(const sc_csr_t* csr, const float* activation_grad,
                                                      float* const* shard_tables, float* const* shard_slot0,
                                                      float* const* shard_slot1, const sc_optimizer_t* optimizer,
                                                      sc_stream_t stream) {
  if (!csr || !optimizer) SC_FAIL(SC_INVALID_ARGUMENT, "null descriptor");
  CsrView v;
  int st = make_view(csr, &v);
  if (st != SC_OK) return st;
  if (v.S != 1 || v.P != 1)
    SC_FAIL(SC_UNSUPPORTED, "the allocation-free update handles one shard and one SparseCore per buffer (got %d, %d)", v.P, v.S);
  const int kind = optimizer->optimizer;
  if (kind < 0 || kind > SC_OPT_F2A) SC_FAIL(SC_INVALID_ARGUMENT, "unknown optimizer");
  if (!activation_grad || !shard_tables || !shard_tables[0]) SC_FAIL(SC_INVALID_ARGUMENT, "null gradient or table pointer");
  const int nslots = optimizer_slots(kind);
  if (nslots >= 1 && (!shard_slot0 || !shard_slot0[0])) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 0");
  if (nslots >= 2 && (!shard_slot1 || !shard_slot1[0])) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 1");
  if (!isnan(optimizer->clip_min) && !isnan(optimizer->clip_max) && optimizer->clip_min > optimizer->clip_max)
    SC_FAIL(SC_INVALID_ARGUMENT, "min_value must be less than or equal to max_value");
  int w, k, g;
  if (!pick_group_shape(v.dim, &w, &k, &g)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the update kernel", v.dim);

  // Layout inside the static array: [TableDesc | 3 shard pointers | partial sums | group sums | chunk flags | group flags].
  const size_t image = kStaticImageBytes;
  const uint32_t chunks = (uint32_t)ceil_div(v.coo, 32);
  const size_t partial_bytes = (size_t)2 * chunks * (size_t)v.dim * sizeof(float);
  const size_t groups = update_groups(chunks);
  const size_t group_bytes = groups * (size_t)v.dim * sizeof(float);
  const size_t need = image + partial_bytes + group_bytes + chunks + groups;
  if (need > (size_t)SC_STATIC_SCRATCH_BYTES)
    SC_FAIL(SC_WORKSPACE_TOO_SMALL,
            "the allocation-free update needs %zu scratch bytes for coo_buffer_size %d and dim %d but the built-in scratch "
            "holds %d; use sc_sparse_dense_matmul_grad with a caller workspace instead", need, v.coo, v.dim,
            (int)SC_STATIC_SCRATCH_BYTES);

  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (stream_is_capturing(cs))
    SC_FAIL(SC_UNSUPPORTED, "the allocation-free update copies its descriptor from the caller's stack and cannot be recorded "
                            "into a CUDA graph");
  int dev = 0;
  SC_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) SC_FAIL(SC_UNSUPPORTED, "device ordinal %d out of range", dev);
  char* base;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
      // In host code the array name is only a handle; the kernels need its device address.
      void* ptr = nullptr;
      SC_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
      g_static_scratch_ptr[dev] = ptr;
    }
    base = static_cast<char*>(g_static_scratch_ptr[dev]);
  }
  float** pool_dev = reinterpret_cast<float**>(base + 512);
  UpdateScratch u;
  u.partial = reinterpret_cast<float*>(base + image);
  u.group_partial = reinterpret_cast<float*>(base + image + partial_bytes);
  u.flags = reinterpret_cast<uint8_t*>(base + image + partial_bytes + group_bytes);
  u.group_flags = u.flags + chunks;
  u.pstride = v.dim;

  struct { TableDesc td; } host;
  memset(&host, 0, sizeof host);
  host.td.v = v;
  host.td.grad = activation_grad;
  host.td.opt.kind = kind;
  host.td.opt.slots = nslots;
  host.td.opt.h0 = optimizer->hyper[0]; host.td.opt.h1 = optimizer->hyper[1];
  host.td.opt.h2 = optimizer->hyper[2]; host.td.opt.h3 = optimizer->hyper[3];
  host.td.opt.h4 = optimizer->hyper[4]; host.td.opt.h5 = optimizer->hyper[5];
  host.td.opt.lo = optimizer->clip_min; host.td.opt.hi = optimizer->clip_max;
  host.td.table = pool_dev;
  host.td.slot0 = nslots >= 1 ? pool_dev + 1 : nullptr;
  host.td.slot1 = nslots >= 2 ? pool_dev + 2 : nullptr;
  host.td.total_rows = (uint32_t)v.rows_per_shard;
  float* pool_host[3] = {shard_tables[0], nslots >= 1 ? shard_slot0[0] : nullptr, nslots >= 2 ? shard_slot1[0] : nullptr};
  // Both sources are pageable stack memory: the copies are staged before the calls return.
  SC_CUDA_OK(cudaMemcpyAsync(base, &host.td, sizeof(TableDesc), cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(cudaMemcpyAsync(pool_dev, pool_host, sizeof pool_host, cudaMemcpyHostToDevice, cs));
  const TableDesc* tabs = reinterpret_cast<const TableDesc*>(base);
  if (w == 4 && pipe_enabled() && aligned16(activation_grad) && aligned16(pool_host[0]) && aligned16(pool_host[1]) &&
      aligned16(pool_host[2]))
    return dispatch_bwd_pipe(tabs, 1, chunks, u, nslots, kind >= SC_OPT_ADAGRAD_MOMENTUM, v.dim, cs);
#define SC_STATIC_CALL(W, K, G) launch_bwd<W, K, G>(tabs, 1, chunks, u, nslots, cs)
  SC_SHAPE_SWITCH(w, k, g, SC_STATIC_CALL);
#undef SC_STATIC_CALL
}
