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

#include <vector>

#include "sc_common.cuh"
#include "sc_sort.cuh"

namespace sc {
namespace {

constexpr int kBlock = 256;
constexpr int kWarpsPerBlock = kBlock / 32;
constexpr uint32_t kNoRow = 0xffffffffu;

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
  int kind;  // 0 sgd, 1 adagrad, 2 adam
  float h0, h1, h2, h3;
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

// ------------------------------------------------------------------------ forward

// key = global activation row of the slot (total_act for slots that hold no entry).
__global__ void fwd_keys_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_slots, uint32_t total_act,
                                uint32_t* __restrict__ keys) {
  const uint32_t gq = blockIdx.x * blockDim.x + threadIdx.x;
  if (gq >= total_slots) return;
  const int t = find_table(count, gq, [&](int i) { return tabs[i].slot_base; });
  const CsrView& v = tabs[t].v;
  const int q = (int)(gq - tabs[t].slot_base);
  const int s = q / v.coo_per_sc, local = q - s * v.coo_per_sc;
  uint32_t key = total_act;
  if (slot_shard(v, s, local) >= 0) {
    const int sid = v.sids[q];
    if (sid >= 0 && sid < v.bsc) key = tabs[t].act_base + (uint32_t)(s * v.bsc + sid);
  }
  keys[gq] = key;
}

// offsets[r] = first sorted position whose key is >= r, for r in [0, total_act].
__global__ void fwd_offsets_kernel(const uint32_t* __restrict__ sorted_keys, uint32_t n, uint32_t total_act,
                                   uint32_t* __restrict__ offsets) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  const int64_t cur = i < n ? (int64_t)min(sorted_keys[i], total_act) : (int64_t)total_act;
  const int64_t prev = i > 0 ? (int64_t)min(sorted_keys[i - 1], total_act) : -1;
  for (int64_t r = prev + 1; r <= cur; ++r) offsets[r] = i;
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

// Resolves the sorted entry `e` of table `td`: byte-free row offset inside its shard (or -1),
// gain and shard.
__device__ __forceinline__ void resolve_entry(const TableDesc& td, const uint32_t* __restrict__ slots, uint32_t e,
                                              int64_t* off, float* gain, int* shard) {
  const CsrView& v = td.v;
  const int q = (int)(slots[e] - td.slot_base);
  const int s = q / v.coo_per_sc;
  const int g = v.P == 1 ? 0 : slot_shard(v, s, q - s * v.coo_per_sc);
  const int id = v.ids[q];
  *gain = v.gains[q];
  *shard = g;
  *off = (g >= 0 && id >= 0 && (int64_t)id < v.rows_per_shard) ? (int64_t)id * v.dim : -1;
}

// One warp per 32 consecutive global activation rows.  Lane l first resolves the range and the
// first entry of row r0 + l, so the dependent index loads of 32 rows overlap; the warp then
// walks the rows, K vectors of width W per lane covering one table row.
template <int W, int K>
__global__ void __launch_bounds__(kBlock) fwd_gather_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_act,
                                                            const uint32_t* __restrict__ offsets,
                                                            const uint32_t* __restrict__ slots) {
  using VT = typename Vec<W>::T;
  const int lane = threadIdx.x & 31;
  const uint32_t r0 = (blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5)) * 32u;
  if (r0 >= total_act) return;
  const uint32_t my_r = r0 + lane;
  uint32_t my_begin = 0, my_end = 0;
  int my_t = 0;
  int64_t first_off = -1;
  float first_gain = 0.f;
  int first_shard = 0;
  if (my_r < total_act) {
    my_begin = offsets[my_r];
    my_end = offsets[my_r + 1];
    my_t = find_table(count, my_r, [&](int i) { return tabs[i].act_base; });
    if (my_end > my_begin) resolve_entry(tabs[my_t], slots, my_begin, &first_off, &first_gain, &first_shard);
  }
  const int rows_here = (int)min(32u, total_act - r0);
  // First entry of row j, broadcast from lane j; its table row is loaded one row ahead.
  auto first_load = [&](int j, VT (&x)[K], float* gain, bool* any) {
    const int tj = __shfl_sync(0xffffffffu, my_t, j);
    const int64_t off0 = __shfl_sync(0xffffffffu, first_off, j);
    const int shard0 = __shfl_sync(0xffffffffu, first_shard, j);
    *gain = __shfl_sync(0xffffffffu, first_gain, j);
    *any = off0 >= 0;
    const TableDesc& tdj = tabs[tj];
    const int vec_per_row = tdj.v.dim / W;
    const VT* src = reinterpret_cast<const VT*>(tdj.table[max(shard0, 0)] + max(off0, (int64_t)0));
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      x[k] = (off0 >= 0 && c < vec_per_row) ? __ldg(src + c) : Vec<W>::zero();
    }
  };
  VT x_nxt[K];
  float gain_nxt;
  bool any_nxt;
  first_load(0, x_nxt, &gain_nxt, &any_nxt);
  for (int j = 0; j < rows_here; ++j) {
    const uint32_t begin = __shfl_sync(0xffffffffu, my_begin, j);
    const uint32_t end = __shfl_sync(0xffffffffu, my_end, j);
    const int t = __shfl_sync(0xffffffffu, my_t, j);
    const TableDesc& td = tabs[t];
    const int vec_per_row = td.v.dim / W;
    VT acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      acc[k] = Vec<W>::zero();
      if (any_nxt) Vec<W>::axpy(acc[k], gain_nxt, x_nxt[k]);
    }
    if (j + 1 < rows_here) first_load(j + 1, x_nxt, &gain_nxt, &any_nxt);
    for (uint32_t base = begin + 1; base < end; base += 32) {
      const uint32_t e = base + lane;
      int64_t e_off = -1;
      float e_gain = 0.f;
      int e_shard = 0;
      if (e < end) resolve_entry(td, slots, e, &e_off, &e_gain, &e_shard);
      const int cnt = (int)min(32u, end - base);
      for (int i = 0; i < cnt; ++i) {
        const int64_t off = __shfl_sync(0xffffffffu, e_off, i);
        const float gain = __shfl_sync(0xffffffffu, e_gain, i);
        const int g = __shfl_sync(0xffffffffu, e_shard, i);
        if (off < 0) continue;
        const VT* src = reinterpret_cast<const VT*>(td.table[g] + off);
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const int c = lane + k * 32;
          if (c < vec_per_row) Vec<W>::axpy(acc[k], gain, __ldg(src + c));
        }
      }
    }
    VT* dst = reinterpret_cast<VT*>(td.act + (int64_t)(r0 + j - td.act_base) * td.v.dim);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      if (c < vec_per_row) dst[c] = acc[k];
    }
  }
}

// ------------------------------------------------------------------------ backward

__device__ __forceinline__ float clip(float x, float lo, float hi) {
  if (!isnan(lo)) x = fmaxf(x, lo);
  if (!isnan(hi)) x = fminf(x, hi);
  return x;
}

// One optimizer step on one scalar; slot values are updated in place.
__device__ __forceinline__ float apply_opt(const OptParams& o, float w, float g, float& s0, float& s1) {
  float nw;
  if (o.kind == 0) {
    nw = w - o.h0 * g;
  } else if (o.kind == 1) {
    s0 = s0 + g * g;
    nw = w - (o.h0 * g) / sqrtf(s0);
  } else {
    s0 = s0 + (1.0f - o.h1) * (g - s0);
    s1 = s1 + (1.0f - o.h2) * (g * g - s1);
    nw = w - (o.h0 * s0) / (sqrtf(s1) + o.h3);
  }
  return clip(nw, o.lo, o.hi);
}

__device__ __forceinline__ int entry_count(const TableDesc& td) {
  return td.indirect ? (int)(td.range[1] - td.range[0]) : min(td.v.row_pointers[0], td.v.coo_per_sc);
}

__device__ __forceinline__ uint32_t entry_row(const TableDesc& td, int e, int n) {
  if (e < 0 || e >= n) return kNoRow;
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
  c.a0 = c.o.kind >= 1 ? td.slot0[0] : nullptr;
  c.b0 = c.o.kind >= 2 ? td.slot1[0] : nullptr;
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
  *a = c.o.kind >= 1 ? c.td->slot0[g] + off : nullptr;
  *b = c.o.kind >= 2 ? c.td->slot1[g] + off : nullptr;
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
template <int W, int K>
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
    for (int i = 0; i < W; ++i) wf[i] = apply_opt(ctx.o, wf[i], gf[i], af[i], bf[i]);
    tw[c] = w[k];
    if (t0) t0[c] = x0[k];
    if (t1) t1[c] = x1[k];
  }
}

// Variants specialised on the number of slot variables (0 sgd, 1 adagrad, 2 adam) so that the
// unused slot rows occupy no registers.
template <int W, int K, int NS>
__device__ __forceinline__ void load_row_ns(const RowCtx& ctx, int64_t grow, int lane, typename Vec<W>::T (&w)[K],
                                            typename Vec<W>::T (&x0)[NS >= 1 ? K : 1],
                                            typename Vec<W>::T (&x1)[NS >= 2 ? K : 1]) {
  using VT = typename Vec<W>::T;
  float *pw, *pa, *pb;
  row_pointers_of(ctx, grow, &pw, &pa, &pb);
  const int vec_per_row = ctx.dim / W;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + k * 32;
    const bool in = c < vec_per_row;
    w[k] = in ? reinterpret_cast<const VT*>(pw)[c] : Vec<W>::zero();
    if (NS >= 1) x0[k] = in ? reinterpret_cast<const VT*>(pa)[c] : Vec<W>::zero();
    if (NS >= 2) x1[k] = in ? reinterpret_cast<const VT*>(pb)[c] : Vec<W>::zero();
  }
}

template <int W, int K, int NS>
__device__ __forceinline__ void store_row_ns(const RowCtx& ctx, int64_t grow, int lane, const typename Vec<W>::T (&gsum)[K],
                                             typename Vec<W>::T (&w)[K], typename Vec<W>::T (&x0)[NS >= 1 ? K : 1],
                                             typename Vec<W>::T (&x1)[NS >= 2 ? K : 1]) {
  using VT = typename Vec<W>::T;
  float *pw, *pa, *pb;
  row_pointers_of(ctx, grow, &pw, &pa, &pb);
  const int vec_per_row = ctx.dim / W;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + k * 32;
    if (c >= vec_per_row) continue;
    float* wf = reinterpret_cast<float*>(&w[k]);
    float* af = NS >= 1 ? reinterpret_cast<float*>(&x0[NS >= 1 ? k : 0]) : nullptr;
    float* bf = NS >= 2 ? reinterpret_cast<float*>(&x1[NS >= 2 ? k : 0]) : nullptr;
    const float* gf = reinterpret_cast<const float*>(&gsum[k]);
    float dead0 = 0.f, dead1 = 0.f;
#pragma unroll
    for (int i = 0; i < W; ++i) wf[i] = apply_opt(ctx.o, wf[i], gf[i], NS >= 1 ? af[i] : dead0, NS >= 2 ? bf[i] : dead1);
    reinterpret_cast<VT*>(pw)[c] = w[k];
    if (NS >= 1) reinterpret_cast<VT*>(pa)[c] = x0[NS >= 1 ? k : 0];
    if (NS >= 2) reinterpret_cast<VT*>(pb)[c] = x1[NS >= 2 ? k : 0];
  }
}

// Warp per 32 consecutive entries of one table.  partial[(2 * global_chunk + k) * dim ...]:
// k = 0 holds the sum of a run that started in an earlier chunk, k = 1 of a run that continues
// into the next chunk.  The loads of run i + 1 (first gradient row, table row, slot rows) are
// issued before run i is finished, so a warp keeps two rows in flight.
template <int W, int K, int NS>
__global__ void __launch_bounds__(kBlock, K == 1 ? 3 : 1) bwd_main_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_chunks,
                                                          float* __restrict__ partial) {
  using VT = typename Vec<W>::T;
  const int lane = threadIdx.x & 31;
  const uint32_t gchunk = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (gchunk >= total_chunks) return;
  const int t = find_table(count, gchunk, [&](int i) { return tabs[i].chunk_base; });
  const TableDesc& td = tabs[t];
  const CsrView& v = td.v;
  const int n = entry_count(td);
  const int e0 = (int)(gchunk - td.chunk_base) * 32;
  if (e0 >= n) return;
  const RowCtx ctx = make_ctx(td);
  const int dim = ctx.dim;
  const int vec_per_row = dim / W;
  const float* __restrict__ grad = td.grad;

  const int e = e0 + lane;
  const uint32_t my_row = entry_row(td, e, n);
  uint32_t prev_row = __shfl_up_sync(0xffffffffu, my_row, 1);
  if (lane == 0) prev_row = entry_row(td, e0 - 1, n);
  const uint32_t next_row = entry_row(td, e0 + 32, n);  // row after the chunk
  const bool valid = my_row != kNoRow;
  const float* my_src = nullptr;  // gradient row of this lane's entry
  float my_gain = 0.f;
  if (valid) {
    const int q = td.indirect ? (int)(td.slots[td.range[0] + (uint32_t)e] - td.ent_base) : e;
    if (td.pull != nullptr) {
      const int s = q / td.pull_cap;
      const PullSrc& src = td.pull[s];
      const int slot = td.pull_begin[s] + (q - s * td.pull_cap);
      const int sid = src.sids[slot];
      my_gain = src.gains[slot];
      if (sid >= 0 && sid < v.bdev) my_src = src.grad + (int64_t)sid * dim;
    } else {
      const int s = q / v.coo_per_sc;
      const int sid = v.sids[q];
      my_gain = v.gains[q];
      if (sid >= 0 && sid < v.bsc) my_src = grad + (int64_t)(s * v.bsc + sid) * dim;
    }
  }
  const uint32_t heads = __ballot_sync(0xffffffffu, valid && my_row != prev_row);
  const uint32_t valids = __ballot_sync(0xffffffffu, valid);
  // Runs start at lane 0 (a continuation when lane 0 is valid but not a head) and at every head.
  uint32_t starts = heads | (valids & 1u);
  if (starts == 0) return;

  // Describes the run that starts at lane `a`: its row, last lane, and whether this warp owns
  // the whole row (then the optimizer is applied here, otherwise a partial sum is stored).
  struct Run { int a, last; uint32_t row; bool is_head, whole; };
  auto describe = [&](int a) {
    Run r;
    r.a = a;
    r.row = __shfl_sync(0xffffffffu, my_row, a);
    const uint32_t same = __ballot_sync(0xffffffffu, my_row == r.row) & (0xffffffffu << a);
    r.last = 31 - __clz(same);
    r.is_head = (heads >> a) & 1u;
    r.whole = r.is_head && !(r.last == 31 && next_row == r.row);
    return r;
  };
  auto load_grad = [&](int j, VT (&g)[K]) {
    const VT* src = reinterpret_cast<const VT*>(
        (const float*)__shfl_sync(0xffffffffu, (unsigned long long)my_src, j));
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      g[k] = (src != nullptr && c < vec_per_row) ? src[c] : Vec<W>::zero();
    }
  };

  constexpr int K0 = NS >= 1 ? K : 1, K1 = NS >= 2 ? K : 1;  // unused slot arrays shrink to one dead element
  VT g_nxt[K], w_nxt[K], x0_nxt[K0], x1_nxt[K1];
  Run nxt = describe(__ffs(starts) - 1);
  starts &= starts - 1;
  load_grad(nxt.a, g_nxt);
  if (nxt.whole) load_row_ns<W, K, NS>(ctx, (int64_t)nxt.row, lane, w_nxt, x0_nxt, x1_nxt);
  bool more = true;
  while (more) {
    const Run cur = nxt;
    VT g_cur[K], w_cur[K], x0_cur[K0], x1_cur[K1];
#pragma unroll
    for (int k = 0; k < K; ++k) { g_cur[k] = g_nxt[k]; w_cur[k] = w_nxt[k]; }
#pragma unroll
    for (int k = 0; k < K0; ++k) x0_cur[k] = x0_nxt[k];
#pragma unroll
    for (int k = 0; k < K1; ++k) x1_cur[k] = x1_nxt[k];
    more = starts != 0;
    if (more) {
      nxt = describe(__ffs(starts) - 1);
      starts &= starts - 1;
      load_grad(nxt.a, g_nxt);
      if (nxt.whole) load_row_ns<W, K, NS>(ctx, (int64_t)nxt.row, lane, w_nxt, x0_nxt, x1_nxt);
    }
    VT acc[K];
    const float gain_a = __shfl_sync(0xffffffffu, my_gain, cur.a);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      acc[k] = Vec<W>::zero();
      Vec<W>::axpy(acc[k], gain_a, g_cur[k]);
    }
    for (int j = cur.a + 1; j <= cur.last; ++j) {
      VT g[K];
      load_grad(j, g);
      const float gain = __shfl_sync(0xffffffffu, my_gain, j);
#pragma unroll
      for (int k = 0; k < K; ++k) Vec<W>::axpy(acc[k], gain, g[k]);
    }
    if (cur.whole) {
      store_row_ns<W, K, NS>(ctx, (int64_t)cur.row, lane, acc, w_cur, x0_cur, x1_cur);
    } else {
      VT* dst = reinterpret_cast<VT*>(partial + ((int64_t)2 * gchunk + (cur.is_head ? 1 : 0)) * dim);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = lane + k * 32;
        if (c < vec_per_row) dst[c] = acc[k];
      }
    }
  }
}

// Warp per chunk: if a run starts in this chunk and continues past it, add its partial
// sums in chunk order and apply the optimizer once.
template <int W, int K>
__global__ void __launch_bounds__(kBlock) bwd_fixup_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_chunks,
                                                           const float* __restrict__ partial) {
  using VT = typename Vec<W>::T;
  const int lane = threadIdx.x & 31;
  const uint32_t gchunk = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (gchunk >= total_chunks) return;
  const int t = find_table(count, gchunk, [&](int i) { return tabs[i].chunk_base; });
  const TableDesc& td = tabs[t];
  const int n = entry_count(td);
  const int chunk = (int)(gchunk - td.chunk_base);
  const int e0 = chunk * 32;
  if (e0 + 32 >= n) return;  // nothing after this chunk
  const uint32_t row = entry_row(td, e0 + 31, n);
  if (row == kNoRow || entry_row(td, e0 + 32, n) != row) return;  // last run ends here
  // The run must start inside this chunk: either it does not cover lane 0, or lane 0 is its head.
  if (entry_row(td, e0, n) == row && entry_row(td, e0 - 1, n) == row) return;
  const int dim = td.v.dim;
  const int vec_per_row = dim / W;
  VT acc[K];
  {
    const VT* src = reinterpret_cast<const VT*>(partial + ((int64_t)2 * gchunk + 1) * dim);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      acc[k] = c < vec_per_row ? src[c] : Vec<W>::zero();
    }
  }
  // Entries are ordered by row, so the run ends at the first entry with a larger row.
  int lo = e0 + 32, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (entry_row(td, mid, n) <= row) lo = mid + 1; else hi = mid;
  }
  const int c_end = (lo + 31) / 32;  // chunks chunk+1 .. c_end-1 hold continuation partials
  const float* pbase = partial + (int64_t)2 * td.chunk_base * dim;
  int c2 = chunk + 1;
  constexpr int U = K == 1 ? 16 : K == 2 ? 8 : K == 4 ? 4 : 2;  // partial rows in flight
  for (; c2 + U <= c_end; c2 += U) {
    VT p[U][K];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const VT* src = reinterpret_cast<const VT*>(pbase + (int64_t)2 * (c2 + u) * dim);
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
  for (; c2 < c_end; ++c2) {
    const VT* src = reinterpret_cast<const VT*>(pbase + (int64_t)2 * c2 * dim);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      if (c < vec_per_row) Vec<W>::add(acc[k], src[c]);
    }
  }
  {
    const RowCtx ctx = make_ctx(td);
    VT w[K], x0[K], x1[K];
    load_row<W, K>(ctx, (int64_t)row, lane, w, x0, x1);
    store_row<W, K>(ctx, (int64_t)row, lane, acc, w, x0, x1);
  }
}

// Entry index space of all indirect tables -> sort key (row_base + global row; `invalid` for
// indices that hold no entry).  Virtual-device tables: entry index = slot of the concatenated
// buffer.  Pull tables: entry index = source * cap + position inside the source's partition.
__global__ void bwd_keys_kernel(const TableDesc* __restrict__ tabs, int count, uint32_t total_ent, uint32_t invalid,
                                uint32_t* __restrict__ keys) {
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

// Picks the vector width and per-lane vector count for a row length.
bool pick_shape(int dim, int* w, int* k) {
  *w = (dim % 4 == 0) ? 4 : 1;
  const int vecs = dim / *w;
  const int need = (vecs + 31) / 32;
  *k = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : need <= 8 ? 8 : 0;
  return *k != 0;
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

template <int W, int K>
int launch_fwd(const TableDesc* tabs, int count, uint32_t total_act, const uint32_t* offsets, const uint32_t* slots,
               cudaStream_t st) {
  const unsigned warps = (unsigned)ceil_div(total_act, 32);
  fwd_gather_kernel<W, K><<<(unsigned)ceil_div(warps, kWarpsPerBlock), kBlock, 0, st>>>(tabs, count, total_act, offsets, slots);
  SC_LAUNCH_OK("fwd_gather_kernel");
  return SC_OK;
}

template <int W, int K>
int launch_bwd(const TableDesc* tabs, int count, uint32_t total_chunks, float* partial, int num_slots, cudaStream_t st) {
  const unsigned blocks = (unsigned)ceil_div(total_chunks, kWarpsPerBlock);
  if (num_slots == 0) bwd_main_kernel<W, K, 0><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, partial);
  else if (num_slots == 1) bwd_main_kernel<W, K, 1><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, partial);
  else bwd_main_kernel<W, K, 2><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, partial);
  SC_LAUNCH_OK("bwd_main_kernel");
  bwd_fixup_kernel<W, K><<<blocks, kBlock, 0, st>>>(tabs, count, total_chunks, partial);
  SC_LAUNCH_OK("bwd_fixup_kernel");
  return SC_OK;
}

#define SC_SHAPE_SWITCH(w, k, CALL)          \
  do {                                       \
    if (w == 4 && k == 1) return CALL(4, 1); \
    if (w == 4 && k == 2) return CALL(4, 2); \
    if (w == 4 && k == 4) return CALL(4, 4); \
    if (w == 4 && k == 8) return CALL(4, 8); \
    if (w == 1 && k == 1) return CALL(1, 1); \
    if (w == 1 && k == 2) return CALL(1, 2); \
    if (w == 1 && k == 4) return CALL(1, 4); \
    return CALL(1, 8);                       \
  } while (0)

// ---- forward group -----------------------------------------------------------------------

struct FwdPlan {
  std::vector<CsrView> views;
  uint64_t total_slots = 0, total_act = 0;
  int total_shards = 0;
  int w = 0, k = 0;
};

int plan_fwd(const sc_fwd_item_t* items, int count, FwdPlan* p) {
  if (!items || count <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "empty forward group");
  p->views.resize(count);
  for (int i = 0; i < count; ++i) {
    int st = make_view(&items[i].csr, &p->views[i]);
    if (st != SC_OK) return st;
    int w, k;
    if (!pick_shape(p->views[i].dim, &w, &k)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the gather kernel", p->views[i].dim);
    if (i == 0) { p->w = w; p->k = k; }
    if (w != p->w || k != p->k) SC_FAIL(SC_INVALID_ARGUMENT, "tables of one group must share the row length class (dim %d vs %d)",
                                       p->views[i].dim, p->views[0].dim);
    p->total_slots += (uint64_t)p->views[i].coo;
    p->total_act += (uint64_t)p->views[i].bdev;
    p->total_shards += p->views[i].P;
  }
  if (p->total_slots >= 0xffffffffull || p->total_act >= 0xffffffffull) SC_FAIL(SC_UNSUPPORTED, "group too large for 32-bit indices");
  return SC_OK;
}

struct FwdScratch {
  char* image;
  SortBuffers sort;
  uint32_t* offsets;
};

bool carve_fwd(Workspace& ws, const FwdPlan& p, int count, FwdScratch* s) {
  s->image = ws.take<char>(image_bytes(count, p.total_shards));
  carve_sort(ws, (size_t)p.total_slots, &s->sort);
  s->offsets = ws.take<uint32_t>((size_t)p.total_act + 1);
  return ws.ok();
}

// ---- backward group ----------------------------------------------------------------------

struct BwdPlan {
  std::vector<CsrView> views;
  std::vector<int> indirect;
  std::vector<uint32_t> n_ent;  // entry index space per table (0 for direct tables)
  uint64_t total_chunks = 0, total_ent = 0, total_rows = 0;
  int total_shards = 0, total_sources = 0;
  int w = 0, k = 0, max_dim = 0, max_slots = 0;
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
    int w, k;
    if (!pick_shape(v.dim, &w, &k)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the update kernel", v.dim);
    if (i == 0) { p->w = w; p->k = k; }
    if (w != p->w || k != p->k) SC_FAIL(SC_INVALID_ARGUMENT, "tables of one group must share the row length class (dim %d vs %d)",
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
    if (o.optimizer < 0 || o.optimizer > 2) SC_FAIL(SC_INVALID_ARGUMENT, "unknown optimizer");
    if (i == 0) p->max_slots = o.optimizer;
    if (o.optimizer != p->max_slots) SC_FAIL(SC_INVALID_ARGUMENT, "tables of one group must share the optimizer kind");
    if ((!pull && !items[i].activation_grad) || !items[i].shard_tables) SC_FAIL(SC_INVALID_ARGUMENT, "null gradient or table pointer");
    if (o.optimizer >= 1 && !items[i].shard_slot0) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 0");
    if (o.optimizer >= 2 && !items[i].shard_slot1) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 1");
    if (!isnan(o.clip_min) && !isnan(o.clip_max) && o.clip_min > o.clip_max)
      SC_FAIL(SC_INVALID_ARGUMENT, "min_value must be less than or equal to max_value");
  }
  if (p->total_chunks >= 0x7fffffffull || p->total_ent >= 0xffffffffull || p->total_rows >= 0xfffffffeull)
    SC_FAIL(SC_UNSUPPORTED, "group too large for 32-bit indices");
  return SC_OK;
}

struct BwdScratch {
  char* image;
  SortBuffers sort;  // one sorted list for all indirect tables
  uint32_t* ranges;
  PullSrc* pull;
  int32_t* pull_begin;
  float* partial;
};

bool carve_bwd(Workspace& ws, const BwdPlan& p, int count, BwdScratch* s) {
  s->image = ws.take<char>(image_bytes(count, p.total_shards));
  if (p.total_ent > 0) carve_sort(ws, (size_t)p.total_ent, &s->sort);
  s->ranges = ws.take<uint32_t>((size_t)count + 1);
  s->pull = ws.take<PullSrc>((size_t)p.total_sources + 1);
  s->pull_begin = ws.take<int32_t>((size_t)p.total_sources + 1);
  s->partial = ws.take<float>((size_t)2 * (size_t)p.total_chunks * (size_t)p.max_dim);
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
  for (int i = 0; i < count; ++i) {
    if (!items[i].shard_tables || !items[i].activations) SC_FAIL(SC_INVALID_ARGUMENT, "null table or activation pointer");
    TableDesc td;
    memset(&td, 0, sizeof td);
    td.v = p.views[i];
    td.act = items[i].activations;
    td.slot_base = slot_base; td.act_base = act_base;
    slot_base += (uint32_t)td.v.coo; act_base += (uint32_t)td.v.bdev;
    pool_index.push_back((int)img.pool.size()); pool_index.push_back(-1); pool_index.push_back(-1);
    for (int g = 0; g < td.v.P; ++g) {
      if (!items[i].shard_tables[g]) SC_FAIL(SC_INVALID_ARGUMENT, "shard %d has no table pointer", g);
      img.pool.push_back(const_cast<float*>(items[i].shard_tables[g]));
    }
    img.tabs.push_back(td);
  }
  SC_CUDA_OK(upload(img, s.image, pool_index, cs));
  const TableDesc* tabs = reinterpret_cast<const TableDesc*>(s.image);
  const uint32_t total_slots = (uint32_t)p.total_slots, total_act = (uint32_t)p.total_act;

  fwd_keys_kernel<<<(unsigned)ceil_div(total_slots, kBlock), kBlock, 0, cs>>>(tabs, count, total_slots, total_act, s.sort.keys[0]);
  SC_LAUNCH_OK("fwd_keys_kernel");
  int res = 0;
  SC_CUDA_OK(radix_sort_pairs(s.sort, (size_t)total_slots, bit_width_u32(total_act), true, &res, cs));
  fwd_offsets_kernel<<<(unsigned)ceil_div((int64_t)total_slots + 1, kBlock), kBlock, 0, cs>>>(s.sort.keys[res], total_slots, total_act,
                                                                                           s.offsets);
  SC_LAUNCH_OK("fwd_offsets_kernel");
#define SC_FWD_CALL(W, K) launch_fwd<W, K>(tabs, count, total_act, s.offsets, s.sort.vals[res], cs)
  SC_SHAPE_SWITCH(p.w, p.k, SC_FWD_CALL);
#undef SC_FWD_CALL
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
  uint32_t chunk_base = 0, ent_base = 0, row_base = 0;
  int source_base = 0;
  for (int i = 0; i < count; ++i) {
    const sc_optimizer_t& o = items[i].optimizer;
    const bool pull = items[i].sources != nullptr;
    TableDesc td;
    memset(&td, 0, sizeof td);
    td.v = p.views[i];
    td.grad = items[i].activation_grad;
    td.opt.kind = o.optimizer;
    td.opt.h0 = o.hyper[0]; td.opt.h1 = o.hyper[1]; td.opt.h2 = o.hyper[2]; td.opt.h3 = o.hyper[3];
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
      td.pull_begin = s.pull_begin + source_base;
      td.pull_cap = items[i].partition_capacity;
      td.pull_shard = items[i].shard;
      td.num_sources = items[i].num_sources;
      for (int sidx = 0; sidx < items[i].num_sources; ++sidx) {
        const sc_pull_source_t& src = items[i].sources[sidx];
        pull_host.push_back(PullSrc{src.row_pointers, src.embedding_ids, src.sample_ids, src.gains, src.activation_grad});
      }
      source_base += items[i].num_sources;
      td.v.P = 1;  // row -> pointer arithmetic of the update sees the owned shard only
    }
    float* const* srcs[3] = {items[i].shard_tables, o.optimizer >= 1 ? items[i].shard_slot0 : nullptr,
                             o.optimizer >= 2 ? items[i].shard_slot1 : nullptr};
    for (int a = 0; a < 3; ++a) {
      if (!srcs[a]) { pool_index.push_back(-1); continue; }
      pool_index.push_back((int)img.pool.size());
      for (int g = 0; g < table_shards; ++g) {
        if (!srcs[a][g]) SC_FAIL(SC_INVALID_ARGUMENT, "shard %d misses a table or slot pointer", g);
        img.pool.push_back(srcs[a][g]);
      }
    }
    img.tabs.push_back(td);
  }
  const uint32_t total_ent = (uint32_t)p.total_ent, invalid = (uint32_t)p.total_rows;
  if (total_ent > 0) {
    // The sorted list lives in one of the two sort buffers; which one is known before launching.
    const int passes = (bit_width_u32(invalid) + kRadixBits - 1) / kRadixBits;
    const int res_index = passes & 1;
    for (auto& td : img.tabs) {
      td.rows = s.sort.keys[res_index];
      td.slots = s.sort.vals[res_index];
    }
  }
  if (!pull_host.empty())
    SC_CUDA_OK(cudaMemcpyAsync(s.pull, pull_host.data(), pull_host.size() * sizeof(PullSrc), cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(upload(img, s.image, pool_index, cs));
  const TableDesc* tabs = reinterpret_cast<const TableDesc*>(s.image);
  if (total_ent > 0) {
    // Entries of several SparseCores / shards / devices: order them by global row first (stable,
    // so contributions to one row keep the order source, sample), one sort for all tables.
    bwd_keys_kernel<<<(unsigned)ceil_div(total_ent, kBlock), kBlock, 0, cs>>>(tabs, count, total_ent, invalid, s.sort.keys[0]);
    SC_LAUNCH_OK("bwd_keys_kernel");
    int res = 0;
    SC_CUDA_OK(radix_sort_pairs(s.sort, (size_t)total_ent, bit_width_u32(invalid), true, &res, cs));
    const int passes = (bit_width_u32(invalid) + kRadixBits - 1) / kRadixBits;
    if (res != (passes & 1)) SC_FAIL(SC_CUDA_ERROR, "internal: unexpected sort buffer parity");
    bwd_ranges_kernel<<<(unsigned)ceil_div(count + 1, kBlock), kBlock, 0, cs>>>(tabs, count, s.sort.keys[res], total_ent, invalid,
                                                                              s.ranges);
    SC_LAUNCH_OK("bwd_ranges_kernel");
  }
  const uint32_t total_chunks = (uint32_t)p.total_chunks;
#define SC_BWD_CALL(W, K) launch_bwd<W, K>(tabs, count, total_chunks, s.partial, p.max_slots, cs)
  SC_SHAPE_SWITCH(p.w, p.k, SC_BWD_CALL);
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

// Copies this device's CSR buffers and activation gradients of every pull-mode item into the
// device's own peer-visible exchange buffers (sources[shard]) with ONE kernel launch; buffers
// that already live there (same address) are skipped.  `workspace` holds the job list
// (sc_sparse_dense_matmul_grad_grouped_workspace_bytes covers it).  The caller separates this
// call from the update with a barrier across the devices.
extern "C" int32_t sc_sparse_dense_matmul_grad_stage(const sc_grad_item_t* items, int32_t count, void* workspace,
                                                     size_t workspace_bytes, sc_stream_t stream) {
  if (!items || count <= 0) SC_FAIL(SC_INVALID_ARGUMENT, "empty backward group");
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  std::vector<CopyJob> jobs;
  for (int i = 0; i < count; ++i) {
    const sc_grad_item_t& it = items[i];
    if (!it.sources) continue;
    CsrView v;
    int st = make_view(&it.csr, &v);
    if (st != SC_OK) return st;
    if (it.shard < 0 || it.shard >= it.num_sources || !it.activation_grad) SC_FAIL(SC_INVALID_ARGUMENT, "bad pull item");
    const sc_pull_source_t& own = it.sources[it.shard];
    const void* srcs[5] = {v.row_pointers, v.ids, v.sids, v.gains, it.activation_grad};
    const void* dsts[5] = {own.row_pointers, own.embedding_ids, own.sample_ids, own.gains, own.activation_grad};
    const uint64_t words[5] = {(uint64_t)v.R * v.S, (uint64_t)v.coo, (uint64_t)v.coo, (uint64_t)v.coo,
                               (uint64_t)v.bdev * v.dim};
    for (int a = 0; a < 5; ++a) {
      if (srcs[a] == dsts[a] || words[a] == 0) continue;
      jobs.push_back(CopyJob{static_cast<const uint32_t*>(srcs[a]),
                             const_cast<uint32_t*>(static_cast<const uint32_t*>(dsts[a])), words[a]});
    }
  }
  if (jobs.empty()) return SC_OK;
  const size_t bytes = jobs.size() * sizeof(CopyJob);
  if (!workspace || workspace_bytes < bytes) SC_FAIL(SC_WORKSPACE_TOO_SMALL, "staging needs %zu workspace bytes", bytes);
  SC_CUDA_OK(cudaMemcpyAsync(workspace, jobs.data(), bytes, cudaMemcpyHostToDevice, cs));
  dim3 grid(32, (unsigned)jobs.size());
  stage_copy_kernel<<<grid, kBlock, 0, cs>>>(static_cast<const CopyJob*>(workspace));
  SC_LAUNCH_OK("stage_copy_kernel");
  return SC_OK;
}

// ---- single-table entry points: groups of one ---------------------------------------------

extern "C" size_t sc_sparse_dense_matmul_fwd_workspace_bytes(const sc_csr_t* csr) {
  if (!csr) return 0;
  float* dummy_ptrs[SC_MAX_SHARDS];
  for (int i = 0; i < SC_MAX_SHARDS; ++i) dummy_ptrs[i] = reinterpret_cast<float*>(256);
  sc_fwd_item_t item = {*csr, dummy_ptrs, reinterpret_cast<float*>(256)};
  return sc_sparse_dense_matmul_fwd_grouped_workspace_bytes(&item, 1);
}

extern "C" int32_t sc_sparse_dense_matmul_fwd(const sc_csr_t* csr, const float* const* shard_tables, float* activations,
                                              void* workspace, size_t workspace_bytes, sc_stream_t stream) {
  if (!csr) SC_FAIL(SC_INVALID_ARGUMENT, "csr descriptor is null");
  sc_fwd_item_t item = {*csr, shard_tables, activations};
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
  if (kind < 0 || kind > 2) SC_FAIL(SC_INVALID_ARGUMENT, "unknown optimizer");
  if (!activation_grad || !shard_tables || !shard_tables[0]) SC_FAIL(SC_INVALID_ARGUMENT, "null gradient or table pointer");
  if (kind >= 1 && (!shard_slot0 || !shard_slot0[0])) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 0");
  if (kind >= 2 && (!shard_slot1 || !shard_slot1[0])) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 1");
  if (!isnan(optimizer->clip_min) && !isnan(optimizer->clip_max) && optimizer->clip_min > optimizer->clip_max)
    SC_FAIL(SC_INVALID_ARGUMENT, "min_value must be less than or equal to max_value");
  int w, k;
  if (!pick_shape(v.dim, &w, &k)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the update kernel", v.dim);

  // Layout inside the static array: [TableDesc | 3 shard pointers | partial sums].
  const size_t image = align_up(sizeof(TableDesc), 256) + align_up(3 * sizeof(float*), 256);
  const uint32_t chunks = (uint32_t)ceil_div(v.coo, 32);
  const size_t need = image + (size_t)2 * chunks * (size_t)v.dim * sizeof(float);
  if (need > (size_t)SC_STATIC_SCRATCH_BYTES)
    SC_FAIL(SC_WORKSPACE_TOO_SMALL,
            "the allocation-free update needs %zu scratch bytes for coo_buffer_size %d and dim %d but the built-in scratch "
            "holds %d; use sc_sparse_dense_matmul_grad with a caller workspace instead", need, v.coo, v.dim,
            (int)SC_STATIC_SCRATCH_BYTES);

  int dev = 0;
  SC_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) SC_FAIL(SC_UNSUPPORTED, "device ordinal %d out of range", dev);
  if (g_static_scratch_ptr[dev] == nullptr) {
    // In host code the array name is only a handle; the kernels need its device address.
    void* ptr = nullptr;
    SC_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    g_static_scratch_ptr[dev] = ptr;
  }
  char* base = static_cast<char*>(g_static_scratch_ptr[dev]);
  float** pool_dev = reinterpret_cast<float**>(base + align_up(sizeof(TableDesc), 256));
  float* partial = reinterpret_cast<float*>(base + image);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  struct { TableDesc td; } host;
  memset(&host, 0, sizeof host);
  host.td.v = v;
  host.td.grad = activation_grad;
  host.td.opt.kind = kind;
  host.td.opt.h0 = optimizer->hyper[0]; host.td.opt.h1 = optimizer->hyper[1];
  host.td.opt.h2 = optimizer->hyper[2]; host.td.opt.h3 = optimizer->hyper[3];
  host.td.opt.lo = optimizer->clip_min; host.td.opt.hi = optimizer->clip_max;
  host.td.table = pool_dev;
  host.td.slot0 = kind >= 1 ? pool_dev + 1 : nullptr;
  host.td.slot1 = kind >= 2 ? pool_dev + 2 : nullptr;
  host.td.total_rows = (uint32_t)v.rows_per_shard;
  float* pool_host[3] = {shard_tables[0], kind >= 1 ? shard_slot0[0] : nullptr, kind >= 2 ? shard_slot1[0] : nullptr};
  // Both sources are pageable stack memory: the copies are staged before the calls return.
  SC_CUDA_OK(cudaMemcpyAsync(base, &host.td, sizeof(TableDesc), cudaMemcpyHostToDevice, cs));
  SC_CUDA_OK(cudaMemcpyAsync(pool_dev, pool_host, sizeof pool_host, cudaMemcpyHostToDevice, cs));
  const TableDesc* tabs = reinterpret_cast<const TableDesc*>(base);
#define SC_STATIC_CALL(W, K) launch_bwd<W, K>(tabs, 1, chunks, partial, kind, cs)
  SC_SHAPE_SWITCH(w, k, SC_STATIC_CALL);
#undef SC_STATIC_CALL
}
