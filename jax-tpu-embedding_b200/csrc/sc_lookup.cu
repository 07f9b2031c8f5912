// Forward gather-combine and backward segment-reduce fused with SGD / Adagrad / Adam.
//
// Data layout in HBM
//   * table shards: float32 [rows_per_shard, dim] row-major, one pointer per shard;
//   * CSR-wrapped COO input of one device: row_pointers / embedding_ids / sample_ids /
//     gains exactly as the reference's preprocessing emits them (id-major: ordered by
//     source SparseCore, destination shard, row of the shard, sample);
//   * activations and activation gradients: float32 [device_batch, dim].
//
// Forward: the COO is id-major, the output is per sample.  The valid slots are
// stably radix-sorted by activation row; one warp then owns one activation row and
// sums gain * table_row over its entries in slot order (ascending shard, row), so the
// result does not depend on scheduling and every activation row is written exactly once.
//
// Backward: every table row is a contiguous run of the (id-major) entry list.  A warp
// owns 32 consecutive entries, finds the runs with one ballot, reduces each run in
// entry order and applies the optimizer with a single read-modify-write of the row and
// its slot variables.  Runs that cross a 32-entry boundary leave per-chunk partial sums
// in scratch; a second kernel adds them in chunk order and applies the update once.
// No floating-point atomics anywhere: results are bitwise reproducible.
//
// All arithmetic is float32 with separately rounded multiply and add (the file is
// compiled with -fmad=false) so that sequential sums match a float32 CPU loop.
#include <math.h>

#include "sc_common.cuh"
#include "sc_sort.cuh"

namespace sc {
namespace {

constexpr int kBlock = 256;
constexpr int kWarpsPerBlock = kBlock / 32;

struct ShardPtrs {
  float* p[SC_MAX_SHARDS];
};

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

// key = activation row of the slot (bdev for slots that hold no entry).
__global__ void fwd_keys_kernel(CsrView v, uint32_t* __restrict__ keys) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= v.coo) return;
  const int s = q / v.coo_per_sc, local = q - s * v.coo_per_sc;
  uint32_t key = (uint32_t)v.bdev;
  if (slot_shard(v, s, local) >= 0) {
    const int sid = v.sids[q];
    if (sid >= 0 && sid < v.bsc) key = (uint32_t)(s * v.bsc + sid);
  }
  keys[q] = key;
}

// offsets[r] = first sorted position whose key is >= r, for r in [0, bdev].
__global__ void fwd_offsets_kernel(const uint32_t* __restrict__ sorted_keys, int n, int bdev, int32_t* __restrict__ offsets) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  const int cur = i < n ? min((int)sorted_keys[i], bdev) : bdev;
  const int prev = i > 0 ? min((int)sorted_keys[i - 1], bdev) : -1;
  for (int r = prev + 1; r <= cur; ++r) offsets[r] = i;
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

// One warp per activation row.  K vectors of width W per lane cover the row.
template <int W, int K>
__global__ void __launch_bounds__(kBlock) fwd_gather_kernel(CsrView v, ShardPtrs shards, const int32_t* __restrict__ offsets,
                                                            const uint32_t* __restrict__ slots, float* __restrict__ act) {
  using VT = typename Vec<W>::T;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= v.bdev) return;
  const int vec_per_row = v.dim / W;
  VT acc[K];
#pragma unroll
  for (int k = 0; k < K; ++k) acc[k] = Vec<W>::zero();
  const int begin = offsets[row], end = offsets[row + 1];
  for (int base = begin; base < end; base += 32) {
    // Each lane resolves one entry; the warp then walks them in order.
    const int e = base + lane;
    int64_t my_off = -1;
    float my_gain = 0.f;
    int my_shard = 0;
    if (e < end) {
      const int q = (int)slots[e];
      const int s = q / v.coo_per_sc;
      my_shard = v.P == 1 ? 0 : slot_shard(v, s, q - s * v.coo_per_sc);
      const int id = v.ids[q];
      my_gain = v.gains[q];
      if (my_shard >= 0 && id >= 0 && (int64_t)id < v.rows_per_shard) my_off = (int64_t)id * v.dim;
    }
    const int cnt = min(32, end - base);
    for (int j = 0; j < cnt; ++j) {
      const int64_t off = __shfl_sync(0xffffffffu, my_off, j);
      const float gain = __shfl_sync(0xffffffffu, my_gain, j);
      const int g = __shfl_sync(0xffffffffu, my_shard, j);
      if (off < 0) continue;
      const VT* src = reinterpret_cast<const VT*>(shards.p[g] + off);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = lane + k * 32;
        if (c < vec_per_row) Vec<W>::axpy(acc[k], gain, __ldg(src + c));
      }
    }
  }
  VT* dst = reinterpret_cast<VT*>(act + (int64_t)row * v.dim);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + k * 32;
    if (c < vec_per_row) dst[c] = acc[k];
  }
}

// ------------------------------------------------------------------------ backward

struct OptParams {
  int kind;  // 0 sgd, 1 adagrad, 2 adam
  float h0, h1, h2, h3;
  float lo, hi;  // NaN = unbounded
};

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

struct SlotPtrs {
  ShardPtrs table, slot0, slot1;
};

template <int W, int K>
__device__ __forceinline__ void update_row(const OptParams& o, const SlotPtrs& sp, int64_t grow, int64_t rows_per_shard, int dim,
                                           int lane, const typename Vec<W>::T (&gsum)[K]) {
  using VT = typename Vec<W>::T;
  const int g = (int)(grow / rows_per_shard);
  const int64_t off = (grow - (int64_t)g * rows_per_shard) * dim;
  const int vec_per_row = dim / W;
  VT* tw = reinterpret_cast<VT*>(sp.table.p[g] + off);
  VT* t0 = o.kind >= 1 ? reinterpret_cast<VT*>(sp.slot0.p[g] + off) : nullptr;
  VT* t1 = o.kind >= 2 ? reinterpret_cast<VT*>(sp.slot1.p[g] + off) : nullptr;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + k * 32;
    if (c >= vec_per_row) continue;
    VT w = tw[c];
    VT a = t0 ? t0[c] : Vec<W>::zero();
    VT b = t1 ? t1[c] : Vec<W>::zero();
    float* wf = reinterpret_cast<float*>(&w);
    float* af = reinterpret_cast<float*>(&a);
    float* bf = reinterpret_cast<float*>(&b);
    const float* gf = reinterpret_cast<const float*>(&gsum[k]);
#pragma unroll
    for (int i = 0; i < W; ++i) wf[i] = apply_opt(o, wf[i], gf[i], af[i], bf[i]);
    tw[c] = w;
    if (t0) t0[c] = a;
    if (t1) t1[c] = b;
  }
}

// The id-major entry list seen by the backward kernels.
//   direct  : entry e is slot e of a single-partition buffer (S == 1, P == 1): row = ids[e].
//   indirect: entries were stably sorted by global row (shard * rows_per_shard + id);
//             rows[e] is the sorted key, slots[e] the slot it came from.
struct EntryList {
  const uint32_t* rows;   // indirect: sorted global rows; invalid entries hold `total_rows`
  const uint32_t* slots;  // indirect: source slot of entry e
  int indirect;
  uint32_t total_rows;    // P * rows_per_shard
};

__device__ __forceinline__ uint32_t entry_row(const CsrView& v, const EntryList& el, int e, int n) {
  if (e < 0 || e >= n) return 0xffffffffu;
  if (el.indirect) {
    const uint32_t r = el.rows[e];
    return r < el.total_rows ? r : 0xffffffffu;
  }
  const int id = v.ids[e];
  return (id >= 0 && (int64_t)id < v.rows_per_shard) ? (uint32_t)id : 0xffffffffu;
}

__device__ __forceinline__ int entry_count(const CsrView& v, const EntryList& el) {
  return el.indirect ? v.coo : min(v.row_pointers[0], v.coo_per_sc);
}

// Warp per 32 consecutive entries.  partial[(2 * chunk + k) * dim ...]: k = 0 holds the
// sum of a run that started in an earlier chunk, k = 1 of a run that continues into the next.
template <int W, int K>
__global__ void __launch_bounds__(kBlock) bwd_main_kernel(CsrView v, EntryList el, SlotPtrs sp, OptParams o,
                                                          const float* __restrict__ grad, float* __restrict__ partial) {
  using VT = typename Vec<W>::T;
  const int lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int n = entry_count(v, el);
  const int e0 = chunk * 32;
  if (e0 >= n) return;
  const int vec_per_row = v.dim / W;

  const int e = e0 + lane;
  const uint32_t my_row = entry_row(v, el, e, n);
  uint32_t prev_row = __shfl_up_sync(0xffffffffu, my_row, 1);
  if (lane == 0) prev_row = entry_row(v, el, e0 - 1, n);
  const uint32_t next_row = entry_row(v, el, e0 + 32, n);  // row after the chunk
  const bool valid = my_row != 0xffffffffu;
  int my_act = 0;
  float my_gain = 0.f;
  if (valid) {
    const int q = el.indirect ? (int)el.slots[e] : e;
    const int s = q / v.coo_per_sc;
    const int sid = v.sids[q];
    my_gain = v.gains[q];
    my_act = (sid >= 0 && sid < v.bsc) ? s * v.bsc + sid : -1;
  }
  const uint32_t heads = __ballot_sync(0xffffffffu, valid && my_row != prev_row);
  const uint32_t valids = __ballot_sync(0xffffffffu, valid);
  // Runs start at lane 0 (a continuation when lane 0 is valid but not a head) and at every head.
  uint32_t starts = heads | (valids & 1u);
  while (starts) {
    const int a = __ffs(starts) - 1;
    starts &= starts - 1;
    const int b = starts ? (__ffs(starts) - 1) : 32;  // next run start (invalid lanes never start a run)
    const uint32_t row = __shfl_sync(0xffffffffu, my_row, a);
    VT acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[k] = Vec<W>::zero();
    int last = a;
    for (int j = a; j < b; ++j) {
      const uint32_t rj = __shfl_sync(0xffffffffu, my_row, j);
      const int act = __shfl_sync(0xffffffffu, my_act, j);
      const float gain = __shfl_sync(0xffffffffu, my_gain, j);
      if (rj != row) break;  // padding lanes after the run
      last = j;
      if (act < 0) continue;
      const VT* src = reinterpret_cast<const VT*>(grad + (int64_t)act * v.dim);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int c = lane + k * 32;
        if (c < vec_per_row) Vec<W>::axpy(acc[k], gain, __ldg(src + c));
      }
    }
    const bool is_head = (heads >> a) & 1u;
    const bool continues = (last == 31) && (next_row == row);
    if (is_head && !continues) {
      update_row<W, K>(o, sp, (int64_t)row, v.rows_per_shard, v.dim, lane, acc);
    } else {
      VT* dst = reinterpret_cast<VT*>(partial + ((int64_t)2 * chunk + (is_head ? 1 : 0)) * v.dim);
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
__global__ void __launch_bounds__(kBlock) bwd_fixup_kernel(CsrView v, EntryList el, SlotPtrs sp, OptParams o,
                                                           const float* __restrict__ partial) {
  using VT = typename Vec<W>::T;
  const int lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int n = entry_count(v, el);
  const int e0 = chunk * 32;
  if (e0 + 32 >= n) return;  // nothing after this chunk
  const uint32_t row = entry_row(v, el, e0 + 31, n);
  if (row == 0xffffffffu || entry_row(v, el, e0 + 32, n) != row) return;  // last run ends here
  // The run must start inside this chunk: either it does not cover lane 0, or lane 0 is its head.
  if (entry_row(v, el, e0, n) == row && entry_row(v, el, e0 - 1, n) == row) return;
  const int vec_per_row = v.dim / W;
  VT acc[K];
  {
    const VT* src = reinterpret_cast<const VT*>(partial + ((int64_t)2 * chunk + 1) * v.dim);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      acc[k] = c < vec_per_row ? src[c] : Vec<W>::zero();
    }
  }
  for (int c2 = chunk + 1; (int64_t)c2 * 32 < n && entry_row(v, el, c2 * 32, n) == row; ++c2) {
    const VT* src = reinterpret_cast<const VT*>(partial + ((int64_t)2 * c2) * v.dim);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + k * 32;
      if (c < vec_per_row) Vec<W>::add(acc[k], src[c]);
    }
  }
  update_row<W, K>(o, sp, (int64_t)row, v.rows_per_shard, v.dim, lane, acc);
}

// key = global row (shard * rows_per_shard + id) of the slot, total_rows for empty slots.
__global__ void bwd_keys_kernel(CsrView v, uint32_t total_rows, uint32_t* __restrict__ keys) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= v.coo) return;
  const int s = q / v.coo_per_sc, local = q - s * v.coo_per_sc;
  uint32_t key = total_rows;
  const int g = slot_shard(v, s, local);
  if (g >= 0) {
    const int id = v.ids[q];
    if (id >= 0 && (int64_t)id < v.rows_per_shard) key = (uint32_t)((int64_t)g * v.rows_per_shard + id);
  }
  keys[q] = key;
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

struct FwdScratch {
  SortBuffers sort;
  int32_t* offsets;
};

bool carve_fwd(Workspace& ws, const CsrView& v, FwdScratch* s) {
  const size_t n = (size_t)v.coo;
  s->sort.keys[0] = ws.take<uint32_t>(n); s->sort.keys[1] = ws.take<uint32_t>(n);
  s->sort.vals[0] = ws.take<uint32_t>(n); s->sort.vals[1] = ws.take<uint32_t>(n);
  s->sort.hist = ws.take<uint32_t>(sort_hist_elems(n));
  s->sort.scan_temp = ws.take<uint32_t>(scan_temp_elems(sort_hist_elems(n)));
  s->offsets = ws.take<int32_t>((size_t)v.bdev + 1);
  return ws.ok();
}

struct BwdScratch {
  SortBuffers sort;
  float* partial;
};

bool carve_bwd(Workspace& ws, const CsrView& v, BwdScratch* s) {
  const size_t n = (size_t)v.coo;
  const bool indirect = !(v.S == 1 && v.P == 1);
  if (indirect) {
    s->sort.keys[0] = ws.take<uint32_t>(n); s->sort.keys[1] = ws.take<uint32_t>(n);
    s->sort.vals[0] = ws.take<uint32_t>(n); s->sort.vals[1] = ws.take<uint32_t>(n);
    s->sort.hist = ws.take<uint32_t>(sort_hist_elems(n));
    s->sort.scan_temp = ws.take<uint32_t>(scan_temp_elems(sort_hist_elems(n)));
  }
  s->partial = ws.take<float>((size_t)2 * (size_t)ceil_div((int64_t)n, 32) * (size_t)v.dim);
  return ws.ok();
}

template <int W, int K>
int launch_fwd(const CsrView& v, const ShardPtrs& sh, const int32_t* offsets, const uint32_t* slots, float* act, cudaStream_t st) {
  const unsigned blocks = (unsigned)ceil_div(v.bdev, kWarpsPerBlock);
  fwd_gather_kernel<W, K><<<blocks, kBlock, 0, st>>>(v, sh, offsets, slots, act);
  SC_LAUNCH_OK("fwd_gather_kernel");
  return SC_OK;
}

template <int W, int K>
int launch_bwd(const CsrView& v, const EntryList& el, const SlotPtrs& sp, const OptParams& o, const float* grad, float* partial,
               cudaStream_t st) {
  const unsigned blocks = (unsigned)ceil_div(ceil_div(v.coo, 32), kWarpsPerBlock);
  bwd_main_kernel<W, K><<<blocks, kBlock, 0, st>>>(v, el, sp, o, grad, partial);
  SC_LAUNCH_OK("bwd_main_kernel");
  bwd_fixup_kernel<W, K><<<blocks, kBlock, 0, st>>>(v, el, sp, o, partial);
  SC_LAUNCH_OK("bwd_fixup_kernel");
  return SC_OK;
}

#define SC_DISPATCH_SHAPE(W, K, CALL)                      \
  if (W == 4 && K == 1) return CALL<4, 1>;                 \
  if (W == 4 && K == 2) return CALL<4, 2>;                 \
  if (W == 4 && K == 4) return CALL<4, 4>;                 \
  if (W == 4 && K == 8) return CALL<4, 8>;                 \
  if (W == 1 && K == 1) return CALL<1, 1>;                 \
  if (W == 1 && K == 2) return CALL<1, 2>;                 \
  if (W == 1 && K == 4) return CALL<1, 4>;                 \
  if (W == 1 && K == 8) return CALL<1, 8>;

}  // namespace
}  // namespace sc

using namespace sc;

extern "C" size_t sc_sparse_dense_matmul_fwd_workspace_bytes(const sc_csr_t* csr) {
  CsrView v;
  if (make_view(csr, &v) != SC_OK) return 0;
  Workspace ws(nullptr, 0);
  FwdScratch s;
  carve_fwd(ws, v, &s);
  return ws.used();
}

extern "C" int32_t sc_sparse_dense_matmul_fwd(const sc_csr_t* csr, const float* const* shard_tables, float* activations,
                                              void* workspace, size_t workspace_bytes, sc_stream_t stream) {
  CsrView v;
  int st = make_view(csr, &v);
  if (st != SC_OK) return st;
  if (!shard_tables || !activations) SC_FAIL(SC_INVALID_ARGUMENT, "null table or activation pointer");
  ShardPtrs sh;
  for (int g = 0; g < v.P; ++g) {
    if (!shard_tables[g]) SC_FAIL(SC_INVALID_ARGUMENT, "shard %d has no table pointer", g);
    sh.p[g] = const_cast<float*>(shard_tables[g]);
  }
  int w, k;
  if (!pick_shape(v.dim, &w, &k)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the gather kernel", v.dim);
  Workspace ws(workspace, workspace_bytes);
  FwdScratch s;
  if (!carve_fwd(ws, v, &s)) SC_FAIL(SC_WORKSPACE_TOO_SMALL, "forward needs %zu workspace bytes, got %zu", ws.used(), workspace_bytes);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  fwd_keys_kernel<<<(unsigned)ceil_div(v.coo, kBlock), kBlock, 0, cs>>>(v, s.sort.keys[0]);
  SC_LAUNCH_OK("fwd_keys_kernel");
  int res = 0;
  SC_CUDA_OK(radix_sort_pairs(s.sort, (size_t)v.coo, bit_width_u32((uint32_t)v.bdev), true, &res, cs));
  fwd_offsets_kernel<<<(unsigned)ceil_div((int64_t)v.coo + 1, kBlock), kBlock, 0, cs>>>(s.sort.keys[res], v.coo, v.bdev, s.offsets);
  SC_LAUNCH_OK("fwd_offsets_kernel");
#define SC_FWD_CALL(W, K) launch_fwd<W, K>(v, sh, s.offsets, s.sort.vals[res], activations, cs)
  if (w == 4 && k == 1) return SC_FWD_CALL(4, 1);
  if (w == 4 && k == 2) return SC_FWD_CALL(4, 2);
  if (w == 4 && k == 4) return SC_FWD_CALL(4, 4);
  if (w == 4 && k == 8) return SC_FWD_CALL(4, 8);
  if (w == 1 && k == 1) return SC_FWD_CALL(1, 1);
  if (w == 1 && k == 2) return SC_FWD_CALL(1, 2);
  if (w == 1 && k == 4) return SC_FWD_CALL(1, 4);
  return SC_FWD_CALL(1, 8);
#undef SC_FWD_CALL
}

extern "C" size_t sc_sparse_dense_matmul_grad_workspace_bytes(const sc_csr_t* csr) {
  CsrView v;
  if (make_view(csr, &v) != SC_OK) return 0;
  Workspace ws(nullptr, 0);
  BwdScratch s;
  carve_bwd(ws, v, &s);
  return ws.used();
}

extern "C" int32_t sc_sparse_dense_matmul_grad(const sc_csr_t* csr, const float* activation_grad, float* const* shard_tables,
                                               float* const* shard_slot0, float* const* shard_slot1,
                                               const sc_optimizer_t* optimizer, void* workspace, size_t workspace_bytes,
                                               sc_stream_t stream) {
  CsrView v;
  int st = make_view(csr, &v);
  if (st != SC_OK) return st;
  if (!optimizer || optimizer->optimizer < 0 || optimizer->optimizer > 2) SC_FAIL(SC_INVALID_ARGUMENT, "unknown optimizer");
  if (!activation_grad || !shard_tables) SC_FAIL(SC_INVALID_ARGUMENT, "null gradient or table pointer");
  if (optimizer->optimizer >= 1 && !shard_slot0) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 0");
  if (optimizer->optimizer >= 2 && !shard_slot1) SC_FAIL(SC_INVALID_ARGUMENT, "optimizer needs slot variable 1");
  if (!isnan(optimizer->clip_min) && !isnan(optimizer->clip_max) && optimizer->clip_min > optimizer->clip_max)
    SC_FAIL(SC_INVALID_ARGUMENT, "min_value must be less than or equal to max_value");
  SlotPtrs sp;
  for (int g = 0; g < v.P; ++g) {
    sp.table.p[g] = shard_tables[g];
    sp.slot0.p[g] = optimizer->optimizer >= 1 ? shard_slot0[g] : nullptr;
    sp.slot1.p[g] = optimizer->optimizer >= 2 ? shard_slot1[g] : nullptr;
    if (!sp.table.p[g] || (optimizer->optimizer >= 1 && !sp.slot0.p[g]) || (optimizer->optimizer >= 2 && !sp.slot1.p[g]))
      SC_FAIL(SC_INVALID_ARGUMENT, "shard %d misses a table or slot pointer", g);
  }
  OptParams o;
  o.kind = optimizer->optimizer;
  o.h0 = optimizer->hyper[0]; o.h1 = optimizer->hyper[1]; o.h2 = optimizer->hyper[2]; o.h3 = optimizer->hyper[3];
  o.lo = optimizer->clip_min; o.hi = optimizer->clip_max;
  int w, k;
  if (!pick_shape(v.dim, &w, &k)) SC_FAIL(SC_UNSUPPORTED, "dim %d is too large for the update kernel", v.dim);
  Workspace ws(workspace, workspace_bytes);
  BwdScratch s;
  if (!carve_bwd(ws, v, &s)) SC_FAIL(SC_WORKSPACE_TOO_SMALL, "backward needs %zu workspace bytes, got %zu", ws.used(), workspace_bytes);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  EntryList el;
  el.indirect = !(v.S == 1 && v.P == 1);
  el.total_rows = (uint32_t)((int64_t)v.P * v.rows_per_shard);
  el.rows = nullptr; el.slots = nullptr;
  if (el.indirect) {
    bwd_keys_kernel<<<(unsigned)ceil_div(v.coo, kBlock), kBlock, 0, cs>>>(v, el.total_rows, s.sort.keys[0]);
    SC_LAUNCH_OK("bwd_keys_kernel");
    int res = 0;
    SC_CUDA_OK(radix_sort_pairs(s.sort, (size_t)v.coo, bit_width_u32(el.total_rows), true, &res, cs));
    el.rows = s.sort.keys[res];
    el.slots = s.sort.vals[res];
  }
#define SC_BWD_CALL(W, K) launch_bwd<W, K>(v, el, sp, o, activation_grad, s.partial, cs)
  if (w == 4 && k == 1) return SC_BWD_CALL(4, 1);
  if (w == 4 && k == 2) return SC_BWD_CALL(4, 2);
  if (w == 4 && k == 4) return SC_BWD_CALL(4, 4);
  if (w == 4 && k == 8) return SC_BWD_CALL(4, 8);
  if (w == 1 && k == 1) return SC_BWD_CALL(1, 1);
  if (w == 1 && k == 2) return SC_BWD_CALL(1, 2);
  if (w == 1 && k == 4) return SC_BWD_CALL(1, 4);
  return SC_BWD_CALL(1, 8);
#undef SC_BWD_CALL
}
