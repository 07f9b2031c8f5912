// Device-wide exclusive scan and stable LSD radix sort (32-bit keys, 32-bit payload).
//
// Both are written for HBM-bound integer work on B200: every pass streams its input
// with fully coalesced loads, ranks keys inside a 4096-key tile with warp match
// instructions, reorders the tile in shared memory and writes digit runs contiguously.
// Nothing here allocates; temporary storage is carved by the caller.
#ifndef SC_SORT_CUH_
#define SC_SORT_CUH_

#include "sc_common.cuh"

namespace sc {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 16;
constexpr int kScanTile = kScanThreads * kScanItems;  // 4096

// ----------------------------------------------------------------------------- scan

template <typename T>
__device__ __forceinline__ T warp_inclusive_scan(T v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    T o = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += o;
  }
  return v;
}

// Exclusive scan of one value per thread across a 256-thread block; returns the
// exclusive prefix and stores the block total in *total (valid for all threads).
template <typename T>
__device__ __forceinline__ T block_exclusive_scan(T v, T* total) {
  __shared__ T warp_sums[kScanThreads / 32];
  __shared__ T block_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T inc = warp_inclusive_scan(v, lane);
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    T w = lane < kScanThreads / 32 ? warp_sums[lane] : T(0);
    T winc = warp_inclusive_scan(w, lane);
    if (lane < kScanThreads / 32) warp_sums[lane] = winc - w;
    if (lane == kScanThreads / 32 - 1) block_total = winc;
  }
  __syncthreads();
  T res = warp_sums[warp] + inc - v;
  *total = block_total;
  __syncthreads();
  return res;
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads) scan_reduce_kernel(const T* __restrict__ in, T* __restrict__ sums, size_t n) {
  const size_t base = (size_t)blockIdx.x * kScanTile;
  T acc = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    size_t idx = base + (size_t)i * kScanThreads + threadIdx.x;
    if (idx < n) acc += in[idx];
  }
  T total;
  block_exclusive_scan(acc, &total);
  if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

// Scans one tile per block; adds offsets[blockIdx.x] when offsets != nullptr.
// When total_out != nullptr (single-block use) the grand total is stored there.
template <typename T>
__global__ void __launch_bounds__(kScanThreads) scan_tile_kernel(const T* in, T* out, size_t n, const T* __restrict__ offsets,
                                                                 T* total_out) {
  const size_t base = (size_t)blockIdx.x * kScanTile + (size_t)threadIdx.x * kScanItems;
  T v[kScanItems];
  T acc = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    v[i] = (base + i < n) ? in[base + i] : T(0);
    acc += v[i];
  }
  T total;
  T prefix = block_exclusive_scan(acc, &total);
  if (offsets != nullptr) prefix += offsets[blockIdx.x];
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (base + i < n) out[base + i] = prefix;
    prefix += v[i];
  }
  if (total_out != nullptr && threadIdx.x == 0) *total_out = total;
}

inline size_t scan_temp_elems(size_t n) {
  size_t total = 0;
  while (n > (size_t)kScanTile) {
    n = (size_t)ceil_div((int64_t)n, kScanTile);
    total += align_up(n, 64);
  }
  return total + 64;
}

// out[i] = sum(in[0..i)); in may alias out.  `temp` holds scan_temp_elems(n) values.
// If total_out != nullptr it receives the sum of all n inputs (device memory).
template <typename T>
inline cudaError_t exclusive_scan(const T* in, T* out, size_t n, T* temp, T* total_out, cudaStream_t stream) {
  if (n == 0) {
    if (total_out) return cudaMemsetAsync(total_out, 0, sizeof(T), stream);
    return cudaSuccess;
  }
  const size_t tiles = (size_t)ceil_div((int64_t)n, kScanTile);
  if (tiles == 1) {
    scan_tile_kernel<T><<<1, kScanThreads, 0, stream>>>(in, out, n, nullptr, total_out);
    count_launch();
    return cudaGetLastError();
  }
  T* sums = temp;
  scan_reduce_kernel<T><<<(unsigned)tiles, kScanThreads, 0, stream>>>(in, sums, n);
  count_launch(2);  // this kernel and the tile scan below
  cudaError_t err = exclusive_scan<T>(sums, sums, tiles, temp + align_up(tiles, 64), total_out, stream);
  if (err != cudaSuccess) return err;
  scan_tile_kernel<T><<<(unsigned)tiles, kScanThreads, 0, stream>>>(in, out, n, sums, nullptr);
  return cudaGetLastError();
}

// ----------------------------------------------------------------------------- radix sort

constexpr int kSortThreads = 256;
constexpr int kSortItems = 16;
constexpr int kSortTile = kSortThreads * kSortItems;  // 4096
constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;

// hist[digit * tiles + tile] = number of keys of `tile` whose digit is `digit`.
static __global__ void __launch_bounds__(kSortThreads) radix_hist_kernel(const uint32_t* __restrict__ keys, uint32_t* __restrict__ hist, size_t n,
                                                                  int shift, uint32_t digit_mask, uint32_t tiles) {
  __shared__ uint32_t bins[kRadix];
  bins[threadIdx.x] = 0;
  __syncthreads();
  const size_t base = (size_t)blockIdx.x * kSortTile;
#pragma unroll
  for (int i = 0; i < kSortItems; ++i) {
    size_t idx = base + (size_t)i * kSortThreads + threadIdx.x;
    if (idx < n) atomicAdd(&bins[(keys[idx] >> shift) & digit_mask], 1u);
  }
  __syncthreads();
  hist[(size_t)threadIdx.x * tiles + blockIdx.x] = bins[threadIdx.x];
}

// hist is [digit][tile].  Block d turns row d into its exclusive prefix over the tiles and stores the row's total
// in totals[d]: together with an exclusive scan of the 256 totals (done by every scatter block for itself) that is
// the position of each (digit, tile) run in the output, in two launches per pass instead of a device-wide scan.
static __global__ void __launch_bounds__(kScanThreads) radix_rowscan_kernel(uint32_t* __restrict__ hist, uint32_t tiles,
                                                                            uint32_t* __restrict__ totals) {
  __shared__ uint32_t s_carry;
  uint32_t* row = hist + (size_t)blockIdx.x * tiles;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (uint32_t base = 0; base < tiles; base += kScanTile) {
    const uint32_t first = base + threadIdx.x * kScanItems;
    uint32_t v[kScanItems];
    uint32_t sum = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
      v[i] = first + i < tiles ? row[first + i] : 0u;
      sum += v[i];
    }
    uint32_t total;
    uint32_t prefix = block_exclusive_scan<uint32_t>(sum, &total) + s_carry;
#pragma unroll
    for (int i = 0; i < kScanItems; ++i) {
      if (first + i < tiles) row[first + i] = prefix;
      prefix += v[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) s_carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = s_carry;
}

// Stable scatter of one tile.  Warp w owns the contiguous span [w*512, (w+1)*512) of
// the tile and visits it in 16 rounds of 32 consecutive keys, so ranks follow input
// order.  vals_in == nullptr means "payload = input index".
static __global__ void __launch_bounds__(kSortThreads) radix_scatter_kernel(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                                                                     uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                                                                     const uint32_t* __restrict__ offsets,
                                                                     const uint32_t* __restrict__ totals, size_t n, int shift,
                                                                     uint32_t digit_mask, uint32_t tiles) {
  constexpr int kWarps = kSortThreads / 32;
  __shared__ uint32_t warp_cnt[kWarps][kRadix];
  __shared__ uint32_t digit_start[kRadix];
  __shared__ uint32_t digit_base[kRadix];  // keys of all tiles with a smaller digit
  __shared__ uint32_t s_keys[kSortTile];
  __shared__ uint32_t s_vals[kSortTile];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t tile_base = (size_t)blockIdx.x * kSortTile;
  const uint32_t tile_count = (uint32_t)min((size_t)kSortTile, n - tile_base);
  for (int i = threadIdx.x; i < kWarps * kRadix; i += kSortThreads) (&warp_cnt[0][0])[i] = 0;
  __syncthreads();

  uint32_t key[kSortItems], val[kSortItems], rank[kSortItems];
  const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const uint32_t local = (uint32_t)warp * (32 * kSortItems) + (uint32_t)r * 32 + lane;
    const bool valid = local < tile_count;
    key[r] = valid ? keys_in[tile_base + local] : 0u;
    val[r] = valid ? (vals_in ? vals_in[tile_base + local] : (uint32_t)(tile_base + local)) : 0u;
    const uint32_t d = (key[r] >> shift) & digit_mask;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? d : (0x10000u | lane));
    const uint32_t before = valid ? warp_cnt[warp][d] : 0u;
    rank[r] = before + __popc(peers & lt_mask);
    __syncwarp();
    if (valid && (peers & lt_mask) == 0) warp_cnt[warp][d] = before + __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  // Per digit: exclusive prefix over warps, then exclusive prefix over digits.
  {
    const int d = threadIdx.x;
    uint32_t run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      uint32_t c = warp_cnt[w][d];
      warp_cnt[w][d] = run;
      run += c;
    }
    uint32_t total;
    uint32_t start = block_exclusive_scan<uint32_t>(run, &total);
    digit_start[d] = start;
    digit_base[d] = block_exclusive_scan<uint32_t>(totals[d], &total);
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const uint32_t local = (uint32_t)warp * (32 * kSortItems) + (uint32_t)r * 32 + lane;
    if (local < tile_count) {
      const uint32_t d = (key[r] >> shift) & digit_mask;
      const uint32_t pos = digit_start[d] + warp_cnt[warp][d] + rank[r];
      s_keys[pos] = key[r];
      s_vals[pos] = val[r];
    }
  }
  __syncthreads();
  for (uint32_t j = threadIdx.x; j < tile_count; j += kSortThreads) {
    const uint32_t k = s_keys[j];
    const uint32_t d = (k >> shift) & digit_mask;
    const size_t dst = (size_t)digit_base[d] + offsets[(size_t)d * tiles + blockIdx.x] + (j - digit_start[d]);
    keys_out[dst] = k;
    vals_out[dst] = s_vals[j];
  }
}

struct SortBuffers {
  uint32_t* keys[2];
  uint32_t* vals[2];
  uint32_t* hist;       // kRadix * tiles
  uint32_t* scan_temp;  // scan_temp_elems(kRadix * tiles)
};

inline size_t sort_tiles(size_t n) { return (size_t)ceil_div((int64_t)(n ? n : 1), kSortTile); }
inline size_t sort_hist_elems(size_t n) { return (size_t)kRadix * sort_tiles(n) + kRadix; }  // + the digit totals

// Sorts (keys[0], vals[0]) ascending by the low `bits` bits of the key, stably.
// vals[0] may be nullptr on entry only through `iota_payload` (payload = position).
// Returns the index (0 or 1) of the buffer pair that holds the result.
inline cudaError_t radix_sort_pairs(SortBuffers& b, size_t n, int bits, bool iota_payload, int* result_index,
                                    cudaStream_t stream) {
  int cur = 0;
  if (bits <= 0 || n == 0) {
    // A zero-bit sort still has to materialise the payload when it was implicit.
    bits = (iota_payload && n > 0) ? 1 : 0;
  }
  const uint32_t tiles = (uint32_t)sort_tiles(n);
  const int passes = (bits + kRadixBits - 1) / kRadixBits;
  for (int p = 0; p < passes; ++p) {
    const int shift = p * kRadixBits;
    const int pass_bits = min(kRadixBits, bits - shift);
    const uint32_t mask = (1u << pass_bits) - 1u;
    radix_hist_kernel<<<tiles, kSortThreads, 0, stream>>>(b.keys[cur], b.hist, n, shift, mask, tiles);
    count_launch(2);  // histogram and scatter of this pass
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    uint32_t* totals = b.hist + (size_t)kRadix * tiles;
    radix_rowscan_kernel<<<kRadix, kScanThreads, 0, stream>>>(b.hist, tiles, totals);
    count_launch();
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    const uint32_t* vin = (p == 0 && iota_payload) ? nullptr : b.vals[cur];
    radix_scatter_kernel<<<tiles, kSortThreads, 0, stream>>>(b.keys[cur], vin, b.keys[cur ^ 1], b.vals[cur ^ 1], b.hist, totals, n,
                                                             shift, mask, tiles);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    cur ^= 1;
  }
  *result_index = cur;
  return cudaSuccess;
}

}  // namespace sc
#endif  // SC_SORT_CUH_
