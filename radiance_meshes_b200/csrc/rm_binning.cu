// Stages 2-4 on the GPU: per-tile tet lists ordered by (depth bits, tet id).
//
// The reference emits one 64-bit key per (tile, tet) pair, sorts all N pairs
// with a 7-pass LSD radix sort and then searches the sorted keys for tile
// boundaries (slang/tile_shader.slang:49-125, sort_by_keys/sort_by_keys.cu:9-53,
// tile_shader_slang.py:36-69).  The sort depth is a per-tet quantity, so the
// same order is produced here with far less traffic:
//
//   1. rank the T tets by (depth bits, tet id) with a 4-pass LSD radix sort of
//      32-bit keys (T elements, not N);
//   2. tile populations come from a 2-D difference array (4 atomics per tet,
//      written by the projection kernel) and two prefix passes; an exclusive
//      scan turns them into tile_ranges directly;
//   3. every (tile, tet) pair writes the tet's 32-bit RANK into its tile's
//      segment (load-balanced over pairs, slot taken with one atomic);
//   4. each tile segment is sorted by rank in shared memory and mapped back to
//      tet ids.
//
// Ascending rank inside a tile is ascending (depth bits, tet id), which is what
// the reference's stable sort produces because it emits pairs in tet order.

#include "rm_common.cuh"

namespace rm {

// ---------------------------------------------------------------------------
// Device-wide exclusive scan of uint32 (three launches: block sums, scan of the
// block sums, apply).  Optional gather: element i is in[gather[i]].
// ---------------------------------------------------------------------------
constexpr int kScanThreads = 256;
constexpr int kScanItems = 16;
constexpr int kScanTile = kScanThreads * kScanItems;

__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t n = __shfl_up_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) >= o) v += n;
  }
  return v;
}

// exclusive scan across the block of one value per thread; returns exclusive prefix, total in *total
template <int THREADS>
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* total, uint32_t* smem /* THREADS/32 + 1 */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = warp_inclusive_scan(v);
  if (lane == 31) smem[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = lane < THREADS / 32 ? smem[lane] : 0;
    uint32_t winc = warp_inclusive_scan(w);
    if (lane < THREADS / 32) smem[lane] = winc - w;
    if (lane == THREADS / 32 - 1) smem[THREADS / 32] = winc;
  }
  __syncthreads();
  uint32_t r = inc - v + smem[warp];
  *total = smem[THREADS / 32];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(kScanThreads)
k_scan_block_sums(const uint32_t* __restrict__ in, const uint32_t* __restrict__ gather, int64_t n,
                  uint32_t* __restrict__ bsum) {
  __shared__ uint32_t sm[kScanThreads / 32 + 1];
  int64_t base = (int64_t)blockIdx.x * kScanTile;
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    int64_t i = base + k * kScanThreads + threadIdx.x;
    if (i < n) s += gather ? in[gather[i]] : in[i];
  }
  uint32_t total;
  block_exclusive_scan<kScanThreads>(s, &total, sm);
  if (threadIdx.x == 0) bsum[blockIdx.x] = total;
}

// single block: exclusive scan of bsum[0..nb) in place; grand total (64-bit) to *total64
__global__ void __launch_bounds__(1024) k_scan_sums(uint32_t* __restrict__ bsum, int64_t nb, unsigned long long* total64) {
  __shared__ uint32_t sm[1024 / 32 + 1];
  unsigned long long carry = 0;
  for (int64_t base = 0; base < nb; base += 1024) {
    int64_t i = base + threadIdx.x;
    uint32_t v = i < nb ? bsum[i] : 0;
    uint32_t total;
    uint32_t ex = block_exclusive_scan<1024>(v, &total, sm);
    if (i < nb) bsum[i] = (uint32_t)(carry + ex);
    carry += total;
  }
  if (threadIdx.x == 0 && total64) *total64 = carry;
}

// inclusive = true writes the inclusive scan instead
__global__ void __launch_bounds__(kScanThreads)
k_scan_apply(const uint32_t* __restrict__ in, const uint32_t* __restrict__ gather, int64_t n,
             const uint32_t* __restrict__ bsum, uint32_t* __restrict__ out, int inclusive) {
  __shared__ uint32_t sm[kScanThreads / 32 + 1];
  // blocked arrangement: thread t owns items [t*kScanItems, (t+1)*kScanItems)
  int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    int64_t i = base + k;
    v[k] = i < n ? (gather ? in[gather[i]] : in[i]) : 0;
    s += v[k];
  }
  uint32_t total;
  uint32_t ex = block_exclusive_scan<kScanThreads>(s, &total, sm) + bsum[blockIdx.x];
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    int64_t i = base + k;
    uint32_t o = inclusive ? ex + v[k] : ex;
    if (i < n) out[i] = o;
    ex += v[k];
  }
}

// ---------------------------------------------------------------------------
// LSD radix sort of (uint32 key, uint32 value) pairs, 8 bits per pass, stable.
// Per pass: block histograms -> per-digit row scan -> stable scatter.
// ---------------------------------------------------------------------------
constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kSortThreads = 256;
constexpr int kSortItems = 16;  // keys per thread
constexpr int kSortTile = kSortThreads * kSortItems;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kWarpSpan = 32 * kSortItems;  // consecutive keys owned by one warp

__global__ void __launch_bounds__(kSortThreads)
k_radix_hist(const uint32_t* __restrict__ keys, int64_t n, int shift, uint32_t* __restrict__ hist, int nblk) {
  __shared__ uint32_t h[kRadix];
  for (int i = threadIdx.x; i < kRadix; i += kSortThreads) h[i] = 0;
  __syncthreads();
  int64_t base = (int64_t)blockIdx.x * kSortTile;
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    int64_t i = base + k * kSortThreads + threadIdx.x;
    if (i < n) atomicAdd(&h[(keys[i] >> shift) & (kRadix - 1)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kRadix; i += kSortThreads) hist[(int64_t)i * nblk + blockIdx.x] = h[i];
}

// one block per digit: exclusive scan of that digit's row of block counts; row total -> digit_total
__global__ void __launch_bounds__(1024)
k_radix_rowscan(uint32_t* __restrict__ hist, int nblk, uint32_t* __restrict__ digit_total) {
  __shared__ uint32_t sm[1024 / 32 + 1];
  uint32_t* row = hist + (int64_t)blockIdx.x * nblk;
  uint32_t carry = 0;
  for (int base = 0; base < nblk; base += 1024) {
    int i = base + threadIdx.x;
    uint32_t v = i < nblk ? row[i] : 0;
    uint32_t total;
    uint32_t ex = block_exclusive_scan<1024>(v, &total, sm);
    if (i < nblk) row[i] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) digit_total[blockIdx.x] = carry;
}

__global__ void __launch_bounds__(kSortThreads)
k_radix_scatter(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, int64_t n, int shift,
                const uint32_t* __restrict__ hist, const uint32_t* __restrict__ digit_total, int nblk,
                uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out) {
  __shared__ uint32_t cnt[kSortWarps][kRadix];  // per-warp digit counts -> offsets
  __shared__ uint32_t dbase[kRadix];
  __shared__ uint32_t sm[kSortThreads / 32 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&cnt[0][0])[i] = 0;
  // global base of each digit = exclusive scan of digit totals (256 values, one per thread)
  {
    uint32_t t = digit_total[threadIdx.x];
    uint32_t total;
    uint32_t ex = block_exclusive_scan<kSortThreads>(t, &total, sm);
    dbase[threadIdx.x] = ex + hist[(int64_t)threadIdx.x * nblk + blockIdx.x];
  }
  __syncthreads();
  // warp w owns keys [base + w*kWarpSpan, +kWarpSpan) in index order (stability)
  int64_t wbase = (int64_t)blockIdx.x * kSortTile + (int64_t)warp * kWarpSpan;
  uint32_t key[kSortItems], val[kSortItems], rnk[kSortItems];
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    int64_t i = wbase + k * 32 + lane;
    bool valid = i < n;
    key[k] = valid ? keys_in[i] : 0xFFFFFFFFu;
    val[k] = valid ? vals_in[i] : 0u;
    uint32_t d = valid ? ((key[k] >> shift) & (kRadix - 1)) : (uint32_t)kRadix;
    uint32_t peers = __match_any_sync(0xffffffffu, d);
    uint32_t before = __popc(peers & ((1u << lane) - 1u));
    uint32_t prev = 0;
    if (valid) prev = cnt[warp][d];
    __syncwarp();
    if (valid && before == 0) cnt[warp][d] = prev + __popc(peers);
    __syncwarp();
    rnk[k] = prev + before;
  }
  __syncthreads();
  // per digit: exclusive scan over warps, plus the global base
  {
    uint32_t run = dbase[threadIdx.x];
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) {
      uint32_t c = cnt[w][threadIdx.x];
      cnt[w][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    int64_t i = wbase + k * 32 + lane;
    if (i < n) {
      uint32_t d = (key[k] >> shift) & (kRadix - 1);
      uint32_t pos = cnt[warp][d] + rnk[k];
      keys_out[pos] = key[k];
      vals_out[pos] = val[k];
    }
  }
}

// ---------------------------------------------------------------------------
// Tile populations from the 2-D difference array.
// diff is (gh+1) x (gw+1); after a prefix along x and along y, entry (y,x) is the
// number of tet rectangles covering tile (y,x).
// ---------------------------------------------------------------------------
__global__ void k_diff_prefix_x(int32_t* __restrict__ diff, int gh, int gw) {
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row > gh) return;
  const int lane = threadIdx.x & 31;
  int32_t* r = diff + (int64_t)row * (gw + 1);
  int32_t carry = 0;
  for (int base = 0; base <= gw; base += 32) {
    int x = base + lane;
    int32_t v = x <= gw ? r[x] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int32_t nb = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += nb;
    }
    v += carry;
    if (x <= gw) r[x] = v;
    carry = __shfl_sync(0xffffffffu, v, 31);
  }
}
__global__ void k_diff_prefix_y(const int32_t* __restrict__ diff, int gh, int gw, uint32_t* __restrict__ counts) {
  int col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (col >= gw) return;
  const int lane = threadIdx.x & 31;
  int32_t carry = 0;
  for (int base = 0; base < gh; base += 32) {
    int y = base + lane;
    int32_t v = y < gh ? diff[(int64_t)y * (gw + 1) + col] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int32_t nb = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += nb;
    }
    v += carry;
    if (y < gh) counts[(int64_t)y * gw + col] = (uint32_t)v;
    carry = __shfl_sync(0xffffffffu, v, 31);
  }
}

// tile_ranges[g] = (start, start+count), or (0,0) for an empty tile
// (compute_tile_ranges leaves untouched tiles at their zero fill).
__global__ void k_write_ranges(const uint32_t* __restrict__ counts, const uint32_t* __restrict__ starts, int64_t G,
                               int2* __restrict__ ranges) {
  int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= G) return;
  uint32_t c = counts[g], s = starts[g];
  ranges[g] = c ? make_int2((int)s, (int)(s + c)) : make_int2(0, 0);
}

__global__ void k_finish_info(RmBinInfo* info, const unsigned long long* total_keys) {
  unsigned long long n = *total_keys;
  info->n_keys = (int64_t)n;
  if (n > 0x7fffffffull) info->status |= RM_STATUS_KEY_OVERFLOW;
}

// ---------------------------------------------------------------------------
// Scatter: one work item per (tile, tet) pair, items numbered in the
// reference's emission order (tets by rank, tile rows then columns), so the
// load is perfectly balanced whatever the rectangle sizes.
//   cum[r]   inclusive scan of tiles_touched in rank order
//   order[r] tet id of rank r
// ---------------------------------------------------------------------------
constexpr int kScatterThreads = 256;
constexpr int kScatterItems = 8;
constexpr int kScatterTile = kScatterThreads * kScatterItems;

__global__ void __launch_bounds__(kScatterThreads)
k_scatter_ranks(const uint32_t* __restrict__ cum, const uint32_t* __restrict__ order, int32_t n_ranked,
                const int4* __restrict__ rect, const int2* __restrict__ ranges, uint32_t* __restrict__ cursor,
                int grid_w, int64_t n_keys, uint32_t* __restrict__ seg) {
  __shared__ uint32_t win[kScatterTile + 1];
  __shared__ int s_r0;
  const int64_t j0 = (int64_t)blockIdx.x * kScatterTile;
  const int64_t j1 = min(j0 + (int64_t)kScatterTile, n_keys);
  if (threadIdx.x == 0) {
    // first rank r with cum[r] > j0
    int lo = 0, hi = n_ranked;
    while (lo < hi) {
      int mid = (lo + hi) >> 1;
      if ((int64_t)cum[mid] > j0) hi = mid; else lo = mid + 1;
    }
    s_r0 = lo;
  }
  __syncthreads();
  const int r0 = s_r0;
  // window of inclusive sums: at most one rank per item plus one
  for (int i = threadIdx.x; i <= kScatterTile; i += kScatterThreads) {
    int r = r0 + i;
    win[i] = r < n_ranked ? cum[r] : 0xFFFFFFFFu;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kScatterItems; ++k) {
    int64_t j = j0 + k * kScatterThreads + threadIdx.x;
    if (j >= j1) continue;
    // first window entry with win[i] > j
    int lo = 0, hi = kScatterTile;
    while (lo < hi) {
      int mid = (lo + hi) >> 1;
      if ((int64_t)win[mid] > j) hi = mid; else lo = mid + 1;
    }
    int r = r0 + lo;
    uint32_t excl = lo > 0 ? win[lo - 1] : (r0 > 0 ? cum[r0 - 1] : 0u);
    uint32_t local = (uint32_t)(j - excl);
    uint32_t tet = order[r];
    int4 rc = __ldg(rect + tet);
    uint32_t w = (uint32_t)(rc.z - rc.x);
    uint32_t ty = rc.y + local / w, tx = rc.x + local % w;
    uint32_t tile = ty * grid_w + tx;
    uint32_t slot = atomicAdd(&cursor[tile], 1u);
    seg[(uint32_t)ranges[tile].x + slot] = (uint32_t)r;
  }
}

// ---------------------------------------------------------------------------
// Per-tile sort of the ranks (unique 32-bit integers) and mapping to tet ids.
// Bitonic network in normalised form (every comparator ascending), so a
// segment of any length sorts without padding: comparators whose upper index
// falls beyond the segment are skipped, which is what +inf padding would do.
// Three size classes share the code: shared memory for segments up to `cap`
// entries, global memory (in place in `seg`) beyond.
// ---------------------------------------------------------------------------
template <bool SHARED>
__device__ __forceinline__ void bitonic_sort(uint32_t* a, uint32_t len) {
  uint32_t P = 1;
  while (P < len) P <<= 1;
  for (uint32_t k = 2; k <= P; k <<= 1) {
    // flip step: i and its mirror inside blocks of k
    for (uint32_t t = threadIdx.x; t < P / 2; t += blockDim.x) {
      uint32_t blk = t / (k / 2), off = t % (k / 2);
      uint32_t i = blk * k + off, l = blk * k + k - 1 - off;
      if (l < len) {
        uint32_t x = a[i], y = a[l];
        if (x > y) { a[i] = y; a[l] = x; }
      }
    }
    __syncthreads();
    for (uint32_t j = k / 4; j >= 1; j >>= 1) {
      for (uint32_t t = threadIdx.x; t < P / 2; t += blockDim.x) {
        uint32_t i = 2 * j * (t / j) + (t % j), l = i + j;
        if (l < len) {
          uint32_t x = a[i], y = a[l];
          if (x > y) { a[i] = y; a[l] = x; }
        }
      }
      __syncthreads();
    }
  }
}

// Segments with lo < len <= hi are handled by this launch (shared-memory variant).
__global__ void k_segment_sort_smem(const int2* __restrict__ ranges, uint32_t* __restrict__ seg,
                                    const uint32_t* __restrict__ order, int32_t* __restrict__ sorted_idx,
                                    uint32_t lo, uint32_t hi) {
  extern __shared__ uint32_t sbuf[];
  int2 rg = ranges[blockIdx.x];
  uint32_t len = (uint32_t)(rg.y - rg.x);
  if (len <= lo || len > hi) return;
  uint32_t* src = seg + rg.x;
  for (uint32_t i = threadIdx.x; i < len; i += blockDim.x) sbuf[i] = src[i];
  __syncthreads();
  bitonic_sort<true>(sbuf, len);
  for (uint32_t i = threadIdx.x; i < len; i += blockDim.x) sorted_idx[rg.x + i] = (int32_t)order[sbuf[i]];
}

__global__ void k_segment_sort_gmem(const int2* __restrict__ ranges, uint32_t* __restrict__ seg,
                                    const uint32_t* __restrict__ order, int32_t* __restrict__ sorted_idx,
                                    uint32_t lo) {
  int2 rg = ranges[blockIdx.x];
  uint32_t len = (uint32_t)(rg.y - rg.x);
  if (len <= lo) return;
  uint32_t* a = seg + rg.x;
  bitonic_sort<false>(a, len);
  for (uint32_t i = threadIdx.x; i < len; i += blockDim.x) sorted_idx[rg.x + i] = (int32_t)order[a[i]];
}

}  // namespace rm

// ---------------------------------------------------------------------------
// Workspace layout (all sub-buffers 256-byte aligned)
// ---------------------------------------------------------------------------
namespace {
struct BinLayout {
  size_t keys_a, keys_b, ord_a, ord_b, hist, digit_total, cum, bsum, tile_diff, tile_count, tile_start, cursor,
      total_keys, total;
  int nblk_sort;
  int64_t nblk_scan_t, nblk_scan_g;
};
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
BinLayout make_layout(int64_t T, int64_t G, int gh, int gw) {
  BinLayout L;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align256(off + bytes);
    return o;
  };
  int64_t Tp = T > 0 ? T : 1;
  L.nblk_sort = (int)((Tp + rm::kSortTile - 1) / rm::kSortTile);
  L.nblk_scan_t = (Tp + rm::kScanTile - 1) / rm::kScanTile;
  L.nblk_scan_g = (G + rm::kScanTile - 1) / rm::kScanTile;
  L.keys_a = take(4 * Tp);
  L.keys_b = take(4 * Tp);
  L.ord_a = take(4 * Tp);
  L.ord_b = take(4 * Tp);
  L.hist = take(4 * (size_t)rm::kRadix * L.nblk_sort);
  L.digit_total = take(4 * rm::kRadix);
  L.cum = take(4 * Tp);
  L.bsum = take(4 * (size_t)(L.nblk_scan_t > L.nblk_scan_g ? L.nblk_scan_t : L.nblk_scan_g) + 4);
  // (gh+1)*(gw+1) <= G + gh + gw + 1; gh, gw <= G
  L.tile_diff = take(4 * (size_t)(gh >= 0 ? (int64_t)(gh + 1) * (gw + 1) : 4 * G + 4));
  L.tile_count = take(4 * (size_t)(G + 1));
  L.tile_start = take(4 * (size_t)(G + 1));
  L.cursor = take(4 * (size_t)(G + 1));
  L.total_keys = take(16);
  L.total = off;
  return L;
}
}  // namespace

size_t rm_bin_layout_bytes(int64_t T, int64_t G) {
  // upper bound that does not need gh, gw: (gh+1)(gw+1) <= 2G + 2 for gh, gw >= 1 ... use 4G + 4
  return make_layout(T, G, -1, -1).total;
}

int rm_launch_bin_prepare(int64_t T, const RmCamera* cam, void* ws, size_t ws_bytes, uint32_t** depth_keys,
                          uint32_t** order_in, int32_t** tile_diff, RmBinInfo* info, cudaStream_t st) {
  const int gh = cam->grid_height, gw = cam->grid_width;
  const int64_t G = (int64_t)gh * gw;
  BinLayout L = make_layout(T, G, gh, gw);
  if (L.total > ws_bytes) return RM_ERR_WORKSPACE;
  char* b = static_cast<char*>(ws);
  *depth_keys = reinterpret_cast<uint32_t*>(b + L.keys_a);
  *order_in = reinterpret_cast<uint32_t*>(b + L.ord_a);
  *tile_diff = reinterpret_cast<int32_t*>(b + L.tile_diff);
  RM_CUDA_CHECK(cudaMemsetAsync(b + L.tile_diff, 0, 4 * (size_t)(gh + 1) * (gw + 1), st));
  RM_CUDA_CHECK(cudaMemsetAsync(b + L.cursor, 0, 4 * (size_t)(G + 1), st));
  RM_CUDA_CHECK(cudaMemsetAsync(info, 0, sizeof(RmBinInfo), st));
  return RM_OK;
}

static int launch_scan(const uint32_t* in, const uint32_t* gather, int64_t n, uint32_t* bsum, uint32_t* out,
                       int inclusive, unsigned long long* total64, cudaStream_t st) {
  if (n <= 0) {
    if (total64) RM_CUDA_CHECK(cudaMemsetAsync(total64, 0, 8, st));
    return RM_OK;
  }
  int64_t nb = (n + rm::kScanTile - 1) / rm::kScanTile;
  rm::k_scan_block_sums<<<(unsigned)nb, rm::kScanThreads, 0, st>>>(in, gather, n, bsum);
  rm::k_scan_sums<<<1, 1024, 0, st>>>(bsum, nb, total64);
  rm::k_scan_apply<<<(unsigned)nb, rm::kScanThreads, 0, st>>>(in, gather, n, bsum, out, inclusive);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

// After k_project: rank the tets, build tile_ranges, the rank-ordered inclusive
// scan of tiles_touched, and the info block.
int rm_launch_bin_finish(int64_t T, const RmCamera* cam, const int32_t* tiles_touched, int32_t* tile_ranges,
                         RmBinInfo* info, void* ws, cudaStream_t st) {
  const int gh = cam->grid_height, gw = cam->grid_width;
  const int64_t G = (int64_t)gh * gw;
  BinLayout L = make_layout(T, G, gh, gw);
  char* b = static_cast<char*>(ws);
  uint32_t* keys[2] = {reinterpret_cast<uint32_t*>(b + L.keys_a), reinterpret_cast<uint32_t*>(b + L.keys_b)};
  uint32_t* ord[2] = {reinterpret_cast<uint32_t*>(b + L.ord_a), reinterpret_cast<uint32_t*>(b + L.ord_b)};
  uint32_t* hist = reinterpret_cast<uint32_t*>(b + L.hist);
  uint32_t* dtot = reinterpret_cast<uint32_t*>(b + L.digit_total);
  uint32_t* cum = reinterpret_cast<uint32_t*>(b + L.cum);
  uint32_t* bsum = reinterpret_cast<uint32_t*>(b + L.bsum);
  int32_t* diff = reinterpret_cast<int32_t*>(b + L.tile_diff);
  uint32_t* tcount = reinterpret_cast<uint32_t*>(b + L.tile_count);
  uint32_t* tstart = reinterpret_cast<uint32_t*>(b + L.tile_start);
  unsigned long long* total_keys = reinterpret_cast<unsigned long long*>(b + L.total_keys);

  // 1. rank tets by (depth bits, id): 4 stable passes; result ends in buffer 0
  if (T > 0) {
    RmProfScope prof("rank_tets_radix_sort(12 launches)", st);
    for (int pass = 0; pass < 4; ++pass) {
      int src = pass & 1, dst = src ^ 1;
      int shift = pass * rm::kRadixBits;
      rm::k_radix_hist<<<L.nblk_sort, rm::kSortThreads, 0, st>>>(keys[src], T, shift, hist, L.nblk_sort);
      rm::k_radix_rowscan<<<rm::kRadix, 1024, 0, st>>>(hist, L.nblk_sort, dtot);
      rm::k_radix_scatter<<<L.nblk_sort, rm::kSortThreads, 0, st>>>(keys[src], ord[src], T, shift, hist, dtot,
                                                                   L.nblk_sort, keys[dst], ord[dst]);
    }
    RM_CUDA_CHECK(cudaPeekAtLastError());
  }
  // 2. tile populations -> tile_ranges
  {
    RmProfScope prof("tile_ranges(6 launches)", st);
    int rows_per_block = 4;  // 128 threads
    rm::k_diff_prefix_x<<<(gh + 1 + rows_per_block - 1) / rows_per_block, 32 * rows_per_block, 0, st>>>(diff, gh, gw);
    rm::k_diff_prefix_y<<<(gw + rows_per_block - 1) / rows_per_block, 32 * rows_per_block, 0, st>>>(diff, gh, gw,
                                                                                                  tcount);
    int rc = launch_scan(tcount, nullptr, G, bsum, tstart, 0, nullptr, st);
    if (rc) return rc;
    rm::k_write_ranges<<<(unsigned)((G + 255) / 256), 256, 0, st>>>(tcount, tstart, G,
                                                                    reinterpret_cast<int2*>(tile_ranges));
    RM_CUDA_CHECK(cudaPeekAtLastError());
  }
  // 3. inclusive scan of tiles_touched in rank order (culled tets sort last with 0 tiles)
  {
    RmProfScope prof("rank_order_scan(4 launches)", st);
    int rc = launch_scan(reinterpret_cast<const uint32_t*>(tiles_touched), ord[0], T, bsum, cum, 1, total_keys, st);
    if (rc) return rc;
    rm::k_finish_info<<<1, 1, 0, st>>>(info, total_keys);
    RM_CUDA_CHECK(cudaPeekAtLastError());
  }
  return RM_OK;
}

int rm_launch_build_lists(const int32_t* rect, const int32_t* tile_ranges, int64_t T, const RmCamera* cam,
                          int64_t n_keys, void* ws, uint32_t* scratch, int32_t* sorted_idx, cudaStream_t st) {
  if (n_keys == 0) return RM_OK;
  const int gh = cam->grid_height, gw = cam->grid_width;
  const int64_t G = (int64_t)gh * gw;
  BinLayout L = make_layout(T, G, gh, gw);
  char* b = static_cast<char*>(ws);
  const uint32_t* order = reinterpret_cast<uint32_t*>(b + L.ord_a);
  const uint32_t* cum = reinterpret_cast<uint32_t*>(b + L.cum);
  uint32_t* cursor = reinterpret_cast<uint32_t*>(b + L.cursor);
  const int2* ranges = reinterpret_cast<const int2*>(tile_ranges);
  RM_CUDA_CHECK(cudaMemsetAsync(cursor, 0, 4 * (size_t)(G + 1), st));
  int64_t nb = (n_keys + rm::kScatterTile - 1) / rm::kScatterTile;
  {
    RmProfScope prof("k_scatter_ranks", st);
    rm::k_scatter_ranks<<<(unsigned)nb, rm::kScatterThreads, 0, st>>>(cum, order, (int32_t)T,
                                                                       reinterpret_cast<const int4*>(rect), ranges,
                                                                       cursor, gw, n_keys, scratch);
  }
  RM_CUDA_CHECK(cudaPeekAtLastError());
  // size classes: (0, 2048] in 8 KB of shared memory, (2048, 32768] in 128 KB, larger in global memory
  const uint32_t small_cap = 2048, big_cap = 32768;
  RM_CUDA_CHECK(cudaFuncSetAttribute(rm::k_segment_sort_smem, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)(big_cap * 4)));
  RmProfScope prof("k_segment_sort(3 launches)", st);
  rm::k_segment_sort_smem<<<(unsigned)G, 256, small_cap * 4, st>>>(ranges, scratch, order, sorted_idx, 0, small_cap);
  rm::k_segment_sort_smem<<<(unsigned)G, 1024, big_cap * 4, st>>>(ranges, scratch, order, sorted_idx, small_cap,
                                                                  big_cap);
  rm::k_segment_sort_gmem<<<(unsigned)G, 1024, 0, st>>>(ranges, scratch, order, sorted_idx, big_cap);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}
