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
//   3. the (tile, tet) pairs, generated in rank order and load-balanced over
//      pairs, go through a stable two-pass counting sort on the tile id alone
//      (17 bits at 1080p, against the reference's 49-bit keys); stability keeps
//      every tile's segment in rank order, so nothing is sorted per tile.
//
// Ascending rank inside a tile is ascending (depth bits, tet id), which is what
// the reference's stable sort produces because it emits pairs in tet order.

#include "rm_common.cuh"

namespace rm {

// ---------------------------------------------------------------------------
// Regions: blocks of kRegW x kRegH tiles, one tile per lane of a warp.
// ---------------------------------------------------------------------------
constexpr int kRegShiftX = 3, kRegShiftY = 2;
constexpr int kRegW = 1 << kRegShiftX, kRegH = 1 << kRegShiftY;  // 8 x 4 = 32 tiles

// number of regions a tile rectangle (x0, y0, x1, y1), max exclusive, touches; 0 for an empty one
__device__ __forceinline__ uint32_t regions_touched(int4 rc) {
  if (rc.z <= rc.x || rc.w <= rc.y) return 0u;
  return (uint32_t)((((rc.z - 1) >> kRegShiftX) - (rc.x >> kRegShiftX) + 1) *
                    (((rc.w - 1) >> kRegShiftY) - (rc.y >> kRegShiftY) + 1));
}

// ---------------------------------------------------------------------------
// Device-wide exclusive scan of uint32 (three launches: block sums, scan of the
// block sums, apply).  Optional gather: element i is in[gather[i]].  With `rect`
// the element is the number of regions rect[gather[i]] touches instead.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t scan_value(const uint32_t* __restrict__ in, const uint32_t* __restrict__ gather,
                                               const int4* __restrict__ rect, int64_t i) {
  if (rect) return regions_touched(__ldg(rect + gather[i]));
  return gather ? in[gather[i]] : in[i];
}
// number of valid items: n, or the device-side count if one is given (the visible tets, known only on the device)
__device__ __forceinline__ int64_t valid_items(int64_t n, const int32_t* __restrict__ n_dev) {
  return n_dev ? min(n, (int64_t)__ldg(n_dev)) : n;
}

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
k_scan_block_sums(const uint32_t* __restrict__ in, const uint32_t* __restrict__ gather,
                  const int4* __restrict__ rect, int64_t n, const int32_t* __restrict__ n_dev,
                  uint32_t* __restrict__ bsum, uint32_t* __restrict__ values_out) {
  __shared__ uint32_t sm[kScanThreads / 32 + 1];
  int64_t base = (int64_t)blockIdx.x * kScanTile;
  const int64_t nv = valid_items(n, n_dev);
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    int64_t i = base + k * kScanThreads + threadIdx.x;
    if (i < n) {
      const uint32_t v = i < nv ? scan_value(in, gather, rect, i) : 0u;
      if (values_out) values_out[i] = v;  // gathered once: the apply pass reads these in place
      s += v;
    }
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
k_scan_apply(const uint32_t* in, const uint32_t* __restrict__ gather, const int4* __restrict__ rect,
             int64_t n, const uint32_t* __restrict__ bsum, uint32_t* out /* may be `in` */, int inclusive) {
  __shared__ uint32_t sm[kScanThreads / 32 + 1];
  // blocked arrangement: thread t owns items [t*kScanItems, (t+1)*kScanItems)
  int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    int64_t i = base + k;
    v[k] = i < n ? scan_value(in, gather, rect, i) : 0;
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
// Stable compaction of the (key, value) pairs whose key is not 0xFFFFFFFF (the visible tets) to the
// front of the output arrays: block counts -> k_scan_sums -> scatter with the block's own scan.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kScanThreads)
k_compact_count(const uint32_t* __restrict__ keys, int64_t n, uint32_t* __restrict__ bsum) {
  __shared__ uint32_t sm[kScanThreads / 32 + 1];
  const int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    const int64_t i = base + k;
    s += (i < n && keys[i] != 0xFFFFFFFFu) ? 1u : 0u;
  }
  uint32_t total;
  block_exclusive_scan<kScanThreads>(s, &total, sm);
  if (threadIdx.x == 0) bsum[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads)
k_compact_scatter(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n,
                  const uint32_t* __restrict__ bsum, uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out) {
  __shared__ uint32_t sm[kScanThreads / 32 + 1];
  // blocked arrangement (thread t owns kScanItems consecutive items), so that the order is kept
  const int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  uint32_t key[kScanItems];
  uint32_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    const int64_t i = base + k;
    key[k] = i < n ? keys[i] : 0xFFFFFFFFu;
    s += key[k] != 0xFFFFFFFFu ? 1u : 0u;
  }
  uint32_t total;
  uint32_t pos = block_exclusive_scan<kScanThreads>(s, &total, sm) + bsum[blockIdx.x];
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    if (key[k] != 0xFFFFFFFFu) {
      if (RM_INDEX_OK(pos, RM_X_TETS, 13)) {
        keys_out[pos] = key[k];
        vals_out[pos] = vals[base + k];
      }
      ++pos;
    }
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
k_radix_hist(const uint32_t* __restrict__ keys, int64_t n_max, const int32_t* __restrict__ n_dev, int shift,
             uint32_t* __restrict__ hist, int nblk) {
  __shared__ uint32_t h[kRadix];
  const int64_t n = valid_items(n_max, n_dev);
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

__device__ __forceinline__ void local_layout(uint32_t bins, uint32_t* cnt, uint32_t* dbase, uint32_t* lstart,
                                             uint32_t* s_scan);

// Stable scatter of one pass.  The block's pairs are first reordered by digit in shared
// memory, so that the global stores of one digit's run are contiguous.
__global__ void __launch_bounds__(kSortThreads, 3)
k_radix_scatter(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, int64_t n_max,
                const int32_t* __restrict__ n_dev, int shift, const uint32_t* __restrict__ hist,
                const uint32_t* __restrict__ digit_total, int nblk, uint32_t* __restrict__ keys_out,
                uint32_t* __restrict__ vals_out) {
  const int64_t n = valid_items(n_max, n_dev);
  __shared__ uint2 sbuf[kSortTile];
  __shared__ uint32_t cnt[kSortWarps * kRadix];  // per-warp digit counts -> offsets
  __shared__ uint32_t dbase[kRadix];
  __shared__ uint32_t lstart[kRadix];
  __shared__ uint32_t sm[kSortThreads / 32 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) cnt[i] = 0;
  // global base of each digit = exclusive scan of digit totals (256 values, one per thread)
  {
    uint32_t t = digit_total[threadIdx.x];
    uint32_t total;
    uint32_t ex = block_exclusive_scan<kSortThreads>(t, &total, sm);
    dbase[threadIdx.x] = ex + hist[(int64_t)threadIdx.x * nblk + blockIdx.x];
  }
  __syncthreads();
  // warp w owns keys [base + w*kWarpSpan, +kWarpSpan) in index order (stability)
  const int64_t bbase = (int64_t)blockIdx.x * kSortTile;
  const int64_t wbase = bbase + (int64_t)warp * kWarpSpan;
  uint32_t* wc = cnt + warp * kRadix;
  uint32_t key[kSortItems], val[kSortItems], rnk[kSortItems];
  // loads first (in flight together); the warp barriers of the ranking rounds would
  // otherwise serialise them
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    int64_t i = wbase + k * 32 + lane;
    bool valid = i < n;
    key[k] = valid ? keys_in[i] : 0xFFFFFFFFu;
    val[k] = valid ? vals_in[i] : 0u;
  }
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    const bool valid = wbase + k * 32 + lane < n;
    uint32_t d = (key[k] >> shift) & (kRadix - 1);
    uint32_t peers = __ballot_sync(0xffffffffu, valid);
#pragma unroll
    for (int b = 0; b < kRadixBits; ++b) {
      const bool bit = (d >> b) & 1u;
      const uint32_t m = __ballot_sync(0xffffffffu, bit);
      peers &= bit ? m : ~m;
    }
    uint32_t before = __popc(peers & ((1u << lane) - 1u));
    uint32_t prev = 0;
    if (valid) prev = wc[d];
    __syncwarp();
    if (valid && before == 0) wc[d] = prev + __popc(peers);
    __syncwarp();
    rnk[k] = prev + before;
  }
  __syncthreads();
  local_layout(kRadix, cnt, dbase, lstart, sm);
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    if (wbase + k * 32 + lane < n) {
      const uint32_t d = (key[k] >> shift) & (kRadix - 1);
      sbuf[lstart[d] + wc[d] + rnk[k]] = make_uint2(key[k], val[k]);
    }
  }
  __syncthreads();
  const int n_block = (int)min((int64_t)kSortTile, n - bbase);
  for (int lp = threadIdx.x; lp < n_block; lp += kSortThreads) {
    const uint2 pr = sbuf[lp];
    const uint32_t g = dbase[(pr.x >> shift) & (kRadix - 1)] + (uint32_t)lp;
    if (!RM_INDEX_OK(g, RM_X_TETS, 13)) continue;
    keys_out[g] = pr.x;
    vals_out[g] = pr.y;
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

// total_keys[0] = sum of the tile populations, total_keys[1] = sum of regions touched
__global__ void k_finish_info(RmBinInfo* info, const unsigned long long* total_keys) {
  unsigned long long n = total_keys[0];
  info->n_keys = (int64_t)n;
  info->n_region_keys = (int64_t)total_keys[1];
  if (n > 0x7fffffffull) info->status |= RM_STATUS_KEY_OVERFLOW;
}

// ---------------------------------------------------------------------------
// Tile lists, built in two levels.
//
// Level 1 (regions).  Work items are the (region, tet) pairs numbered in rank
// order (tets by rank, then region rows, then columns): item j belongs to the
// rank r with cum[r-1] <= j < cum[r].  A stable two-pass counting sort on the
// region id (low digit first, then high digit) leaves every region's segment
// ordered by rank, i.e. by (depth bits, tet id): no per-region sort, no atomics
// on the data path, deterministic.  A tet touches far fewer regions than tiles
// (about 9 times fewer at 1080p with 4 x 4 pixel tiles), so this sort moves a
// fraction of the pairs.  Every sorted entry carries the tet id and a 32-bit
// mask of the region's tiles its rectangle covers.
//   generate: the (tet, region) pairs, their low-digit histogram and the region populations
//   pass 1: stable split on the low  b1 bits of the region id
//   pass 2: stable split on the high b2 bits -> entries (tet id, tile mask)
// Each pass is: per-block digit histogram, per-digit scan over the blocks,
// stable scatter (warp-level match ranking, warps own consecutive item spans).
//
// Level 2 (tiles).  A region's segment is cut into chunks of kChunk entries, one
// warp per chunk, lane l owning tile l of the region.  A lane's tile list is the
// subsequence of entries whose mask has bit l: the count pass adds up the bits
// per chunk and lane (a 32 x 32 bit transpose and a popcount per 32 entries), a
// per-region scan over the chunks turns the counts into write cursors starting
// at the tile's range, and the write pass walks the chunk again: per round of 32
// entries and per tile, the lanes whose entry covers the tile (one ballot) store
// their tet ids behind the tile's cursor as one contiguous run.  Order inside a
// tile is the order of the region's segment: rank order.
// ---------------------------------------------------------------------------
constexpr int kBinThreads = 256;
constexpr int kBinItems = 16;
constexpr int kBinTile = kBinThreads * kBinItems;  // items per block
constexpr int kBinWarps = kBinThreads / 32;
static_assert(kBinThreads == kSortThreads, "local_layout is shared by the rank sort and the region sort");
constexpr int kBinSpan = 32 * kBinItems;  // consecutive items owned by one warp

template <int THREADS>
__device__ __forceinline__ uint32_t block_exclusive_maxscan(uint32_t v, uint32_t* smem /* THREADS/32 */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc = max(inc, n);
  }
  if (lane == 31) smem[warp] = inc;
  __syncthreads();
  uint32_t prev = 0;
  for (int w = 0; w < warp; ++w) prev = max(prev, smem[w]);
  uint32_t up = __shfl_up_sync(0xffffffffu, inc, 1);
  uint32_t ex = lane ? max(prev, up) : prev;
  __syncthreads();
  return ex;
}

// First rank of every block of kBinTile items (first r with cum[r] > block start),
// one thread per block so that the dependent loads of the searches overlap.
__global__ void k_block_start_ranks(const uint32_t* __restrict__ cum, int n_ranked, int nblk,
                                    uint32_t* __restrict__ start_rank) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblk) return;
  const int64_t j0 = (int64_t)b * kBinTile;
  int lo = 0, hi = n_ranked;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((int64_t)__ldg(cum + mid) > j0) hi = mid; else lo = mid + 1;
  }
  start_rank[b] = (uint32_t)lo;
}

// Owner table of the block's items: after this call item jl (0 <= jl < items of the
// block) belongs to rank *r0 + own[jl]; win[i] = cum[*r0 + i].
__device__ __forceinline__ void owners_of_items(const uint32_t* __restrict__ cum, int n_ranked, int64_t j0,
                                                const uint32_t* __restrict__ start_rank,
                                                uint32_t* win /* kBinTile+1 */, uint16_t* own /* kBinTile */,
                                                uint32_t* s_misc /* 16 words */) {
  if (threadIdx.x == 0) {
    const uint32_t lo = start_rank[blockIdx.x];
    s_misc[8] = lo;
    s_misc[9] = lo > 0 ? cum[lo - 1] : 0u;  // items before rank r0
  }
  for (int i = threadIdx.x; i < kBinTile; i += kBinThreads) own[i] = 0;
  __syncthreads();
  const int r0 = (int)s_misc[8];
  for (int i = threadIdx.x; i <= kBinTile; i += kBinThreads) {
    int r = r0 + i;
    uint32_t c = r < n_ranked ? cum[r] : 0xFFFFFFFFu;
    win[i] = c;
    // rank r0+i+1 starts at item c (visible tets have at least one item, so starts are distinct)
    int64_t start = (int64_t)c - j0;
    if (c != 0xFFFFFFFFu && start < kBinTile && r + 1 < n_ranked) own[start] = (uint16_t)(i + 1);
  }
  __syncthreads();
  // inclusive max-scan of own[], thread t owning items [16t, 16t+16)
  uint32_t loc[kBinItems];
  uint32_t m = 0;
#pragma unroll
  for (int k = 0; k < kBinItems; ++k) {
    m = max(m, (uint32_t)own[threadIdx.x * kBinItems + k]);
    loc[k] = m;
  }
  uint32_t ex = block_exclusive_maxscan<kBinThreads>(m, s_misc);
#pragma unroll
  for (int k = 0; k < kBinItems; ++k) own[threadIdx.x * kBinItems + k] = (uint16_t)max(ex, loc[k]);
  __syncthreads();
}

// region id and tet id of local item jl
__device__ __forceinline__ void item_region(int jl, int64_t j0, int r0, uint32_t before_r0, const uint32_t* win,
                                            const uint16_t* own, const uint32_t* __restrict__ order,
                                            const int4* __restrict__ rect, int reg_w, uint32_t& region,
                                            uint32_t& tet) {
  const int i = own[jl];
  const uint32_t rank = (uint32_t)(r0 + i);
  const uint32_t excl = i > 0 ? win[i - 1] : before_r0;
  const uint32_t local = (uint32_t)(j0 + jl - excl);
  tet = order[rank];
  const int4 rc = __ldg(rect + tet);
  const uint32_t cx0 = (uint32_t)(rc.x >> kRegShiftX);
  const uint32_t w = (uint32_t)((rc.z - 1) >> kRegShiftX) - cx0 + 1u;
  const uint32_t dy = local / w;
  region = ((uint32_t)(rc.y >> kRegShiftY) + dy) * (uint32_t)reg_w + cx0 + (local - dy * w);
}

// Sorted entry of (tet, region): the tet id and the mask of the region's tiles (bit = 8 * row + column)
// that the tet's rectangle covers.
__device__ __forceinline__ uint2 region_entry(uint32_t tet, uint32_t region, const int4* __restrict__ rect,
                                              int reg_w) {
  const int4 rc = __ldg(rect + tet);
  const int gy = (int)(region / (uint32_t)reg_w), gx = (int)(region - (uint32_t)gy * (uint32_t)reg_w);
  const int lx0 = max(rc.x - gx * kRegW, 0), lx1 = min(rc.z - gx * kRegW, kRegW);
  const int ly0 = max(rc.y - gy * kRegH, 0), ly1 = min(rc.w - gy * kRegH, kRegH);
  const uint32_t row = (1u << lx1) - (1u << lx0);
  const uint32_t rows = 0x01010101u & (uint32_t)((1ull << (8 * ly1)) - (1ull << (8 * ly0)));
  return make_uint2(tet, row * rows);
}

// Generates the block's (tet, region) pairs, writes them out, and forms their pass-1 digit
// histogram; also the population of every region
// (region_count, zeroed by the caller), accumulated in shared memory when the
// region table fits (n_regions_smem = n_regions) and with global atomics otherwise
// (n_regions_smem = 0).
__global__ void __launch_bounds__(kBinThreads)
k_region_hist1(const uint32_t* __restrict__ cum, const uint32_t* __restrict__ start_rank,
               const uint32_t* __restrict__ order, int n_ranked, const int4* __restrict__ rect, int reg_w,
               int64_t n_items, uint32_t bins, uint32_t* __restrict__ hist, int nblk, uint32_t n_regions_smem,
               uint32_t* __restrict__ region_count, uint2* __restrict__ pairs_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* win = reinterpret_cast<uint32_t*>(smem_raw);
  uint32_t* s_misc = win + kBinTile + 4;
  uint16_t* own = reinterpret_cast<uint16_t*>(s_misc + 16);
  uint32_t* h = reinterpret_cast<uint32_t*>(own + kBinTile);
  uint32_t* rh = h + bins;
  const int64_t j0 = (int64_t)blockIdx.x * kBinTile;
  const int cnt = (int)min((int64_t)kBinTile, n_items - j0);
  for (uint32_t i = threadIdx.x; i < bins + n_regions_smem; i += kBinThreads) h[i] = 0;
  owners_of_items(cum, n_ranked, j0, start_rank, win, own, s_misc);
  const int r0 = (int)s_misc[8];
  const uint32_t before = s_misc[9];
  for (int jl = threadIdx.x; jl < cnt; jl += kBinThreads) {
    uint32_t region, tet;
    item_region(jl, j0, r0, before, win, own, order, rect, reg_w, region, tet);
    if (!(RM_INDEX_OK(region, RM_X_REGIONS, 11) && RM_INDEX_OK(tet, RM_X_TETS, 13))) continue;
    pairs_out[j0 + jl] = make_uint2(tet, region);  // generated once; the scatter passes read them back
    atomicAdd(&h[region & (bins - 1)], 1u);
    if (n_regions_smem) atomicAdd(&rh[region], 1u);
    else atomicAdd(region_count + region, 1u);
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < bins; i += kBinThreads) hist[(int64_t)i * nblk + blockIdx.x] = h[i];
  for (uint32_t i = threadIdx.x; i < n_regions_smem; i += kBinThreads)
    if (rh[i]) atomicAdd(region_count + i, rh[i]);
}

__global__ void __launch_bounds__(kBinThreads)
k_region_hist2(const uint2* __restrict__ pairs, int64_t n, int shift, uint32_t bins, uint32_t* __restrict__ hist,
             int nblk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* h = reinterpret_cast<uint32_t*>(smem_raw);
  for (uint32_t i = threadIdx.x; i < bins; i += kBinThreads) h[i] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kBinTile;
#pragma unroll
  for (int k = 0; k < kBinItems; ++k) {
    int64_t i = base + k * kBinThreads + threadIdx.x;
    if (i < n) atomicAdd(&h[(pairs[i].y >> shift) & (bins - 1)], 1u);
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < bins; i += kBinThreads) hist[(int64_t)i * nblk + blockIdx.x] = h[i];
}

// Stable placement of the block's items, in three steps shared by both passes:
//   digit_bases   global base of each digit for this block -> dbase[]
//   rank_round    one round of 32 consecutive items per warp: rank of each item
//                 among the earlier items of the same digit in the warp's span
//   warp_offsets  turns the per-warp digit counts into absolute offsets
// cnt is [kBinWarps][bins], zeroed by the caller.
__device__ __forceinline__ void digit_bases(uint32_t bins, const uint32_t* __restrict__ hist,
                                            const uint32_t* __restrict__ digit_total, int nblk, uint32_t* dbase,
                                            uint32_t* s_scan) {
  const uint32_t per = bins > kBinThreads ? bins / kBinThreads : 1;
  uint32_t s = 0;
  for (uint32_t q = 0; q < per; ++q) {
    uint32_t dgt = threadIdx.x * per + q;
    if (dgt < bins) s += digit_total[dgt];
  }
  uint32_t total;
  uint32_t ex = block_exclusive_scan<kBinThreads>(s, &total, s_scan);
  for (uint32_t q = 0; q < per; ++q) {
    uint32_t dgt = threadIdx.x * per + q;
    if (dgt < bins) {
      dbase[dgt] = ex + hist[(int64_t)dgt * nblk + blockIdx.x];
      ex += digit_total[dgt];
    }
  }
}

// Lanes of the warp holding the same `nbits`-bit digit (valid lanes only), from one
// ballot per bit: constant cost, where match.any slows down with the number of
// distinct values.
__device__ __forceinline__ uint32_t match_digit(uint32_t digit, bool valid, int nbits) {
  uint32_t peers = __ballot_sync(0xffffffffu, valid);
  for (int b = 0; b < nbits; ++b) {
    const bool bit = (digit >> b) & 1u;
    const uint32_t m = __ballot_sync(0xffffffffu, bit);
    peers &= bit ? m : ~m;
  }
  return peers;
}

__device__ __forceinline__ uint32_t rank_round(uint32_t digit, bool valid, uint32_t* wc, int nbits) {
  const int lane = threadIdx.x & 31;
  const uint32_t peers = match_digit(digit, valid, nbits);
  const uint32_t before = __popc(peers & ((1u << lane) - 1u));
  uint32_t prev = 0;
  if (valid) prev = wc[digit];
  __syncwarp();
  if (valid && before == 0) wc[digit] = prev + __popc(peers);
  __syncwarp();
  return prev + before;
}

// After the ranking rounds: cnt[w][d] becomes the offset of warp w inside digit d's
// run of this block, lstart[d] the run's start inside the block's reordered buffer,
// and dbase[d] the difference (global position) - (position in the buffer).
__device__ __forceinline__ void local_layout(uint32_t bins, uint32_t* cnt, uint32_t* dbase, uint32_t* lstart,
                                             uint32_t* s_scan) {
  for (uint32_t dgt = threadIdx.x; dgt < bins; dgt += kBinThreads) {
    uint32_t run = 0;
#pragma unroll
    for (int w = 0; w < kBinWarps; ++w) {
      uint32_t c = cnt[(size_t)w * bins + dgt];
      cnt[(size_t)w * bins + dgt] = run;
      run += c;
    }
    lstart[dgt] = run;  // run length for now
  }
  __syncthreads();
  const uint32_t per = bins > kBinThreads ? bins / kBinThreads : 1;
  uint32_t s = 0;
  for (uint32_t q = 0; q < per; ++q) {
    uint32_t dgt = threadIdx.x * per + q;
    if (dgt < bins) s += lstart[dgt];
  }
  uint32_t total;
  uint32_t ex = block_exclusive_scan<kBinThreads>(s, &total, s_scan);
  for (uint32_t q = 0; q < per; ++q) {
    uint32_t dgt = threadIdx.x * per + q;
    if (dgt < bins) {
      uint32_t len = lstart[dgt];
      lstart[dgt] = ex;
      dbase[dgt] -= ex;
      ex += len;
    }
  }
  __syncthreads();
}

// One stable counting pass on the digit (region >> shift) & (bins - 1).  final == 0: the reordered
// pairs go to pairs_out; final != 0: the sorted entries (tet id, tile mask) are written instead.
// Items are reordered by digit in shared memory first, so that the global writes of one digit's
// run are contiguous.
__global__ void __launch_bounds__(kBinThreads, 3)
k_region_scatter(const uint2* __restrict__ pairs, int64_t n, int shift, uint32_t bins,
                 const uint32_t* __restrict__ hist, const uint32_t* __restrict__ digit_total, int nblk, int final,
                 const int4* __restrict__ rect, int reg_w, uint2* __restrict__ pairs_out,
                 uint2* __restrict__ entries) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint2* sbuf = reinterpret_cast<uint2*>(smem_raw);
  uint32_t* dbase = reinterpret_cast<uint32_t*>(smem_raw + 8 * kBinTile);
  uint32_t* lstart = dbase + bins;
  uint32_t* cnt = lstart + bins;
  uint32_t* s_scan = cnt + (size_t)kBinWarps * bins;
  for (uint32_t i = threadIdx.x; i < kBinWarps * bins; i += kBinThreads) cnt[i] = 0;
  digit_bases(bins, hist, digit_total, nblk, dbase, s_scan);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t* wc = cnt + (size_t)warp * bins;
  const int64_t base = (int64_t)blockIdx.x * kBinTile;
  const int cntItems = (int)min((int64_t)kBinTile, n - base);
  uint2 pr[kBinItems];
#pragma unroll
  for (int k = 0; k < kBinItems; ++k) {
    const int jl = warp * kBinSpan + k * 32 + lane;
    pr[k] = jl < cntItems ? pairs[base + jl] : make_uint2(0u, 0u);
  }
  uint32_t rnk[kBinItems / 2];
#pragma unroll
  for (int k = 0; k < kBinItems; ++k) {
    const bool valid = warp * kBinSpan + k * 32 + lane < cntItems;
    const uint32_t r = rank_round((pr[k].y >> shift) & (bins - 1), valid, wc, 31 - __clz(bins));
    if (k & 1) rnk[k >> 1] |= r << 16; else rnk[k >> 1] = r;
  }
  __syncthreads();
  local_layout(bins, cnt, dbase, lstart, s_scan);
#pragma unroll
  for (int k = 0; k < kBinItems; ++k) {
    if (warp * kBinSpan + k * 32 + lane >= cntItems) continue;
    const uint32_t dgt = (pr[k].y >> shift) & (bins - 1);
    const uint32_t lp = lstart[dgt] + wc[dgt] + ((rnk[k >> 1] >> (16 * (k & 1))) & 0xFFFFu);
    sbuf[lp] = pr[k];
  }
  __syncthreads();
  for (int lp = threadIdx.x; lp < cntItems; lp += kBinThreads) {
    const uint2 p2 = sbuf[lp];
    const uint32_t g = dbase[(p2.y >> shift) & (bins - 1)] + (uint32_t)lp;
    if (!RM_INDEX_OK(g, RM_X_PAIRS, 9)) continue;
    if (final) entries[g] = region_entry(p2.x, p2.y, rect, reg_w);
    else pairs_out[g] = p2;
  }
}

// ---------------------------------------------------------------------------
// Level 2: from the region segments to the tile lists.
// ---------------------------------------------------------------------------
constexpr int kChunk = 256;        // entries of a region segment handled by one warp
constexpr int kFineThreads = 256;  // 8 warps = 8 chunks per block
constexpr int kFineWarps = kFineThreads / 32;

// Single block: region_start = exclusive scan of region_count, chunk_base = exclusive scan of
// ceil(region_count / kChunk) (both with a closing total at index n_regions), and the region of
// every chunk.
__global__ void __launch_bounds__(1024)
k_region_layout(const uint32_t* __restrict__ region_count, uint32_t n_regions, uint32_t* __restrict__ region_start,
                uint32_t* __restrict__ chunk_base, uint32_t* __restrict__ chunk_region) {
  __shared__ uint32_t sm[1024 / 32 + 1];
  uint32_t carry_e = 0, carry_c = 0;
  for (uint32_t base = 0; base < n_regions; base += 1024) {
    const uint32_t r = base + threadIdx.x;
    const uint32_t c = r < n_regions ? region_count[r] : 0u;
    const uint32_t q = (c + kChunk - 1) / kChunk;
    uint32_t total;
    const uint32_t ex_e = block_exclusive_scan<1024>(c, &total, sm);
    if (r < n_regions) region_start[r] = carry_e + ex_e;
    carry_e += total;
    const uint32_t ex_c = block_exclusive_scan<1024>(q, &total, sm);
    if (r < n_regions) {
      chunk_base[r] = carry_c + ex_c;
      for (uint32_t k = 0; k < q; ++k)
        if (RM_INDEX_OK(carry_c + ex_c + k, RM_X_CHUNKS, 10)) chunk_region[carry_c + ex_c + k] = r;
    }
    carry_c += total;
  }
  if (threadIdx.x == 0) {
    region_start[n_regions] = carry_e;
    chunk_base[n_regions] = carry_c;
  }
}

// 32 x 32 bit transpose across the warp: lane l ends with bit i = bit l of lane i's word.
__device__ __forceinline__ uint32_t warp_bit_transpose(uint32_t a) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 16; j >= 1; j >>= 1) {
    const uint32_t m = j == 16 ? 0x0000FFFFu : j == 8 ? 0x00FF00FFu : j == 4 ? 0x0F0F0F0Fu : j == 2 ? 0x33333333u
                                                                                                    : 0x55555555u;
    const uint32_t b = __shfl_xor_sync(0xffffffffu, a, j);
    a = (lane & j) ? (((b >> j) & m) | (a & ~m)) : ((a & m) | ((b & m) << j));
  }
  return a;
}

struct ChunkSpan {
  uint32_t begin, end;  // entries [begin, end) of the sorted entry array
  uint32_t region;
};
__device__ __forceinline__ bool chunk_span(uint32_t chunk, const uint32_t* __restrict__ region_start,
                                           const uint32_t* __restrict__ chunk_base,
                                           const uint32_t* __restrict__ chunk_region, uint32_t n_regions,
                                           ChunkSpan* sp) {
  if (chunk >= chunk_base[n_regions]) return false;
  if (!RM_INDEX_OK(chunk, RM_X_CHUNKS, 10)) return false;
  const uint32_t r = chunk_region[chunk];
  if (!RM_INDEX_OK(r, RM_X_REGIONS, 11)) return false;
  const uint32_t k = chunk - chunk_base[r];
  sp->region = r;
  sp->begin = region_start[r] + k * kChunk;
  sp->end = min(sp->begin + (uint32_t)kChunk, region_start[r + 1]);
  if (sp->end > sp->begin && !RM_INDEX_OK(sp->end - 1, RM_X_PAIRS, 9)) return false;
  return true;
}

// count pass: chunk_cursor[chunk][lane] = number of the chunk's entries covering the lane's tile
__global__ void __launch_bounds__(kFineThreads)
k_fine_count(const uint2* __restrict__ entries, const uint32_t* __restrict__ region_start,
             const uint32_t* __restrict__ chunk_base, const uint32_t* __restrict__ chunk_region, uint32_t n_regions,
             uint32_t* __restrict__ chunk_cursor) {
  const int lane = threadIdx.x & 31;
  const uint32_t chunk = blockIdx.x * kFineWarps + (threadIdx.x >> 5);
  ChunkSpan sp;
  if (!chunk_span(chunk, region_start, chunk_base, chunk_region, n_regions, &sp)) return;
  uint32_t count = 0;
  for (uint32_t e0 = sp.begin; e0 < sp.end; e0 += 32) {
    const uint32_t e = e0 + lane;
    const uint32_t mask = e < sp.end ? __ldg(&entries[e].y) : 0u;
    count += __popc(warp_bit_transpose(mask));
  }
  chunk_cursor[(size_t)chunk * 32 + lane] = count;
}

// One warp per region: exclusive scan of the chunk counts along the region's chunks, starting
// at the first list position of the lane's tile.
__global__ void __launch_bounds__(kFineThreads)
k_fine_cursors(const uint32_t* __restrict__ chunk_base, uint32_t n_regions, int reg_w, int grid_w, int grid_h,
               const uint32_t* __restrict__ tile_start, uint32_t* __restrict__ chunk_cursor) {
  const int lane = threadIdx.x & 31;
  const uint32_t r = blockIdx.x * kFineWarps + (threadIdx.x >> 5);
  if (r >= n_regions) return;
  const int gy = (int)(r / (uint32_t)reg_w), gx = (int)(r - (uint32_t)gy * (uint32_t)reg_w);
  const int tx = gx * kRegW + (lane & (kRegW - 1)), ty = gy * kRegH + (lane >> kRegShiftX);
  uint32_t pos = (tx < grid_w && ty < grid_h && RM_INDEX_OK((int64_t)ty * grid_w + tx, RM_X_TILES, 12))
                     ? tile_start[(int64_t)ty * grid_w + tx] : 0u;
  const uint32_t q1 = chunk_base[r + 1];
  constexpr int kBatch = 8;  // independent loads in flight per step of the serial scan
  for (uint32_t q = chunk_base[r]; q < q1; q += kBatch) {
    uint32_t c[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) c[k] = q + k < q1 ? chunk_cursor[(size_t)(q + k) * 32 + lane] : 0u;
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      if (q + k < q1) chunk_cursor[(size_t)(q + k) * 32 + lane] = pos;
      pos += c[k];
    }
  }
}

// write pass: the warp appends, tile by tile, the tet ids of the round's 32 entries that cover
// the tile.  For tile l the covering entries are the lanes whose mask has bit l (one ballot); they
// store their tet id at the tile's cursor plus their position among the covering lanes, so the ids
// of one tile leave as one contiguous store.
__global__ void __launch_bounds__(kFineThreads)
k_fine_write(const uint2* __restrict__ entries, const uint32_t* __restrict__ region_start,
             const uint32_t* __restrict__ chunk_base, const uint32_t* __restrict__ chunk_region, uint32_t n_regions,
             const uint32_t* __restrict__ chunk_cursor, uint32_t n_keys, int32_t* __restrict__ sorted_idx) {
  const int lane = threadIdx.x & 31;
  const uint32_t lt = (1u << lane) - 1u;
  const uint32_t chunk = blockIdx.x * kFineWarps + (threadIdx.x >> 5);
  ChunkSpan sp;
  if (!chunk_span(chunk, region_start, chunk_base, chunk_region, n_regions, &sp)) return;
  uint32_t c = chunk_cursor[(size_t)chunk * 32 + lane];  // next list position of this lane's tile
  uint2 nxt = make_uint2(0u, 0u);
  if (sp.begin + lane < sp.end) nxt = __ldg(entries + sp.begin + lane);
  for (uint32_t e0 = sp.begin; e0 < sp.end; e0 += 32) {
    const uint2 en = nxt;
    const uint32_t e_next = e0 + 32 + lane;
    nxt = make_uint2(0u, 0u);
    if (e_next < sp.end) nxt = __ldg(entries + e_next);  // in flight while this round is written
    uint32_t appended = 0;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
      const bool covers = (en.y >> l) & 1u;
      const uint32_t col = __ballot_sync(0xffffffffu, covers);
      const uint32_t pos = __shfl_sync(0xffffffffu, c, l) + __popc(col & lt);
      // pos < n_keys always holds when the masks agree with the tile populations; the test keeps a
      // disagreement from writing outside the list array
      if (covers && pos < n_keys && RM_INDEX_OK(pos, RM_X_LIST, 8)) sorted_idx[pos] = (int32_t)en.x;
      if (lane == l) appended = __popc(col);
    }
    c += appended;
  }
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
  // a band-restricted frame compacts the visible tets from buffer b to buffer a before ranking them
  const bool banded = cam->tile_row_begin > 0 || cam->tile_row_end < gh;
  *depth_keys = reinterpret_cast<uint32_t*>(b + (banded ? L.keys_b : L.keys_a));
  *order_in = reinterpret_cast<uint32_t*>(b + (banded ? L.ord_b : L.ord_a));
  *tile_diff = reinterpret_cast<int32_t*>(b + L.tile_diff);
  RM_CUDA_CHECK(cudaMemsetAsync(b + L.tile_diff, 0, 4 * (size_t)(gh + 1) * (gw + 1), st));
  RM_CUDA_CHECK(cudaMemsetAsync(b + L.cursor, 0, 4 * (size_t)(G + 1), st));
  RM_CUDA_CHECK(cudaMemsetAsync(info, 0, sizeof(RmBinInfo), st));
  return RM_OK;
}

static int launch_scan(const uint32_t* in, const uint32_t* gather, const int4* rect, int64_t n, const int32_t* n_dev,
                       uint32_t* bsum, uint32_t* out, int inclusive, unsigned long long* total64, cudaStream_t st) {
  if (n <= 0) {
    if (total64) RM_CUDA_CHECK(cudaMemsetAsync(total64, 0, 8, st));
    return RM_OK;
  }
  int64_t nb = (n + rm::kScanTile - 1) / rm::kScanTile;
  // with a gather the values are fetched once, left in `out`, and scanned there in place
  const bool stash = gather != nullptr;
  rm_count_launch(), rm::k_scan_block_sums<<<(unsigned)nb, rm::kScanThreads, 0, st>>>(in, gather, rect, n, n_dev, bsum,
                                                                                       stash ? out : nullptr);
  rm_count_launch(), rm::k_scan_sums<<<1, 1024, 0, st>>>(bsum, nb, total64);
  if (stash) rm_count_launch(), rm::k_scan_apply<<<(unsigned)nb, rm::kScanThreads, 0, st>>>(out, nullptr, nullptr, n, bsum, out, inclusive);
  else rm_count_launch(), rm::k_scan_apply<<<(unsigned)nb, rm::kScanThreads, 0, st>>>(in, gather, rect, n, bsum, out, inclusive);
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

// After k_project: rank the tets, build tile_ranges, the rank-ordered inclusive
// scan of tiles_touched, and the info block.
int rm_launch_bin_finish(int64_t T, const RmCamera* cam, const int32_t* rect, int32_t* tile_ranges,
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

  rm_set_extent(RM_X_TETS, T, st);
  rm_set_extent(RM_X_TILES, G, st);
  // 1. rank the tets by (depth bits, id): four stable radix passes that start and end in buffer 0; culled
  //    tets carry key 0xFFFFFFFF and sort last.  A band-restricted frame sees a fraction of the tets, and
  //    every rank of a band-split job would still sort all T of them: there k_project left its pairs in
  //    buffer 1, a stable compaction moves the visible ones to the front of buffer 0, and the passes run over
  //    those only (their number is known on the device: info->n_visible).  Ranks past the visible tets then
  //    hold nothing that later stages read.
  if (T > 0) {
    RmProfScope prof("rank_tets_radix_sort", st);
    const bool banded = cam->tile_row_begin > 0 || cam->tile_row_end < gh;
    const int32_t* n_sort = banded ? &info->n_visible : nullptr;
    if (banded) {
      const int64_t nbc = (T + rm::kScanTile - 1) / rm::kScanTile;
      rm_count_launch(), rm::k_compact_count<<<(unsigned)nbc, rm::kScanThreads, 0, st>>>(keys[1], T, bsum);
      rm_count_launch(), rm::k_scan_sums<<<1, 1024, 0, st>>>(bsum, nbc, nullptr);
      rm_count_launch(), rm::k_compact_scatter<<<(unsigned)nbc, rm::kScanThreads, 0, st>>>(keys[1], ord[1], T, bsum, keys[0],
                                                                                   ord[0]);
    }
    for (int pass = 0; pass < 4; ++pass) {
      int src = pass & 1, dst = src ^ 1;
      int shift = pass * rm::kRadixBits;
      rm_count_launch(), rm::k_radix_hist<<<L.nblk_sort, rm::kSortThreads, 0, st>>>(keys[src], T, n_sort, shift, hist,
                                                                              L.nblk_sort);
      rm_count_launch(), rm::k_radix_rowscan<<<rm::kRadix, 1024, 0, st>>>(hist, L.nblk_sort, dtot);
      rm_count_launch(), rm::k_radix_scatter<<<L.nblk_sort, rm::kSortThreads, 0, st>>>(
          keys[src], ord[src], T, n_sort, shift, hist, dtot, L.nblk_sort, keys[dst], ord[dst]);
    }
    RM_CUDA_CHECK(cudaPeekAtLastError());
  }
  // 2. tile populations -> tile_ranges
  {
    RmProfScope prof("tile_ranges(6 launches)", st);
    int rows_per_block = 4;  // 128 threads
    rm_count_launch(), rm::k_diff_prefix_x<<<(gh + 1 + rows_per_block - 1) / rows_per_block, 32 * rows_per_block, 0, st>>>(diff, gh, gw);
    rm_count_launch(), rm::k_diff_prefix_y<<<(gw + rows_per_block - 1) / rows_per_block, 32 * rows_per_block, 0, st>>>(diff, gh, gw,
                                                                                                  tcount);
    int rc = launch_scan(tcount, nullptr, nullptr, G, nullptr, bsum, tstart, 0, total_keys, st);
    if (rc) return rc;
    rm_count_launch(), rm::k_write_ranges<<<(unsigned)((G + 255) / 256), 256, 0, st>>>(tcount, tstart, G,
                                                                    reinterpret_cast<int2*>(tile_ranges));
    RM_CUDA_CHECK(cudaPeekAtLastError());
  }
  // 3. inclusive scan, in rank order, of the number of regions every tet touches (culled tets
  //    have an empty rectangle and sort last)
  {
    RmProfScope prof("rank_order_scan(4 launches)", st);
    int rc = launch_scan(nullptr, ord[0], reinterpret_cast<const int4*>(rect), T, &info->n_visible, bsum, cum, 1,
                         total_keys + 1, st);
    if (rc) return rc;
    rm_count_launch(), rm::k_finish_info<<<1, 1, 0, st>>>(info, total_keys);
    RM_CUDA_CHECK(cudaPeekAtLastError());
  }
  return RM_OK;
}

namespace {
struct ListPlan {
  int reg_w, reg_h, bits1, bits2, nblk;
  uint32_t n_regions, n_regions_smem, max_chunks;
  size_t pairs_a, pairs_b, entries, hist, dtot, starts, region_count, region_start, chunk_base, chunk_region, chunk_cursor,
      total;
};
constexpr uint32_t kMaxSmemRegions = 16384;  // 64 KB of per-block region counters
// region grid, split of the region-id bits into the two digits, and the scratch layout
bool make_list_plan(int64_t n_region_keys, int gh, int gw, ListPlan* P) {
  P->reg_w = (gw + rm::kRegW - 1) / rm::kRegW;
  P->reg_h = (gh + rm::kRegH - 1) / rm::kRegH;
  const int64_t R = (int64_t)P->reg_w * P->reg_h;
  int bits = 1;
  while (((int64_t)1 << bits) < R) ++bits;
  if (bits > 22 || n_region_keys > 0x7fffffffll) return false;
  P->n_regions = (uint32_t)R;
  P->n_regions_smem = P->n_regions <= kMaxSmemRegions ? P->n_regions : 0u;
  P->bits1 = bits <= 11 ? bits : (bits + 1) / 2;
  P->bits2 = bits - P->bits1;
  P->nblk = (int)((n_region_keys + rm::kBinTile - 1) / rm::kBinTile);
  P->max_chunks = (uint32_t)(n_region_keys / rm::kChunk + R + 1);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align256(off + bytes);
    return o;
  };
  P->pairs_a = take(8 * (size_t)n_region_keys);
  P->pairs_b = take(P->bits2 ? 8 * (size_t)n_region_keys : 0);
  P->entries = take(8 * (size_t)n_region_keys);
  P->hist = take(4 * ((size_t)1 << P->bits1) * (size_t)(P->nblk > 0 ? P->nblk : 1));
  P->dtot = take(4 * ((size_t)1 << P->bits1));
  P->starts = take(4 * (size_t)(P->nblk > 0 ? P->nblk : 1));
  P->region_count = take(4 * (size_t)(R + 1));
  P->region_start = take(4 * (size_t)(R + 1));
  P->chunk_base = take(4 * (size_t)(R + 1));
  P->chunk_region = take(4 * (size_t)P->max_chunks);
  P->chunk_cursor = take(4 * 32 * (size_t)P->max_chunks);
  P->total = off;
  return true;
}
}  // namespace

size_t rm_list_plan_bytes(int64_t n_region_keys, int gh, int gw) {
  ListPlan P;
  if (!make_list_plan(n_region_keys, gh, gw, &P)) return 0;
  return P.total;
}

int rm_launch_build_lists(const int32_t* rect, const int32_t* tile_ranges, int64_t T, const RmCamera* cam,
                          int64_t n_keys, int64_t n_region_keys, void* ws, void* scratch, size_t scratch_bytes,
                          int32_t* sorted_idx, cudaStream_t st) {
  (void)tile_ranges;
  if (n_keys == 0) return RM_OK;
  const int gh = cam->grid_height, gw = cam->grid_width;
  const int64_t G = (int64_t)gh * gw;
  BinLayout L = make_layout(T, G, gh, gw);
  ListPlan P;
  if (n_region_keys < 1 || n_region_keys > n_keys || !make_list_plan(n_region_keys, gh, gw, &P))
    return RM_ERR_INVALID_ARG;
  if (P.total > scratch_bytes || (reinterpret_cast<uintptr_t>(scratch) & 255)) return RM_ERR_WORKSPACE;
  rm_set_extent(RM_X_TETS, T, st);
  rm_set_extent(RM_X_TILES, G, st);
  rm_set_extent(RM_X_LIST, n_keys, st);
  rm_set_extent(RM_X_PAIRS, n_region_keys, st);
  rm_set_extent(RM_X_CHUNKS, P.max_chunks, st);
  rm_set_extent(RM_X_REGIONS, P.n_regions, st);
  char* b = static_cast<char*>(ws);
  const uint32_t* order = reinterpret_cast<uint32_t*>(b + L.ord_a);
  const uint32_t* cum = reinterpret_cast<uint32_t*>(b + L.cum);
  const uint32_t* tile_start = reinterpret_cast<uint32_t*>(b + L.tile_start);
  char* sb = static_cast<char*>(scratch);
  uint2* pairs_a = reinterpret_cast<uint2*>(sb + P.pairs_a);
  uint2* pairs_b = reinterpret_cast<uint2*>(sb + P.pairs_b);
  uint2* entries = reinterpret_cast<uint2*>(sb + P.entries);
  uint32_t* hist = reinterpret_cast<uint32_t*>(sb + P.hist);
  uint32_t* dtot = reinterpret_cast<uint32_t*>(sb + P.dtot);
  uint32_t* starts = reinterpret_cast<uint32_t*>(sb + P.starts);
  uint32_t* region_count = reinterpret_cast<uint32_t*>(sb + P.region_count);
  uint32_t* region_start = reinterpret_cast<uint32_t*>(sb + P.region_start);
  uint32_t* chunk_base = reinterpret_cast<uint32_t*>(sb + P.chunk_base);
  uint32_t* chunk_region = reinterpret_cast<uint32_t*>(sb + P.chunk_region);
  uint32_t* chunk_cursor = reinterpret_cast<uint32_t*>(sb + P.chunk_cursor);
  const uint32_t bins1 = 1u << P.bits1, bins2 = 1u << P.bits2;
  const int4* rect4 = reinterpret_cast<const int4*>(rect);
  const size_t gen = 4 * (rm::kBinTile + 4 + 16) + 2 * rm::kBinTile;
  const size_t smem_h1 = gen + 4 * bins1 + 4 * (size_t)P.n_regions_smem;
  const size_t smem_s1 = 8 * rm::kBinTile + 4 * bins1 * (2 + rm::kBinWarps) + 64;
  const size_t smem_s2 = 8 * rm::kBinTile + 4 * bins2 * (2 + rm::kBinWarps) + 64;
  RM_CUDA_CHECK(cudaFuncSetAttribute(rm::k_region_hist1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_h1));
  RM_CUDA_CHECK(cudaFuncSetAttribute(rm::k_region_scatter, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)(smem_s1 > smem_s2 ? smem_s1 : smem_s2)));
  RM_CUDA_CHECK(cudaMemsetAsync(region_count, 0, 4 * (size_t)(P.n_regions + 1), st));
  {
    RmProfScope prof("k_block_start_ranks+k_region_hist1", st);
    rm_count_launch(), rm::k_block_start_ranks<<<(P.nblk + 255) / 256, 256, 0, st>>>(cum, (int)T, P.nblk, starts);
    rm_count_launch(), rm::k_region_hist1<<<P.nblk, rm::kBinThreads, smem_h1, st>>>(cum, starts, order, (int)T, rect4, P.reg_w,
                                                                n_region_keys, bins1, hist, P.nblk,
                                                                P.n_regions_smem, region_count, pairs_a);
  }
  {
    RmProfScope prof("k_radix_rowscan+k_region_scatter(pass 1)", st);
    rm_count_launch(), rm::k_radix_rowscan<<<bins1, 1024, 0, st>>>(hist, P.nblk, dtot);
    rm_count_launch(), rm::k_region_scatter<<<P.nblk, rm::kBinThreads, smem_s1, st>>>(pairs_a, n_region_keys, 0, bins1, hist, dtot,
                                                                  P.nblk, P.bits2 == 0, rect4, P.reg_w, pairs_b,
                                                                  entries);
  }
  RM_CUDA_CHECK(cudaPeekAtLastError());
  if (P.bits2) {
    {
      RmProfScope prof("k_region_hist2", st);
      rm_count_launch(), rm::k_region_hist2<<<P.nblk, rm::kBinThreads, 4 * bins2, st>>>(pairs_b, n_region_keys, P.bits1, bins2, hist,
                                                                    P.nblk);
    }
    {
      RmProfScope prof("k_radix_rowscan+k_region_scatter(pass 2)", st);
      rm_count_launch(), rm::k_radix_rowscan<<<bins2, 1024, 0, st>>>(hist, P.nblk, dtot);
      rm_count_launch(), rm::k_region_scatter<<<P.nblk, rm::kBinThreads, smem_s2, st>>>(pairs_b, n_region_keys, P.bits1, bins2, hist,
                                                                    dtot, P.nblk, 1, rect4, P.reg_w, nullptr, entries);
    }
    RM_CUDA_CHECK(cudaPeekAtLastError());
  }
  const unsigned chunk_blocks = (P.max_chunks + rm::kFineWarps - 1) / rm::kFineWarps;
  {
    RmProfScope prof("k_region_layout", st);
    rm_count_launch(), rm::k_region_layout<<<1, 1024, 0, st>>>(region_count, P.n_regions, region_start, chunk_base, chunk_region);
  }
  {
    RmProfScope prof("k_fine_count", st);
    rm_count_launch(), rm::k_fine_count<<<chunk_blocks, rm::kFineThreads, 0, st>>>(entries, region_start, chunk_base, chunk_region,
                                                               P.n_regions, chunk_cursor);
  }
  {
    RmProfScope prof("k_fine_cursors", st);
    rm_count_launch(), rm::k_fine_cursors<<<(P.n_regions + rm::kFineWarps - 1) / rm::kFineWarps, rm::kFineThreads, 0, st>>>(
        chunk_base, P.n_regions, P.reg_w, gw, gh, tile_start, chunk_cursor);
  }
  {
    RmProfScope prof("k_fine_write", st);
    rm_count_launch(), rm::k_fine_write<<<chunk_blocks, rm::kFineThreads, 0, st>>>(entries, region_start, chunk_base, chunk_region,
                                                               P.n_regions, chunk_cursor, (uint32_t)n_keys, sorted_idx);
  }
  RM_CUDA_CHECK(cudaPeekAtLastError());
  return RM_OK;
}

unsigned rm_bounds_status_binning() { return rm_take_bounds_status(); }
