// points -> octree on the device, for a whole batch of clouds at once.
//
// What the reference does per cloud on one CPU core (Octree::build, octree/octree/octree.cpp:74-121)
// and then per batch (merge_octrees, octree/octree/merge_octrees.cpp:7-198) is done here in one
// pass over all clouds: every point gets the composite key  (cloud << 3*depth) | morton(cell),
// one stable LSD radix sort orders all clouds at once (equal to the reference's std::sort of
// (key, index) pairs per cloud), and each level is then a segmented "unique" of the level below.
// The composite key of a level-d node is also its rank basis: ranks in the batch-wide unique list
// are exactly the rebased child indices that merge_octrees produces.
//
// Phase 1 (plan) leaves in the workspace, for d = full..depth, the sorted unique composite keys
// Kd of the non-empty nodes and, for each such node, where its children (or its points, at the
// finest level) start in the list below.  One device->host copy of the per-level counts follows;
// the caller allocates the exact output.  Phase 2 (emit) writes header, keys, children, split
// labels, finest-level signal and — for a merged batch — the neighbour table.
//
// All scans are reduce-then-scan over a fixed grid (no inter-block waiting anywhere).
// This file is compiled with --fmad=false: the signal must round exactly like the reference's
// separate multiplies and adds (octree.cpp:330-348).
#include <cstring>
#include <vector>

#include "header.h"

namespace ocnn {
namespace {

constexpr int kThreads = 256;
constexpr int kScanItems = 4;
constexpr int kScanTile = kThreads * kScanItems;
constexpr int kMaxScanGrid = kSMs * 4;   // 592 blocks: 4 CTAs of 256 threads per SM
constexpr int kSortItems = 8;            // keys per thread per sort tile
constexpr int kSortTile = kThreads * kSortItems;   // 2048 keys

// One entry per cloud (plus a sentinel holding the total point count), uploaded by the plan call.
struct CloudRef {
  const float* xyz;
  const float* normal;
  const float* feat;
  const float* label;
  long long offset;     // index of the cloud's first point in the batch-wide numbering
};

// ---- workspace layout --------------------------------------------------------------------------
struct Layout {
  int64_t n;            // total points
  int batch, depth, full;
  int key_bytes_sort;   // 4 or 8: width of the sort key
  int nvb;              // sort: number of CTAs, each owning one contiguous chunk of the keys
  int vchunk;           // sort: keys per CTA chunk (multiple of the 2048-key tile)
  int64_t cap[OCNN_MAX_DEPTH + 1];   // capacity of Kd
  size_t off_offsets, off_counts, off_blockcnt, off_hist, off_bintot;
  size_t off_keys[2], off_idx[2];
  size_t off_K[OCNN_MAX_DEPTH + 1], off_start[OCNN_MAX_DEPTH + 2];
  size_t total;
};

size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

int bits_for(int64_t v) {  // number of bits needed to represent values 0..v-1
  int b = 0;
  while ((1LL << b) < v) ++b;
  return b;
}

Layout make_layout(int64_t n, int batch, int depth, int full) {
  Layout L;
  memset(&L, 0, sizeof(L));
  L.n = n; L.batch = batch; L.depth = depth; L.full = full;
  L.key_bytes_sort = (3 * depth + bits_for(batch) <= 32) ? 4 : 8;
  int64_t nvb = (n + kSortTile - 1) / kSortTile;       // one tile per CTA until the grid is 4 waves
  if (nvb < 1) nvb = 1;
  if (nvb > kSMs * 4) nvb = kSMs * 4;
  int64_t vchunk = (n + nvb - 1) / nvb;
  vchunk = (vchunk + kSortTile - 1) / kSortTile * kSortTile;
  nvb = (n + vchunk - 1) / vchunk;                   // drop chunks the rounding left empty
  L.nvb = (int)nvb;
  L.vchunk = (int)vchunk;
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t at = o; o = align_up(o + bytes); return at; };
  L.off_offsets = take(sizeof(CloudRef) * (size_t)(batch + 1));
  L.off_counts = take(sizeof(int) * 32);
  L.off_blockcnt = take(sizeof(int) * kMaxScanGrid);
  L.off_hist = take(sizeof(int) * 256 * (size_t)L.nvb);
  L.off_bintot = take(sizeof(int) * 256 * 8);      // one row of digit totals per sort pass (<= 8)
  for (int i = 0; i < 2; ++i) L.off_keys[i] = take((size_t)L.key_bytes_sort * (size_t)n);
  for (int i = 0; i < 2; ++i) L.off_idx[i] = take(sizeof(uint32_t) * (size_t)n);
  for (int d = full; d <= depth; ++d) {
    int64_t full_nodes = d >= 20 ? INT64_MAX : (int64_t)batch << (3 * d);
    L.cap[d] = n < full_nodes ? n : full_nodes;
    L.off_K[d] = take(sizeof(uint64_t) * (size_t)L.cap[d]);
    // start[d][a]: first entry, in the list below Kd (K(d+1), or the sorted points for d = depth),
    // that belongs to node a of Kd
    L.off_start[d] = take(sizeof(int) * (size_t)(L.cap[d] + 1));
  }
  L.total = o;
  return L;
}

// ---- Morton -------------------------------------------------------------------------------------
// bit i of v -> bit 3i for v < 2^21 (octree/octree/octree_nn.cpp:551-560 interleaves x,y,z so)
__device__ __forceinline__ uint64_t spread3(uint32_t v) {
  uint64_t x = v & 0x1fffffu;
  x = (x | (x << 32)) & 0x001f00000000ffffULL;
  x = (x | (x << 16)) & 0x001f0000ff0000ffULL;
  x = (x | (x << 8)) & 0x100f00f00f00f00fULL;
  x = (x | (x << 4)) & 0x10c30c30c30c30c3ULL;
  x = (x | (x << 2)) & 0x1249249249249249ULL;
  return x;
}

struct EncodeArgs {
  const CloudRef* clouds;   // device table, batch + 1 entries
  int batch, depth;
  long long n;
  float bbmin[3];
  float mul;
};

__device__ __forceinline__ int cloud_of(const CloudRef* clouds, int batch, long long i) {
  int lo = 0, hi = batch;          // clouds[lo].offset <= i < clouds[hi].offset
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (clouds[mid].offset <= i) lo = mid; else hi = mid;
  }
  return lo;
}

// normalize_pts + sort_keys' key computation (octree.cpp:155-170, 180-186): cell = trunc((p -
// bbmin) * mul), only `depth` bits per axis enter the key.
template <typename KeyT>
__global__ void encode_kernel(EncodeArgs a, KeyT* __restrict__ keys, int* __restrict__ bintot,
                              int bintot_n) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  // the sort's per-pass digit totals start at zero (the histogram kernels add into them)
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < bintot_n; i += blockDim.x) bintot[i] = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = cloud_of(a.clouds, a.batch, i);
    const float* xyz = a.clouds[b].xyz + 3 * (i - a.clouds[b].offset);
    const uint32_t mask = (1u << a.depth) - 1u;
    uint32_t c[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const float s = (xyz[j] - a.bbmin[j]) * a.mul;
      c[j] = (uint32_t)s & mask;
    }
    const uint64_t key = (spread3(c[0]) << 2) | (spread3(c[1]) << 1) | spread3(c[2]);
    keys[i] = (KeyT)(((uint64_t)b << (3 * a.depth)) | key);
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// ---- stable LSD radix sort, 8 bits per pass -------------------------------------------------------
// Each CTA owns one contiguous chunk of the keys.  A pass is: per-CTA digit histogram -> exclusive
// scan over (digit, CTA) -> stable scatter.  The scatter works in tiles of 2048 keys: every warp
// ranks its 256 keys 32 at a time with match_any (stable inside the warp), the per-warp digit counts
// are prefixed across warps and digits, the tile is written to shared memory in digit order, and
// only then copied out — consecutive threads then write consecutive global addresses of one digit
// run, so the 4-byte scatter of the naive formulation becomes coalesced runs.
template <typename KeyT>
__global__ void __launch_bounds__(kThreads) sort_hist_kernel(const KeyT* __restrict__ keys,
                                                             long long n, int shift, int vchunk,
                                                             int nvb, int* __restrict__ hist,
                                                             int* __restrict__ bintot) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  // one private histogram per warp (shared-memory atomics never cross warps), summed at the end
  __shared__ int sh[kThreads / 32][256];
  const int warp = threadIdx.x >> 5;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) sh[w][threadIdx.x] = 0;
  __syncthreads();
  const long long beg = (long long)blockIdx.x * vchunk;
  long long end = beg + vchunk;
  if (end > n) end = n;
  // Eight keys per thread are requested before the first is counted.  Keys that are close in
  // memory often share the digit (the input is sorted by the lower digits, and the top digit is
  // the cloud index): a run of equal digits in consecutive lanes is added once, by its first lane.
  const int lane = threadIdx.x & 31;
  for (long long i0 = beg; i0 < end; i0 += 8 * kThreads) {
    KeyT k[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const long long i = i0 + u * kThreads + threadIdx.x;
      k[u] = i < end ? keys[i] : 0;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const long long i = i0 + u * kThreads + threadIdx.x;
      // lanes past the end carry digit 256, which no counted lane has
      const int digit = i < end ? (int)((k[u] >> shift) & 255) : 256;
      const int prev = __shfl_up_sync(0xffffffffu, digit, 1);
      const bool head = lane == 0 || prev != digit;
      const unsigned heads = __ballot_sync(0xffffffffu, head);
      if (head && digit < 256) {
        // the run ends before the next head (or at the end of the warp)
        const unsigned later = lane == 31 ? 0u : (heads >> (lane + 1));
        const int run = later ? __ffs(later) : 32 - lane;
        atomicAdd(&sh[warp][digit], run);
      }
    }
  }
  __syncthreads();
  int total = 0;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) total += sh[w][threadIdx.x];
  hist[(long long)threadIdx.x * nvb + blockIdx.x] = total;
  // digit totals over all CTAs (integer additions: the order does not matter); bintot was cleared
  // by the encode kernel
  if (total) atomicAdd(&bintot[threadIdx.x], total);
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// Exclusive scan of hist[256][nvb] in (digit, CTA) order: one CTA per digit row (sort_rowscan_kernel
// below); the digit totals it starts from were accumulated by the histogram kernel.
__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
  // exclusive prefix of v over the CTA's kThreads threads
  __shared__ int wsum[kThreads / 32];
  __shared__ int wtot;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();   // protects wsum/wtot of a previous call
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < kThreads / 32 ? wsum[lane] : 0;
    int winc = w;
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < kThreads / 32) wsum[lane] = winc - w;
    if (lane == kThreads / 32 - 1) wtot = winc;
  }
  __syncthreads();
  *total = wtot;
  return inc - v + wsum[warp];
}

__global__ void __launch_bounds__(kThreads) sort_rowscan_kernel(int* __restrict__ hist, int nvb,
                                                                const int* __restrict__ bintot) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  // first slot of this digit = number of keys with a smaller digit (kThreads == 256 digits)
  int below_total;
  block_exclusive_scan(threadIdx.x < blockIdx.x ? bintot[threadIdx.x] : 0, &below_total);
  int base = below_total;
  int* row = hist + (long long)blockIdx.x * nvb;
  for (int i0 = 0; i0 < nvb; i0 += kThreads) {
    const int i = i0 + threadIdx.x;
    const int v = i < nvb ? row[i] : 0;
    int total;
    const int ex = block_exclusive_scan(v, &total);
    if (i < nvb) row[i] = base + ex;
    base += total;
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// The lanes of `mask` whose 8-bit digit equals this lane's: eight ballots, one per bit.  (Measured
// several times faster here than match.any, which the histogram used to spend most of its time in.)
__device__ __forceinline__ unsigned match_digit(unsigned mask, int digit) {
  unsigned peers = mask;
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const bool bit = (digit >> b) & 1;
    const unsigned with = __ballot_sync(mask, bit);
    peers &= bit ? with : ~with;
  }
  return peers;
}

template <typename KeyT, bool FIRST>
__global__ void __launch_bounds__(kThreads) sort_scatter_kernel(
    const KeyT* __restrict__ keys_in, const uint32_t* __restrict__ idx_in,
    KeyT* __restrict__ keys_out, uint32_t* __restrict__ idx_out, long long n, int shift,
    int vchunk, int nvb, const int* __restrict__ hist) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  constexpr int kWarps = kThreads / 32;
  __shared__ int cnt[kWarps][256];        // per-warp digit counts, then per-warp digit bases
  __shared__ int tile_start[256];         // first slot of each digit inside the sorted tile
  __shared__ int gofs[256];               // next global slot of each digit for this CTA
  __shared__ KeyT skey[kSortTile];
  __shared__ uint32_t sidx[kSortTile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  gofs[threadIdx.x] = hist[(long long)threadIdx.x * nvb + blockIdx.x];
  const long long beg = (long long)blockIdx.x * vchunk;
  long long end = beg + vchunk;
  if (end > n) end = n;
  for (long long t0 = beg; t0 < end; t0 += kSortTile) {
    const int tile_n = (int)((end - t0) < kSortTile ? (end - t0) : kSortTile);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) cnt[w][threadIdx.x] = 0;
    __syncthreads();
    // 1. rank inside the warp's 256 keys (index order = rank order: stable)
    KeyT key[kSortItems];
    uint32_t idx[kSortItems];
    int rank[kSortItems];
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {      // all loads of the tile first: one latency, not 8
      const int local = warp * (32 * kSortItems) + r * 32 + lane;
      key[r] = 0;
      idx[r] = 0;
      if (local < tile_n) {
        key[r] = keys_in[t0 + local];
        idx[r] = FIRST ? (uint32_t)(t0 + local) : idx_in[t0 + local];
      }
    }
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
      const int local = warp * (32 * kSortItems) + r * 32 + lane;
      const bool valid = local < tile_n;
      const unsigned mask = __ballot_sync(0xffffffffu, valid);
      rank[r] = -1;
      if (valid) {
        const int digit = (int)((key[r] >> shift) & 255);
        const unsigned peers = match_digit(mask, digit);
        const int before = __popc(peers & ((1u << lane) - 1));
        rank[r] = cnt[warp][digit] + before;
        __syncwarp(mask);
        if (before == 0) cnt[warp][digit] += __popc(peers);
      }
      __syncwarp();
    }
    __syncthreads();
    // 2. thread d: prefix digit d over the warps, then over the digits
    int total_d = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int c = cnt[w][threadIdx.x];
      cnt[w][threadIdx.x] = total_d;
      total_d += c;
    }
    int tile_total;
    const int start_d = block_exclusive_scan(total_d, &tile_total);
    tile_start[threadIdx.x] = start_d;
    __syncthreads();
    // 3. tile into shared memory in digit order
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
      if (rank[r] >= 0) {
        const int digit = (int)((key[r] >> shift) & 255);
        const int pos = tile_start[digit] + cnt[warp][digit] + rank[r];
        skey[pos] = key[r];
        sidx[pos] = idx[r];
      }
    }
    __syncthreads();
    // 4. copy out: slot i of the sorted tile goes to gofs[digit] + (i - tile_start[digit])
    for (int i = threadIdx.x; i < tile_n; i += kThreads) {
      const KeyT k = skey[i];
      const int digit = (int)((k >> shift) & 255);
      const long long pos = (long long)gofs[digit] + (i - tile_start[digit]);
      keys_out[pos] = k;
      idx_out[pos] = sidx[i];
    }
    __syncthreads();
    gofs[threadIdx.x] += total_d;
    __syncthreads();
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// ---- segmented unique (reduce, then scan) ---------------------------------------------------------
// out = unique(in >> shift) for sorted `in`; start[a] = first i with (in[i] >> shift) == out[a];
// start[count] = n; *count_out = count.  n is read from n_ptr when given (a count produced on the
// device by the previous stage).
template <typename InT>
__device__ __forceinline__ bool is_head(const InT* __restrict__ in, long long i, int shift) {
  return i == 0 || (in[i] >> shift) != (in[i - 1] >> shift);
}

__device__ __forceinline__ void scan_range(long long n, long long* beg, long long* end) {
  long long chunk = (n + gridDim.x - 1) / gridDim.x;
  chunk = (chunk + kScanTile - 1) / kScanTile * kScanTile;
  *beg = (long long)blockIdx.x * chunk;
  long long e = *beg + chunk;
  *end = e < n ? e : n;
}

template <typename InT>
__global__ void __launch_bounds__(kThreads) unique_count_kernel(const InT* __restrict__ in,
                                                                const int* __restrict__ n_ptr,
                                                                long long n_host, int shift,
                                                                int* __restrict__ blockcnt) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  __shared__ int red[kThreads / 32];
  const long long n = n_ptr ? (long long)*n_ptr : n_host;
  long long beg, end;
  scan_range(n, &beg, &end);
  int c = 0;
  for (long long i = beg + threadIdx.x; i < end; i += kThreads) c += is_head(in, i, shift) ? 1 : 0;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < kThreads / 32; ++w) t += red[w];
    blockcnt[blockIdx.x] = t;
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

template <typename InT>
__global__ void __launch_bounds__(kThreads) unique_compact_kernel(
    const InT* __restrict__ in, const int* __restrict__ n_ptr, long long n_host, int shift,
    const int* __restrict__ blockcnt, uint64_t* __restrict__ out, int* __restrict__ start,
    int* __restrict__ count_out) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  __shared__ int red[kThreads / 32];
  __shared__ int base_s;
  const long long n = n_ptr ? (long long)*n_ptr : n_host;
  // base = heads in all lower blocks
  int c = 0;
  for (int g = threadIdx.x; g < (int)blockIdx.x; g += kThreads) c += blockcnt[g];
  for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < kThreads / 32; ++w) t += red[w];
    base_s = t;
  }
  __syncthreads();
  int base = base_s;
  long long beg, end;
  scan_range(n, &beg, &end);
  for (long long t0 = beg; t0 < end; t0 += kScanTile) {
    const long long i0 = t0 + (long long)threadIdx.x * kScanItems;
    bool head[kScanItems];
    int local = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
      head[k] = (i0 + k < end) && is_head(in, i0 + k, shift);
      local += head[k] ? 1 : 0;
    }
    int total;
    int at = base + block_exclusive_scan(local, &total);
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
      if (head[k]) {
        out[at] = (uint64_t)(in[i0 + k] >> shift);
        start[at] = (int)(i0 + k);
        ++at;
      }
    }
    base += total;
  }
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
    *count_out = base;
    start[base] = (int)n;
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// ---- emit ------------------------------------------------------------------------------------
struct EmitLevelArgs {
  uint8_t* out;               // octree buffer
  long long off_key, off_child, off_split;   // byte offsets of this level (split < 0: absent)
  int key_bytes;
  int d;
};

__device__ __forceinline__ void store_key(uint8_t* base, long long off, long long i, uint64_t local,
                                          int b, int key_bytes) {
  // batch index into the top lane of the key: byte 3 of a 32-bit key, uint16 lane 3 of a 64-bit
  // key (merge_octrees.cpp:127-131); a single octree has b = 0.
  if (key_bytes == 8) {
    reinterpret_cast<uint64_t*>(base + off)[i] = (local & 0x0000ffffffffffffULL) | ((uint64_t)(b & 0xffff) << 48);
  } else {
    reinterpret_cast<uint32_t*>(base + off)[i] = ((uint32_t)local & 0x00ffffffu) | ((uint32_t)(b & 0xff) << 24);
  }
}

// levels 0..full: every node exists; key = index inside its octree; child = itself below the
// full level, -1 at the full level (filled from K_full afterwards) — octree.cpp:210-224.
// All levels in one launch: a block serves one level (EmitAll::block0 is the first block of each).
struct EmitAll {
  int nlev, batch, full;
  int block0[OCNN_MAX_DEPTH + 2];
  long long nnum[OCNN_MAX_DEPTH + 1];
  EmitLevelArgs a[OCNN_MAX_DEPTH + 1];
  const uint64_t* Kp[OCNN_MAX_DEPTH + 1];     // K(d-1), levels above the full ones only
  const uint64_t* Kc[OCNN_MAX_DEPTH + 1];     // Kd
  const int* start[OCNN_MAX_DEPTH + 1];       // first entry of Kc under each parent
};

__device__ __forceinline__ void emit_full_node(const EmitLevelArgs& a, long long i, int batch, int full) {
  const long long per = 1LL << (3 * a.d);
  const int b = (int)(i / per);
  store_key(a.out, a.off_key, i, (uint64_t)(i - b * per), b, a.key_bytes);
  const int ch = a.d < full ? (int)i : -1;
  reinterpret_cast<int*>(a.out + a.off_child)[i] = ch;
  if (a.off_split >= 0) reinterpret_cast<float*>(a.out + a.off_split)[i] = ch < 0 ? 0.f : 1.f;
}

// children of the full level: the composite key of a level-`full` node IS its batch-wide node
// index, so child[K_full[r]] = r (octree.cpp:277-282 + the rebasing of merge_octrees.cpp:136-144).
__global__ void emit_full_children_kernel(EmitLevelArgs a, const uint64_t* __restrict__ K,
                                          const int* __restrict__ count) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  const int n = *count;
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
    const long long node = (long long)K[r];
    reinterpret_cast<int*>(a.out + a.off_child)[node] = r;
    if (a.off_split >= 0) reinterpret_cast<float*>(a.out + a.off_split)[node] = 1.f;
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// level d > full: node 8a+j is the j-th child slot of the a-th non-empty node of level d-1
// (octree.cpp:226-273).  Kp = K(d-1), Kc = Kd, start = first entry of Kc under each parent.
__global__ void __launch_bounds__(kThreads) emit_levels_kernel(const EmitAll A) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  int l = 0;
  while (l + 1 < A.nlev && (int)blockIdx.x >= A.block0[l + 1]) ++l;
  const EmitLevelArgs& a = A.a[l];
  const long long i = (long long)((int)blockIdx.x - A.block0[l]) * kThreads + threadIdx.x;
  if (i >= A.nnum[l]) return;          // (whole sibling groups leave together: nnum is a multiple of 8)
  if (a.d <= A.full) {
    emit_full_node(a, i, A.batch, A.full);
    return;
  }
  const uint64_t* __restrict__ Kp = A.Kp[l];
  const uint64_t* __restrict__ Kc = A.Kc[l];
  const int* __restrict__ start = A.start[l];
  const uint64_t local_mask = (1ULL << (3 * (a.d - 1))) - 1ULL;
  const long long p = i >> 3;
  const int j = (int)(i & 7);
  const uint64_t pk = Kp[p];
  const int b = (int)(pk >> (3 * (a.d - 1)));
  store_key(a.out, a.off_key, i, ((pk & local_mask) << 3) | (uint64_t)j, b, a.key_bytes);
  // The group's children are the s1 - s0 <= 8 keys Kc[s0..s1): lane j of the group's 8 lanes
  // fetches Kc[s0 + j], and each lane then picks, among the group's lanes, the one whose key
  // ends in its own octant.  (A level above the full ones holds whole sibling groups and a block
  // starts on a multiple of 8, so the 8 lanes of a group always run together.)
  const int s0 = start[p], s1 = start[p + 1];
  const int mine = s0 + j < s1 ? (int)(Kc[s0 + j] & 7) : -1;
  const unsigned group_mask = 0xffu << (threadIdx.x & 24);
  int ch = -1;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int oct = __shfl_sync(group_mask, mine, u, 8);
    if (oct == j) ch = s0 + u;
  }
  reinterpret_cast<int*>(a.out + a.off_child)[i] = ch;
  if (a.off_split >= 0) reinterpret_cast<float*>(a.out + a.off_split)[i] = ch < 0 ? 0.f : 1.f;
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// finest-level signal, octree.cpp:312-452 restated per node.  Rows of the feature block, in
// order: normals, displacement, point features, average points (octree.cpp:916-926).
struct SignalArgs {
  const int* child;          // level `depth` children = index into seg
  const int* seg;            // point segment starts per non-empty finest node
  const uint32_t* sorted_idx;
  const uint64_t* K;         // composite keys of the non-empty finest nodes (cloud in the top bits)
  const CloudRef* clouds;
  int depth;
  int has_normal, has_feat;
  float* f_out;              // feature block of the finest level, [C, nnum]
  float* l_out;              // label block or NULL
  long long nnum;
  int cf, node_dis, save_pts;
  float bbmin[3];
  float mul;
};

// The common case — normals only, no displacement, point features, labels or average points —
// with four nodes per thread in lock step: child, then segment + key, then the first point's
// index, then its normal are each requested for all four nodes before any is used, so a thread has
// four dependent-load chains in flight instead of one (with one chain the grid-stride loop of the
// general kernel below is a latency loop: ~5 dependent reads per node).  The arithmetic and its
// order are those of the general kernel, so the results are bit-identical.
__global__ void __launch_bounds__(256) signal_normals_kernel(SignalArgs a) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  constexpr int U = 4;
  const long long nn = a.nnum;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float* f_normal = a.f_out;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nn; i0 += stride * U) {
    int t[U], s0[U], s1[U];
    uint64_t key[U];
    long long h0[U];
    const float* normals[U];
    long long base[U];
    float first[U][3];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      t[u] = i < nn ? a.child[i] : -2;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      s0[u] = 0; s1[u] = 0; key[u] = 0;
      if (t[u] >= 0) { s0[u] = a.seg[t[u]]; s1[u] = a.seg[t[u] + 1]; key[u] = a.K[t[u]]; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      h0[u] = 0; normals[u] = nullptr; base[u] = 0;
      if (t[u] >= 0) {
        const CloudRef cl = a.clouds[(int)(key[u] >> (3 * a.depth))];
        normals[u] = cl.normal;
        base[u] = cl.offset;
        h0[u] = a.sorted_idx[s0[u]] - base[u];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      first[u][0] = first[u][1] = first[u][2] = 0.f;
      if (t[u] >= 0) {
        first[u][0] = normals[u][3 * h0[u]];
        first[u][1] = normals[u][3 * h0[u] + 1];
        first[u][2] = normals[u][3 * h0[u] + 2];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (t[u] == -2) continue;
      if (t[u] < 0) {
        for (int c = 0; c < 3; ++c) f_normal[c * nn + i] = 0.f;
        continue;
      }
      float nrm[3] = {0.f, 0.f, 0.f};
      nrm[0] += first[u][0]; nrm[1] += first[u][1]; nrm[2] += first[u][2];
      for (int j = s0[u] + 1; j < s1[u]; ++j) {
        const long long h = a.sorted_idx[j] - base[u];
        nrm[0] += normals[u][3 * h]; nrm[1] += normals[u][3 * h + 1]; nrm[2] += normals[u][3 * h + 2];
      }
      float len = 0.f;
      len += nrm[0] * nrm[0]; len += nrm[1] * nrm[1]; len += nrm[2] * nrm[2];
      float factor = sqrtf(len);
      if (factor < 1.0e-6f) {
        nrm[0] = first[u][0]; nrm[1] = first[u][1]; nrm[2] = first[u][2];
        len = 0.f;
        len += nrm[0] * nrm[0]; len += nrm[1] * nrm[1]; len += nrm[2] * nrm[2];
        factor = sqrtf(len) + 1.0e-30f;
      }
      for (int c = 0; c < 3; ++c) { nrm[c] = nrm[c] / factor; f_normal[c * nn + i] = nrm[c]; }
    }
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

__global__ void signal_kernel(SignalArgs a) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  const long long nn = a.nnum;
  const int cn = a.has_normal ? 3 : 0;
  const int cdis = a.node_dis ? (a.has_normal ? 1 : 4) : 0;
  float* f_normal = a.f_out;
  float* f_dis = f_normal + cn * nn;
  float* f_feat = f_dis + cdis * nn;
  float* f_pts = f_feat + (long long)a.cf * nn;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nn;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = a.child[i];
    if (t < 0) {
      const int ctot = cn + cdis + a.cf + (a.save_pts ? 3 : 0);
      for (int c = 0; c < ctot; ++c) a.f_out[c * nn + i] = 0.f;
      if (a.l_out) a.l_out[i] = -1.f;
      continue;
    }
    const int s0 = a.seg[t], s1 = a.seg[t + 1];
    // every point of a node comes from the node's own cloud; sorted_idx is batch-wide
    const CloudRef cl = a.clouds[(int)(a.K[t] >> (3 * a.depth))];
    const float* normals = cl.normal;
    const float* feats = cl.feat;
    const float* labels = cl.label;
    const float* xyz = cl.xyz;
    const long long base = cl.offset;
    float nrm[3] = {0.f, 0.f, 0.f};
    if (a.has_normal) {
      for (int j = s0; j < s1; ++j) {
        const long long h = a.sorted_idx[j] - base;
        nrm[0] += normals[3 * h]; nrm[1] += normals[3 * h + 1]; nrm[2] += normals[3 * h + 2];
      }
      float len = 0.f;
      len += nrm[0] * nrm[0]; len += nrm[1] * nrm[1]; len += nrm[2] * nrm[2];
      float factor = sqrtf(len);
      if (factor < 1.0e-6f) {
        const long long h = a.sorted_idx[s0] - base;
        nrm[0] = normals[3 * h]; nrm[1] = normals[3 * h + 1]; nrm[2] = normals[3 * h + 2];
        len = 0.f;
        len += nrm[0] * nrm[0]; len += nrm[1] * nrm[1]; len += nrm[2] * nrm[2];
        factor = sqrtf(len) + 1.0e-30f;
      }
      for (int c = 0; c < 3; ++c) { nrm[c] = nrm[c] / factor; f_normal[c * nn + i] = nrm[c]; }
    }
    const float cnt = (float)(unsigned)(s1 - s0) + 1.0e-30f;
    for (int c = 0; c < a.cf; ++c) {
      float acc = 0.f;
      for (int j = s0; j < s1; ++j) acc += feats[(long long)a.cf * (a.sorted_idx[j] - base) + c];
      f_feat[c * nn + i] = acc / cnt;
    }
    if (a.l_out) {
      // majority vote over labels >= 0, smallest label on ties (octree.cpp:376-401)
      int best = -1, best_cnt = 0;
      for (int j = s0; j < s1; ++j) {
        const int l = (int)labels[a.sorted_idx[j] - base];
        if (l < 0) continue;
        int c = 0;
        for (int k = s0; k < s1; ++k) c += ((int)labels[a.sorted_idx[k] - base] == l) ? 1 : 0;
        if (c > best_cnt || (c == best_cnt && l < best)) { best = l; best_cnt = c; }
      }
      a.l_out[i] = best < 0 ? -1.f : (float)best;
    }
    if (a.node_dis || a.save_pts) {
      float avg[3] = {0.f, 0.f, 0.f}, dis[4] = {0.f, 0.f, 0.f, 0.f};
      for (int j = s0; j < s1; ++j) {
        const long long h = a.sorted_idx[j] - base;
        for (int c = 0; c < 3; ++c) avg[c] += (xyz[3 * h + c] - a.bbmin[c]) * a.mul;
      }
      for (int c = 0; c < 3; ++c) {
        avg[c] = avg[c] / cnt;
        float ip;
        dis[c] = modff(avg[c], &ip) - 0.5f;
        if (a.has_normal) dis[3] += dis[c] * nrm[c]; else dis[3] = 1.f;
        if (a.save_pts) f_pts[c * nn + i] = avg[c];
      }
      if (a.node_dis) {
        if (a.has_normal) {
          f_dis[i] = dis[3] * 1.1547f;
        } else {
          for (int c = 0; c < 3; ++c) f_dis[c * nn + i] = dis[c];
          f_dis[3 * nn + i] = dis[3] * 1.1547f;
        }
      }
    }
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// ---- host drivers -----------------------------------------------------------------------------
template <typename KeyT>
int sort_and_unique(const ocnn_points_batch* pts, const ocnn_build_params* prm, const Layout& L,
                    uint8_t* ws, cudaStream_t st, int* final_buf) {
  const int64_t n = L.n;
  KeyT* keys[2] = {reinterpret_cast<KeyT*>(ws + L.off_keys[0]), reinterpret_cast<KeyT*>(ws + L.off_keys[1])};
  uint32_t* idx[2] = {reinterpret_cast<uint32_t*>(ws + L.off_idx[0]), reinterpret_cast<uint32_t*>(ws + L.off_idx[1])};
  int* hist = reinterpret_cast<int*>(ws + L.off_hist);
  int* bintot = reinterpret_cast<int*>(ws + L.off_bintot);

  EncodeArgs ea;
  ea.clouds = reinterpret_cast<const CloudRef*>(ws + L.off_offsets);
  ea.batch = pts->batch; ea.depth = prm->depth; ea.n = n;
  float width = prm->bbmax[0] - prm->bbmin[0];
  for (int j = 1; j < 3; ++j) {
    const float w = prm->bbmax[j] - prm->bbmin[j];
    if (w > width) width = w;
  }
  if (width == 0.0f) width = 1.0e-10f;
  ea.mul = (float)(1 << prm->depth) / width;
  for (int j = 0; j < 3; ++j) ea.bbmin[j] = prm->bbmin[j];
  OCNN_CUDA_OK(launch_chained(encode_kernel<KeyT>, dim3(grid_for(n, kThreads)), dim3(kThreads), 0, st, ea, keys[0], bintot, 256 * 8));
  OCNN_LAUNCH_OK("encode_kernel");

  const int nbits = 3 * prm->depth + bits_for(pts->batch);
  const int passes = (nbits + 7) / 8 < 1 ? 1 : (nbits + 7) / 8;
  const int sort_grid = L.nvb;
  int cur = 0;
  for (int p = 0; p < passes; ++p) {
    const int shift = 8 * p;
    OCNN_CUDA_OK(launch_chained(sort_hist_kernel<KeyT>, dim3(sort_grid), dim3(kThreads), 0, st, keys[cur], n, shift, L.vchunk, L.nvb, hist, bintot + 256 * p));
    OCNN_CUDA_OK(launch_chained(sort_rowscan_kernel, dim3(256), dim3(kThreads), 0, st, hist, L.nvb, bintot + 256 * p));
    if (p == 0)
      OCNN_CUDA_OK(launch_chained(sort_scatter_kernel<KeyT, true>, dim3(sort_grid), dim3(kThreads), 0, st, keys[cur], nullptr, keys[cur ^ 1], idx[cur ^ 1], n, shift, L.vchunk, L.nvb, hist));
    else
      OCNN_CUDA_OK(launch_chained(sort_scatter_kernel<KeyT, false>, dim3(sort_grid), dim3(kThreads), 0, st, keys[cur], idx[cur], keys[cur ^ 1], idx[cur ^ 1], n, shift, L.vchunk, L.nvb, hist));
    OCNN_LAUNCHES_OK("radix sort pass", 3);
    cur ^= 1;
  }
  *final_buf = cur;

  int* counts = reinterpret_cast<int*>(ws + L.off_counts);
  int* blockcnt = reinterpret_cast<int*>(ws + L.off_blockcnt);
  const int D = prm->depth, F = prm->full_depth;
  const int g0 = grid_for(n, kScanTile, 4);
  OCNN_CUDA_OK(launch_chained(unique_count_kernel<KeyT>, dim3(g0), dim3(kThreads), 0, st, keys[cur], nullptr, n, 0, blockcnt));
  OCNN_CUDA_OK(launch_chained(unique_compact_kernel<KeyT>, dim3(g0), dim3(kThreads), 0, st, keys[cur], nullptr, n, 0, blockcnt, reinterpret_cast<uint64_t*>(ws + L.off_K[D]), reinterpret_cast<int*>(ws + L.off_start[D]), counts + D));
  OCNN_LAUNCHES_OK("unique (finest level)", 2);
  for (int d = D; d > F; --d) {
    const uint64_t* Kd = reinterpret_cast<const uint64_t*>(ws + L.off_K[d]);
    const int g = grid_for(L.cap[d], kScanTile, 4);
    OCNN_CUDA_OK(launch_chained(unique_count_kernel<uint64_t>, dim3(g), dim3(kThreads), 0, st, Kd, counts + d, 0, 3, blockcnt));
    OCNN_CUDA_OK(launch_chained(unique_compact_kernel<uint64_t>, dim3(g), dim3(kThreads), 0, st, Kd, counts + d, 0, 3, blockcnt, reinterpret_cast<uint64_t*>(ws + L.off_K[d - 1]), reinterpret_cast<int*>(ws + L.off_start[d - 1]), counts + d - 1));
    OCNN_LAUNCHES_OK("unique (parent level)", 2);
  }
  return OCNN_OK;
}

int check_args(const ocnn_points_batch* pts, const ocnn_build_params* prm, const char* who) {
  OCNN_REQUIRE(pts && prm, "%s: null argument", who);
  OCNN_REQUIRE(pts->batch >= 1 && pts->offsets_host && pts->xyz_dev, "%s: empty batch", who);
  for (int b = 0; b < pts->batch; ++b)
    OCNN_REQUIRE(pts->xyz_dev[b] && (!pts->normal_dev || pts->normal_dev[b]) &&
                     (!pts->feature_dev || pts->feature_dev[b]) &&
                     (!pts->label_dev || pts->label_dev[b]),
                 "%s: cloud %d lacks a property the batch declares", who, b);
  OCNN_REQUIRE(prm->key_bits == 32 || prm->key_bits == 64, "%s: key_bits must be 32 or 64", who);
  // the header's 16-entry nnum_cum array must hold index depth + 2
  const int max_depth = prm->key_bits == 64 ? 13 : 8;
  OCNN_REQUIRE(prm->depth >= 1 && prm->depth <= max_depth,
               "%s: depth %d outside [1, %d] for %d-bit keys", who, prm->depth, max_depth,
               prm->key_bits);
  OCNN_REQUIRE(prm->full_depth >= 1 && prm->full_depth <= prm->depth,
               "%s: full_depth %d outside [1, depth]", who, prm->full_depth);
  OCNN_REQUIRE(prm->full_depth <= 7, "%s: full_depth %d too large", who, prm->full_depth);
  OCNN_REQUIRE(pts->batch <= (prm->key_bits == 64 ? 65535 : 255),
               "%s: batch %d does not fit the batch lane of a %d-bit key", who, pts->batch,
               prm->key_bits);
  OCNN_REQUIRE(prm->merged || pts->batch == 1, "%s: an un-merged build takes one cloud", who);
  OCNN_REQUIRE(pts->offsets_host[0] == 0, "%s: offsets must start at 0", who);
  for (int b = 0; b < pts->batch; ++b)
    OCNN_REQUIRE(pts->offsets_host[b + 1] > pts->offsets_host[b],
                 "%s: cloud %d is empty (the reference rejects empty point clouds)", who, b);
  OCNN_REQUIRE(pts->normal_dev || pts->feature_dev,
               "%s: points need normals or features (or both)", who);
  OCNN_REQUIRE(pts->feature_dev == nullptr || pts->feature_channels > 0,
               "%s: feature_channels must be positive", who);
  OCNN_REQUIRE(3 * prm->depth + bits_for(pts->batch) <= 64, "%s: composite key overflow", who);
  return OCNN_OK;
}

void fill_static_meta(const ocnn_points_batch* pts, const ocnn_build_params* prm,
                      ocnn_octree_meta* m) {
  memset(m, 0, sizeof(*m));
  m->key_bits = prm->key_bits;
  m->batch_size = prm->merged ? pts->batch : 1;
  m->depth = prm->depth;
  m->full_depth = prm->full_depth;
  m->has_node_dis = prm->node_dis != 0;
  m->save_pts = prm->save_pts != 0;
  // OctreeInfo::initialize, octree_info.cpp:28-64
  m->channels[OCNN_PROP_KEY] = 1; m->locations[OCNN_PROP_KEY] = -1;
  m->channels[OCNN_PROP_CHILD] = 1; m->locations[OCNN_PROP_CHILD] = -1;
  if (prm->merged) { m->channels[OCNN_PROP_NEIGH] = 8; m->locations[OCNN_PROP_NEIGH] = -1; }
  int cfeat = (pts->normal_dev ? 3 : 0) + (pts->feature_dev ? pts->feature_channels : 0);
  if (prm->node_dis) cfeat += pts->normal_dev ? 1 : 4;
  if (prm->save_pts) cfeat += 3;
  m->channels[OCNN_PROP_FEATURE] = cfeat; m->locations[OCNN_PROP_FEATURE] = prm->depth;
  if (pts->label_dev) { m->channels[OCNN_PROP_LABEL] = 1; m->locations[OCNN_PROP_LABEL] = prm->depth; }
  if (prm->split_label) { m->channels[OCNN_PROP_SPLIT] = 1; m->locations[OCNN_PROP_SPLIT] = -1; }
}

}  // namespace
}  // namespace ocnn

extern "C" {

size_t ocnn_octree_build_workspace_bytes(int64_t total_points, int batch, int depth,
                                         int full_depth) {
  if (total_points < 1 || batch < 1 || depth < 1 || depth >= OCNN_MAX_DEPTH || full_depth < 1 ||
      full_depth > depth)
    return 0;
  return ocnn::make_layout(total_points, batch, depth, full_depth).total;
}

int ocnn_octree_build_plan(const ocnn_points_batch* pts, const ocnn_build_params* prm,
                           void* workspace, size_t workspace_bytes, ocnn_octree_meta* meta,
                           void* stream) {
  using namespace ocnn;
  if (int s = check_args(pts, prm, "ocnn_octree_build_plan")) return s;
  OCNN_REQUIRE(workspace && meta, "ocnn_octree_build_plan: null workspace or meta");
  const int64_t n = pts->offsets_host[pts->batch];
  OCNN_REQUIRE(n < (1LL << 31), "ocnn_octree_build_plan: too many points");
  const Layout L = make_layout(n, pts->batch, prm->depth, prm->full_depth);
  if (workspace_bytes < L.total)
    return fail(OCNN_ERR_CAPACITY, "ocnn_octree_build_plan: workspace of %zu bytes, need %zu",
                workspace_bytes, L.total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  {
    std::vector<CloudRef> table((size_t)pts->batch + 1);
    for (int b = 0; b <= pts->batch; ++b) {
      CloudRef& c = table[b];
      const bool real = b < pts->batch;
      c.xyz = real ? pts->xyz_dev[b] : nullptr;
      c.normal = real && pts->normal_dev ? pts->normal_dev[b] : nullptr;
      c.feat = real && pts->feature_dev ? pts->feature_dev[b] : nullptr;
      c.label = real && pts->label_dev ? pts->label_dev[b] : nullptr;
      c.offset = pts->offsets_host[b];
    }
    // pageable source: the runtime stages it before returning, so `table` may go out of scope
    OCNN_CUDA_OK(cudaMemcpyAsync(ws + L.off_offsets, table.data(), sizeof(CloudRef) * table.size(),
                                 cudaMemcpyHostToDevice, st));
  }
  OCNN_CUDA_OK(cudaMemsetAsync(ws + L.off_counts, 0, sizeof(int) * 32, st));
  int final_buf = 0;
  int s = L.key_bytes_sort == 4 ? sort_and_unique<uint32_t>(pts, prm, L, ws, st, &final_buf)
                                : sort_and_unique<uint64_t>(pts, prm, L, ws, st, &final_buf);
  if (s != OCNN_OK) return s;
  int counts[32];
  OCNN_CUDA_OK(cudaMemcpyAsync(counts, ws + L.off_counts, sizeof(counts), cudaMemcpyDeviceToHost, st));
  OCNN_CUDA_OK(cudaStreamSynchronize(st));

  fill_static_meta(pts, prm, meta);
  const int D = prm->depth, F = prm->full_depth, B = pts->batch;
  for (int d = 0; d <= D; ++d) {
    if (d <= F) {
      meta->nnum[d] = B << (3 * d);
      meta->nnum_nempty[d] = d < F ? meta->nnum[d] : (D > F ? counts[F] : 0);
    } else {
      meta->nnum[d] = 8 * counts[d - 1];
      meta->nnum_nempty[d] = counts[d];
    }
  }
  for (int d = F; d <= D; ++d)
    OCNN_REQUIRE(counts[d] > 0 && (int64_t)counts[d] <= L.cap[d],
                 "ocnn_octree_build_plan: inconsistent node count %d at level %d", counts[d], d);
  finish_meta(meta);
  OCNN_REQUIRE(meta->ptr_dis[OCNN_PROP_COUNT] < (1LL << 31),
               "ocnn_octree_build_plan: octree of %lld bytes exceeds the format's 2 GiB limit",
               (long long)meta->ptr_dis[OCNN_PROP_COUNT]);
  return OCNN_OK;
}

int ocnn_octree_build_emit(const ocnn_points_batch* pts, const ocnn_build_params* prm,
                           const ocnn_octree_meta* meta, void* workspace, size_t workspace_bytes,
                           void* out, size_t out_bytes, void* header_host_out, void* stream) {
  using namespace ocnn;
  if (int s = check_args(pts, prm, "ocnn_octree_build_emit")) return s;
  OCNN_REQUIRE(workspace && meta && out, "ocnn_octree_build_emit: null argument");
  const int64_t n = pts->offsets_host[pts->batch];
  const Layout L = make_layout(n, pts->batch, prm->depth, prm->full_depth);
  if (workspace_bytes < L.total)
    return fail(OCNN_ERR_CAPACITY, "ocnn_octree_build_emit: workspace too small");
  if ((int64_t)out_bytes < meta->ptr_dis[OCNN_PROP_COUNT])
    return fail(OCNN_ERR_CAPACITY, "ocnn_octree_build_emit: output of %zu bytes, need %lld",
                out_bytes, (long long)meta->ptr_dis[OCNN_PROP_COUNT]);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* o = static_cast<uint8_t*>(out);
  const int D = prm->depth, F = prm->full_depth, B = pts->batch;

  uint8_t hdr[OCNN_HEADER_BYTES];
  HeaderExtras ex;
  ex.adp_depth = prm->adp_depth;
  ex.th_distance = prm->th_distance;
  ex.th_normal = prm->th_normal;
  for (int j = 0; j < 3; ++j) { ex.bbmin[j] = prm->bbmin[j]; ex.bbmax[j] = prm->bbmax[j]; }
  write_header(meta, ex, hdr);
  if (header_host_out) memcpy(header_host_out, hdr, OCNN_HEADER_BYTES);
  OCNN_CUDA_OK(cudaMemcpyAsync(o, hdr, OCNN_HEADER_BYTES, cudaMemcpyHostToDevice, st));

  const int* counts = reinterpret_cast<const int*>(ws + L.off_counts);
  EmitAll all;
  memset(&all, 0, sizeof(all));
  all.batch = B; all.full = F;
  int blocks = 0;
  EmitLevelArgs full_args;
  memset(&full_args, 0, sizeof(full_args));
  for (int d = 0; d <= D; ++d) {
    EmitLevelArgs a;
    a.out = o;
    a.off_key = ocnn_prop_offset(meta, OCNN_PROP_KEY, d);
    a.off_child = ocnn_prop_offset(meta, OCNN_PROP_CHILD, d);
    a.off_split = meta->channels[OCNN_PROP_SPLIT] ? ocnn_prop_offset(meta, OCNN_PROP_SPLIT, d) : -1;
    a.key_bytes = prm->key_bits / 8;
    a.d = d;
    if (d == F) full_args = a;
    const long long nnum = meta->nnum[d];
    if (nnum == 0) continue;
    const int l = all.nlev++;
    all.a[l] = a;
    all.nnum[l] = nnum;
    all.block0[l] = blocks;
    blocks += (int)((nnum + kThreads - 1) / kThreads);
    if (d > F) {
      all.Kp[l] = reinterpret_cast<const uint64_t*>(ws + L.off_K[d - 1]);
      all.Kc[l] = reinterpret_cast<const uint64_t*>(ws + L.off_K[d]);
      all.start[l] = reinterpret_cast<const int*>(ws + L.off_start[d - 1]);
    }
  }
  all.block0[all.nlev] = blocks;
  if (blocks > 0) {
    OCNN_CUDA_OK(launch_chained(emit_levels_kernel, dim3(blocks), dim3(kThreads), 0, st, all));
    OCNN_LAUNCH_OK("emit_levels_kernel");
  }
  if (D > F && meta->nnum_nempty[F] > 0) {
    // (after the level itself: it overwrites the -1 the full level wrote for every node)
    OCNN_CUDA_OK(launch_chained(emit_full_children_kernel, dim3(grid_for(meta->nnum_nempty[F], kThreads)),
                                dim3(kThreads), 0, st, full_args,
                                reinterpret_cast<const uint64_t*>(ws + L.off_K[F]), counts + F));
    OCNN_LAUNCH_OK("emit_full_children_kernel");
  }

  if (meta->nnum[D] > 0) {
    // which of the two sort buffers holds the final order: passes are a function of (depth, batch)
    const int nbits = 3 * D + bits_for(B);
    const int passes = (nbits + 7) / 8 < 1 ? 1 : (nbits + 7) / 8;
    SignalArgs sa;
    sa.child = reinterpret_cast<const int*>(o + ocnn_prop_offset(meta, OCNN_PROP_CHILD, D));
    sa.seg = reinterpret_cast<const int*>(ws + L.off_start[D]);
    sa.sorted_idx = reinterpret_cast<const uint32_t*>(ws + L.off_idx[passes & 1]);
    sa.K = reinterpret_cast<const uint64_t*>(ws + L.off_K[D]);
    sa.clouds = reinterpret_cast<const CloudRef*>(ws + L.off_offsets);
    sa.depth = D;
    sa.has_normal = pts->normal_dev != nullptr;
    sa.has_feat = pts->feature_dev != nullptr;
    sa.f_out = reinterpret_cast<float*>(o + ocnn_prop_offset(meta, OCNN_PROP_FEATURE, D));
    sa.l_out = pts->label_dev ? reinterpret_cast<float*>(o + ocnn_prop_offset(meta, OCNN_PROP_LABEL, D)) : nullptr;
    sa.nnum = meta->nnum[D];
    sa.cf = pts->feature_dev ? pts->feature_channels : 0;
    sa.node_dis = prm->node_dis; sa.save_pts = prm->save_pts;
    float width = prm->bbmax[0] - prm->bbmin[0];
    for (int j = 1; j < 3; ++j) {
      const float w = prm->bbmax[j] - prm->bbmin[j];
      if (w > width) width = w;
    }
    if (width == 0.0f) width = 1.0e-10f;
    sa.mul = (float)(1 << D) / width;
    for (int j = 0; j < 3; ++j) sa.bbmin[j] = prm->bbmin[j];
    if (sa.has_normal && sa.cf == 0 && sa.l_out == nullptr && !sa.node_dis && !sa.save_pts)
      OCNN_CUDA_OK(launch_chained(signal_normals_kernel, dim3(grid_for((sa.nnum + 3) / 4, 256, 8)), dim3(256), 0, st, sa));
    else
      OCNN_CUDA_OK(launch_chained(signal_kernel, dim3(grid_for(sa.nnum, 256, 8)), dim3(256), 0, st, sa));
    OCNN_LAUNCH_OK("signal_kernel");
  }

  if (prm->merged) return ocnn_calc_neigh(out, meta, stream);
  return OCNN_OK;
}

}  // extern "C"
