// Octree editing for the generative networks (O-UNet decoder): octree_new, octree_grow,
// octree_update (pytorch/cpp/octree_grow.cpp).  Not on the inference hot path; the point of having
// them on the device is that a decoder can keep its octree in GPU memory between levels.
//
// The header is edited on the host exactly as the reference's OctreeInfo setters do it
// (octree/octree/octree_info.cpp:188-268): the caller passes the 720 header bytes it already holds
// and gets the new ones back, so nothing here reads the device to learn sizes, except
// ocnn_octree_update, whose result (how many nodes split) depends on the data.
#include <cstring>

#include "header.h"

namespace ocnn {
namespace {

constexpr int kThreads = 256;
constexpr int kUpdateGrid = kSMs * 4;

// Patch the fields the reference rewrites after set_nnum / set_nempty: nnum_cum (set_nnum_cum with
// no capacity) and ptr_dis (set_ptr_dis), plus the scalars of `m`; everything else in the header
// stays as it came.
void patch_header(uint8_t* hdr, const ocnn_octree_meta& m) {
  auto i32 = [&](int off) { return reinterpret_cast<int32_t*>(hdr + off); };
  *i32(kOffDepth) = m.depth;
  *i32(kOffFull) = m.full_depth;
  for (int d = 0; d <= m.depth; ++d) {
    i32(kOffNnum)[d] = m.nnum[d];
    i32(kOffNnumNempty)[d] = m.nnum_nempty[d];
  }
  for (int d = 0; d <= m.depth + 2; ++d) i32(kOffNnumCum)[d] = m.nnum_cum[d];
  for (int p = 0; p <= OCNN_PROP_COUNT; ++p) i32(kOffPtrDis)[p] = (int32_t)m.ptr_dis[p];
}

// generate_key_cpu / gen_key_kernel (octree_nn.cpp:428-444, octree_nn.cu:420-444): the eight
// children of a non-empty node double its x, y, z lanes and append the bits of their octant;
// lane 3 (the batch index) is inherited.  LaneT = uint8_t (32-bit keys) or uint16_t (64-bit).
template <typename KeyT, typename LaneT>
__global__ void grow_key_kernel(KeyT* __restrict__ key_child, const KeyT* __restrict__ key,
                                const int* __restrict__ child, long long n_child_slots) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_child_slots;
       i += (long long)gridDim.x * blockDim.x) {
    const long long parent = i >> 3;
    const int j = (int)(i & 7);
    const int label = child[parent];
    if (label < 0) continue;
    KeyT k0 = key[parent], k1 = 0;
    const LaneT* a = reinterpret_cast<const LaneT*>(&k0);
    LaneT* b = reinterpret_cast<LaneT*>(&k1);
    b[0] = (LaneT)((a[0] << 1) | ((j & 4) >> 2));
    b[1] = (LaneT)((a[1] << 1) | ((j & 2) >> 1));
    b[2] = (LaneT)((a[2] << 1) | (j & 1));
    b[3] = a[3];
    key_child[8LL * label + j] = k1;
  }
}

// generate_key_cpu for a full level (octree_nn.cpp:446-464): de-interleave the node's index.
template <typename KeyT, typename LaneT>
__global__ void grow_full_key_kernel(KeyT* __restrict__ key, int depth, long long total) {
  const long long per = 1LL << (3 * depth);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long k = (unsigned long long)(i % per);
    KeyT xyz = 0;
    LaneT* p = reinterpret_cast<LaneT*>(&xyz);
    for (int d = 0; d < depth; ++d) {
      p[0] |= (LaneT)((k & (1ULL << (3 * d + 2))) >> (2 * d + 2));
      p[1] |= (LaneT)((k & (1ULL << (3 * d + 1))) >> (2 * d + 1));
      p[2] |= (LaneT)((k & (1ULL << (3 * d + 0))) >> (2 * d + 0));
    }
    p[3] = (LaneT)(i / per);
    key[i] = xyz;
  }
}

__global__ void sequence_kernel(int* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = (int)i;
}

// generate_label (octree_nn.cpp:466-473): child[i] = rank of i among the nodes with label ==
// split, else -1.  Reduce, then scan, over a fixed grid; blockcnt[gridDim.x] receives the total.
__device__ __forceinline__ void update_range(long long n, long long* beg, long long* end) {
  long long chunk = (n + gridDim.x - 1) / gridDim.x;
  chunk = (chunk + kThreads - 1) / kThreads * kThreads;
  *beg = (long long)blockIdx.x * chunk;
  const long long e = *beg + chunk;
  *end = e < n ? e : n;
  if (*beg > n) *beg = n;
}

__global__ void __launch_bounds__(kThreads) update_count_kernel(const int* __restrict__ label, long long n,
                                                                int split, int* __restrict__ blockcnt) {
  __shared__ int red[kThreads / 32];
  long long beg, end;
  update_range(n, &beg, &end);
  int c = 0;
  for (long long i = beg + threadIdx.x; i < end; i += kThreads) c += label[i] == split ? 1 : 0;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < kThreads / 32; ++w) t += red[w];
    blockcnt[blockIdx.x] = t;
  }
}

__global__ void __launch_bounds__(kThreads) update_scan_kernel(const int* __restrict__ label, long long n,
                                                               int split, int* __restrict__ blockcnt,
                                                               int* __restrict__ child) {
  __shared__ int red[kThreads / 32];
  __shared__ int wsum[kThreads / 32];
  __shared__ int base_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int c = 0;
  for (int g = threadIdx.x; g < (int)blockIdx.x; g += kThreads) c += blockcnt[g];
  for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
  if (lane == 0) red[warp] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < kThreads / 32; ++w) t += red[w];
    base_s = t;
  }
  __syncthreads();
  int base = base_s;
  long long beg, end;
  update_range(n, &beg, &end);
  for (long long t0 = beg; t0 < end; t0 += kThreads) {
    const long long i = t0 + threadIdx.x;
    const bool hit = i < end && label[i] == split;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) wsum[warp] = __popc(ballot);
    __syncthreads();
    int wbase = 0, total = 0;
    for (int w = 0; w < kThreads / 32; ++w) {
      if (w < warp) wbase += wsum[w];
      total += wsum[w];
    }
    if (i < end) child[i] = hit ? base + wbase + before : -1;
    base += total;
    __syncthreads();
  }
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) blockcnt[gridDim.x] = base;
}

__global__ void set_first_child_kernel(int* child) { child[0] = 0; }

int parse_in(const uint8_t* header_in, ocnn_octree_meta* m, const char* who) {
  OCNN_REQUIRE(header_in != nullptr, "%s: null header", who);
  return ocnn_parse_header(header_in, OCNN_HEADER_BYTES, m);
}

}  // namespace
}  // namespace ocnn

extern "C" {

size_t ocnn_octree_new_bytes(int batch_size, int channel, int key_bits) {
  if (batch_size < 1 || channel < 0 || (key_bits != 32 && key_bits != 64)) return 0;
  // header + per node: key, child, 8 neigh ints, `channel` floats
  return OCNN_HEADER_BYTES + (size_t)batch_size * (key_bits / 8 + 4 + 32 + 4 * (size_t)channel);
}

int ocnn_octree_new(int batch_size, int channel, int node_dis, int adaptive_layer, int key_bits,
                    void* out_host, size_t capacity) {
  using namespace ocnn;
  OCNN_REQUIRE(batch_size >= 1, "ocnn_octree_new: batch size %d", batch_size);
  OCNN_REQUIRE(channel >= 0, "ocnn_octree_new: negative channel count");
  OCNN_REQUIRE(key_bits == 32 || key_bits == 64, "ocnn_octree_new: key_bits must be 32 or 64");
  const size_t bytes = ocnn_octree_new_bytes(batch_size, channel, key_bits);
  OCNN_REQUIRE(out_host != nullptr && capacity >= bytes, "ocnn_octree_new: output buffer of %zu bytes, "
               "%zu needed", capacity, bytes);
  ocnn_octree_meta m;
  memset(&m, 0, sizeof(m));
  m.key_bits = key_bits;
  m.batch_size = batch_size;
  m.depth = 0;
  m.full_depth = 1;                 // set_full_layer(0) clamps to 1 (octree_info.cpp:192-194)
  m.is_adaptive = adaptive_layer > 1;
  m.key2xyz = 1;
  m.has_node_dis = node_dis != 0;
  m.nnum[0] = batch_size;
  m.nnum_nempty[0] = batch_size;
  const int ch[4] = {1, 1, 8, channel};
  for (int p = 0; p < 4; ++p) {
    m.channels[p] = ch[p];
    m.locations[p] = -1;
  }
  finish_meta(&m);
  uint8_t* out = static_cast<uint8_t*>(out_host);
  memset(out, 0, bytes);
  HeaderExtras ex;
  ex.adp_depth = adaptive_layer > 1 ? adaptive_layer : 0;
  for (int j = 0; j < 3; ++j) { ex.bbmin[j] = 0.f; ex.bbmax[j] = 2.f; }
  write_header(&m, ex, out);
  // a property without channels keeps location 0 in write_header; the reference stores what
  // set_property was given (-1) even for Feature with 0 channels
  reinterpret_cast<int32_t*>(out + kOffLocations)[OCNN_PROP_FEATURE] = -1;
  for (int i = 0; i < batch_size; ++i) {
    if (key_bits == 64) reinterpret_cast<uint64_t*>(out + m.ptr_dis[OCNN_PROP_KEY])[i] = (uint64_t)i;
    else reinterpret_cast<uint32_t*>(out + m.ptr_dis[OCNN_PROP_KEY])[i] = (uint32_t)i;
    reinterpret_cast<int32_t*>(out + m.ptr_dis[OCNN_PROP_CHILD])[i] = i;
  }
  return OCNN_OK;
}

int ocnn_octree_grow_header(const void* header_in, int target_depth, int full_octree, void* header_out) {
  using namespace ocnn;
  ocnn_octree_meta m;
  if (int rc = parse_in(static_cast<const uint8_t*>(header_in), &m, "ocnn_octree_grow")) return rc;
  OCNN_REQUIRE(header_out != nullptr, "ocnn_octree_grow: null output header");
  OCNN_REQUIRE(target_depth >= 1 && target_depth < OCNN_MAX_DEPTH &&
                   target_depth <= (m.key_bits == 64 ? 16 : 8),
               "ocnn_octree_grow: target depth %d out of range", target_depth);
  OCNN_REQUIRE(target_depth <= m.depth + 1, "ocnn_octree_grow: target depth %d skips a level of a depth-%d "
               "octree", target_depth, m.depth);
  for (int p = 0; p < 4; ++p)
    OCNN_REQUIRE(m.channels[p] == 0 || m.locations[p] == -1, "ocnn_octree_grow: the octree must keep its "
                 "properties on every level (as octree_new makes it)");
  OCNN_REQUIRE(m.channels[OCNN_PROP_KEY] == 1 && m.channels[OCNN_PROP_CHILD] == 1 &&
                   m.channels[OCNN_PROP_NEIGH] == 8,
               "ocnn_octree_grow: the octree needs Key, Child and Neigh blocks");
  const long long node_num = (long long)m.nnum_nempty[target_depth - 1] << 3;
  OCNN_REQUIRE(node_num < (1LL << 31), "ocnn_octree_grow: level too large");
  if (full_octree)
    OCNN_REQUIRE(node_num == ((long long)m.batch_size << (3 * target_depth)),
                 "ocnn_octree_grow: a full level %d of %d octrees has %lld nodes, the level above offers %lld "
                 "(every node of it must be non-empty)", target_depth, m.batch_size,
                 (long long)m.batch_size << (3 * target_depth), node_num);
  // update_octreeinfo (octree_grow.cpp:58-73), setter by setter
  m.depth = m.full_depth < target_depth ? target_depth : m.full_depth;     // set_depth
  if (full_octree) m.full_depth = target_depth < 1 ? 1 : target_depth;     // set_full_layer
  m.nnum[target_depth] = (int)node_num;
  m.nnum_nempty[target_depth] = (int)node_num;
  finish_meta(&m);
  uint8_t* out = static_cast<uint8_t*>(header_out);
  if (out != header_in) memcpy(out, header_in, OCNN_HEADER_BYTES);
  patch_header(out, m);
  const float width = (float)(1 << target_depth);
  for (int j = 0; j < 3; ++j) {
    reinterpret_cast<float*>(out + kOffBbmin)[j] = 0.f;
    reinterpret_cast<float*>(out + kOffBbmax)[j] = width;
  }
  return OCNN_OK;
}

int ocnn_octree_grow(const void* in_dev, const void* header_in, void* out_dev, const void* header_out,
                     int target_depth, int full_octree, void* stream) {
  using namespace ocnn;
  ocnn_octree_meta mi, mo;
  if (int rc = parse_in(static_cast<const uint8_t*>(header_in), &mi, "ocnn_octree_grow")) return rc;
  if (int rc = parse_in(static_cast<const uint8_t*>(header_out), &mo, "ocnn_octree_grow")) return rc;
  OCNN_REQUIRE(in_dev && out_dev && in_dev != out_dev, "ocnn_octree_grow: null or aliased buffers");
  OCNN_REQUIRE(target_depth >= 1 && target_depth <= mo.depth, "ocnn_octree_grow: target depth %d does not match "
               "the output header (depth %d)", target_depth, mo.depth);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* in = static_cast<const uint8_t*>(in_dev);
  uint8_t* out = static_cast<uint8_t*>(out_dev);
  OCNN_CUDA_OK(cudaMemsetAsync(out, 0, (size_t)mo.ptr_dis[OCNN_PROP_COUNT], st));
  OCNN_CUDA_OK(cudaMemcpyAsync(out, header_out, OCNN_HEADER_BYTES, cudaMemcpyHostToDevice, st));
  // copy_octree_gpu (octree_grow.cpp:75-88): the levels above the new one, block by block
  const long long cum = mi.nnum_cum[target_depth];
  const int esz[4] = {mi.key_bits / 8, 4, 4, 4};
  for (int p = 0; p < 4; ++p) {
    const size_t bytes = (size_t)cum * mi.channels[p] * esz[p];
    if (bytes == 0) continue;
    OCNN_CUDA_OK(cudaMemcpyAsync(out + mo.ptr_dis[p], in + mi.ptr_dis[p], bytes, cudaMemcpyDeviceToDevice, st));
  }
  const long long node_num = mo.nnum[target_depth];
  if (node_num == 0) return OCNN_OK;
  int32_t* neigh_new = reinterpret_cast<int32_t*>(out + ocnn_prop_offset(&mo, OCNN_PROP_NEIGH, target_depth));
  int32_t* child_new = reinterpret_cast<int32_t*>(out + ocnn_prop_offset(&mo, OCNN_PROP_CHILD, target_depth));
  uint8_t* key_new = out + ocnn_prop_offset(&mo, OCNN_PROP_KEY, target_depth);
  if (full_octree) {
    if (int rc = ocnn_calc_neigh_full(neigh_new, target_depth, mo.batch_size, stream)) return rc;
    if (mo.key_bits == 64)
      grow_full_key_kernel<uint64_t, uint16_t><<<grid_for(node_num, kThreads), kThreads, 0, st>>>(
          reinterpret_cast<uint64_t*>(key_new), target_depth, node_num);
    else
      grow_full_key_kernel<uint32_t, uint8_t><<<grid_for(node_num, kThreads), kThreads, 0, st>>>(
          reinterpret_cast<uint32_t*>(key_new), target_depth, node_num);
    OCNN_LAUNCH_OK("grow_full_key_kernel");
  } else {
    const int n_parent = mo.nnum[target_depth - 1];
    const int32_t* neigh_par = reinterpret_cast<const int32_t*>(out + ocnn_prop_offset(&mo, OCNN_PROP_NEIGH, target_depth - 1));
    const int32_t* child_par = reinterpret_cast<const int32_t*>(out + ocnn_prop_offset(&mo, OCNN_PROP_CHILD, target_depth - 1));
    const uint8_t* key_par = out + ocnn_prop_offset(&mo, OCNN_PROP_KEY, target_depth - 1);
    if (n_parent % 8 == 0) {
      if (int rc = ocnn_calc_neigh_split(neigh_new, neigh_par, child_par, n_parent, stream)) return rc;
    } else {
      return fail(OCNN_ERR_UNSUPPORTED, "ocnn_octree_grow: level %d holds %d nodes, not whole sibling groups "
                  "(grow the first levels with full_octree)", target_depth - 1, n_parent);
    }
    const long long slots = (long long)n_parent * 8;
    if (mo.key_bits == 64)
      grow_key_kernel<uint64_t, uint16_t><<<grid_for(slots, kThreads), kThreads, 0, st>>>(
          reinterpret_cast<uint64_t*>(key_new), reinterpret_cast<const uint64_t*>(key_par), child_par, slots);
    else
      grow_key_kernel<uint32_t, uint8_t><<<grid_for(slots, kThreads), kThreads, 0, st>>>(
          reinterpret_cast<uint32_t*>(key_new), reinterpret_cast<const uint32_t*>(key_par), child_par, slots);
    OCNN_LAUNCH_OK("grow_key_kernel");
  }
  sequence_kernel<<<grid_for(node_num, kThreads), kThreads, 0, st>>>(child_new, node_num);
  OCNN_LAUNCH_OK("sequence_kernel");
  return OCNN_OK;
}

size_t ocnn_octree_update_workspace_bytes(void) { return sizeof(int) * (size_t)(ocnn::kUpdateGrid + 1); }

int ocnn_octree_update(void* octree_dev, const void* header_in, const int32_t* label_dev, int depth,
                       int split, void* workspace_dev, void* header_out, void* stream) {
  using namespace ocnn;
  ocnn_octree_meta m;
  if (int rc = parse_in(static_cast<const uint8_t*>(header_in), &m, "ocnn_octree_update")) return rc;
  OCNN_REQUIRE(octree_dev && label_dev && workspace_dev && header_out, "ocnn_octree_update: null pointer");
  OCNN_REQUIRE(depth >= 0 && depth <= m.depth, "ocnn_octree_update: depth %d outside the octree", depth);
  OCNN_REQUIRE(m.channels[OCNN_PROP_CHILD] == 1 && m.locations[OCNN_PROP_CHILD] == -1,
               "ocnn_octree_update: the octree has no per-level Child block");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long n = m.nnum[depth];
  OCNN_REQUIRE(n > 0, "ocnn_octree_update: level %d is empty", depth);
  uint8_t* o = static_cast<uint8_t*>(octree_dev);
  int* child = reinterpret_cast<int*>(o + ocnn_prop_offset(&m, OCNN_PROP_CHILD, depth));
  int* blockcnt = static_cast<int*>(workspace_dev);
  long long want = (n + kThreads - 1) / kThreads;
  const int grid = (int)(want < kUpdateGrid ? want : kUpdateGrid);
  update_count_kernel<<<grid, kThreads, 0, st>>>(label_dev, n, split, blockcnt);
  update_scan_kernel<<<grid, kThreads, 0, st>>>(label_dev, n, split, blockcnt, child);
  OCNN_LAUNCHES_OK("octree_update scan", 2);
  int split_num = 0;
  OCNN_CUDA_OK(cudaMemcpyAsync(&split_num, blockcnt + grid, sizeof(int), cudaMemcpyDeviceToHost, st));
  OCNN_CUDA_OK(cudaStreamSynchronize(st));
  if (split_num == 0) {
    // the degenerate case of the reference (octree_grow.cpp:166-171): keep one node
    split_num = 1;
    set_first_child_kernel<<<1, 1, 0, st>>>(child);
    OCNN_LAUNCH_OK("set_first_child_kernel");
  }
  uint8_t* out = static_cast<uint8_t*>(header_out);
  if (out != header_in) memcpy(out, header_in, OCNN_HEADER_BYTES);
  reinterpret_cast<int32_t*>(out + kOffNnumNempty)[depth] = split_num;
  OCNN_CUDA_OK(cudaMemcpyAsync(o, out, OCNN_HEADER_BYTES, cudaMemcpyHostToDevice, st));
  return OCNN_OK;
}

}  // extern "C"
