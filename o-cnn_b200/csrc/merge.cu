// octree_batch on the device: merge already-built octrees (device buffers) into one batch octree
// and compute its neighbour table.  Restates merge_octrees, octree/octree/merge_octrees.cpp:7-198:
// level-wise concatenation in batch order, batch index stamped into the top key lane, children
// rebased by the running non-empty count, features re-interleaved so each channel row spans the
// whole batch level.
#include <cstring>
#include <mutex>
#include <vector>

#include "header.h"

namespace ocnn {
namespace {

struct MergeEntry {
  const uint8_t* src;     // device pointer of the source octree
  long long key, child, feat, label, split;   // byte offsets inside src at this level (-1: none)
  int n;                  // nodes of this octree at this level
  int node0;              // first destination node
  int ne0;                // non-empty nodes of earlier octrees at this level
  int b, d;
};

struct MergeDst {
  uint8_t* out;
  long long key[OCNN_MAX_DEPTH], child[OCNN_MAX_DEPTH], feat[OCNN_MAX_DEPTH],
      label[OCNN_MAX_DEPTH], split[OCNN_MAX_DEPTH];
  int nnum[OCNN_MAX_DEPTH];
  int key_bytes, cfeat;
};

__global__ void merge_kernel(const MergeEntry* __restrict__ entries, int nentries, MergeDst dst) {
  for (int e = blockIdx.y; e < nentries; e += gridDim.y) {
    const MergeEntry en = entries[e];
    const int d = en.d;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < en.n; j += gridDim.x * blockDim.x) {
      const long long o = en.node0 + j;
      if (en.key >= 0) {
        if (dst.key_bytes == 8) {
          const uint64_t k = reinterpret_cast<const uint64_t*>(en.src + en.key)[j];
          reinterpret_cast<uint64_t*>(dst.out + dst.key[d])[o] =
              (k & 0x0000ffffffffffffULL) | ((uint64_t)(en.b & 0xffff) << 48);
        } else {
          const uint32_t k = reinterpret_cast<const uint32_t*>(en.src + en.key)[j];
          reinterpret_cast<uint32_t*>(dst.out + dst.key[d])[o] =
              (k & 0x00ffffffu) | ((uint32_t)(en.b & 0xff) << 24);
        }
      }
      if (en.child >= 0) {
        const int c = reinterpret_cast<const int*>(en.src + en.child)[j];
        reinterpret_cast<int*>(dst.out + dst.child[d])[o] = c == -1 ? -1 : c + en.ne0;
      }
      if (en.feat >= 0) {
        const float* fs = reinterpret_cast<const float*>(en.src + en.feat);
        float* fd = reinterpret_cast<float*>(dst.out + dst.feat[d]);
        for (int c = 0; c < dst.cfeat; ++c) fd[(long long)c * dst.nnum[d] + o] = fs[(long long)c * en.n + j];
      }
      if (en.label >= 0)
        reinterpret_cast<float*>(dst.out + dst.label[d])[o] = reinterpret_cast<const float*>(en.src + en.label)[j];
      if (en.split >= 0)
        reinterpret_cast<float*>(dst.out + dst.split[d])[o] = reinterpret_cast<const float*>(en.src + en.split)[j];
    }
  }
}

bool at_level(const ocnn_octree_meta* m, int prop, int d) {
  return m->channels[prop] != 0 && (m->locations[prop] == -1 || m->locations[prop] == d);
}

// The merged header: the first octree's header with batch size, neighbour property, node counts
// and block offsets replaced (MergeOctrees::set_batch_info, merge_octrees.cpp:92-106).
void merged_header(const void* first_header_host, const ocnn_octree_meta* merged,
                   uint8_t (&hdr)[OCNN_HEADER_BYTES]) {
  const int depth = merged->depth;
  memset(hdr, 0, sizeof(hdr));
  memcpy(hdr, first_header_host, 716);
  auto i32 = [&](int off) { return reinterpret_cast<int32_t*>(hdr + off); };
  *i32(kOffBatch) = merged->batch_size;
  int flags = 0;
  for (int d = 0; d < OCNN_MAX_DEPTH; ++d) {
    if (d <= depth) { i32(kOffNnum)[d] = merged->nnum[d]; i32(kOffNnumNempty)[d] = merged->nnum_nempty[d]; }
    if (d <= depth + 2) i32(kOffNnumCum)[d] = merged->nnum_cum[d];
  }
  for (int p = 0; p < OCNN_PROP_COUNT; ++p) {
    i32(kOffChannels)[p] = merged->channels[p];
    if (merged->channels[p] != 0) { i32(kOffLocations)[p] = merged->locations[p]; flags |= 1 << p; }
  }
  for (int p = 0; p <= OCNN_PROP_COUNT; ++p) i32(kOffPtrDis)[p] = (int32_t)merged->ptr_dis[p];
  *i32(kOffFlags) = flags;
}

// The (octree, level) table merge_kernel walks, written to `entries` (room for batch*(depth+1));
// returns the number of entries; *max_n = the largest node count of any entry.
int merge_table(const void* const* octrees_dev, const ocnn_octree_meta* in, int batch, int depth,
                MergeEntry* entries, int* max_n) {
  int ne = 0;
  *max_n = 1;
  for (int d = 0; d <= depth; ++d) {
    int node0 = 0, ne0 = 0;
    for (int b = 0; b < batch; ++b) {
      const ocnn_octree_meta* m = &in[b];
      MergeEntry e;
      e.src = static_cast<const uint8_t*>(octrees_dev[b]);
      e.key = at_level(m, OCNN_PROP_KEY, d) ? ocnn_prop_offset(m, OCNN_PROP_KEY, d) : -1;
      e.child = at_level(m, OCNN_PROP_CHILD, d) ? ocnn_prop_offset(m, OCNN_PROP_CHILD, d) : -1;
      e.feat = at_level(m, OCNN_PROP_FEATURE, d) ? ocnn_prop_offset(m, OCNN_PROP_FEATURE, d) : -1;
      e.label = at_level(m, OCNN_PROP_LABEL, d) ? ocnn_prop_offset(m, OCNN_PROP_LABEL, d) : -1;
      e.split = at_level(m, OCNN_PROP_SPLIT, d) ? ocnn_prop_offset(m, OCNN_PROP_SPLIT, d) : -1;
      e.n = m->nnum[d]; e.node0 = node0; e.ne0 = ne0; e.b = b; e.d = d;
      if (e.n > 0) entries[ne++] = e;
      if (e.n > *max_n) *max_n = e.n;
      node0 += m->nnum[d];
      ne0 += m->nnum_nempty[d];
    }
  }
  return ne;
}

MergeDst merge_destination(const ocnn_octree_meta* merged, uint8_t* out) {
  MergeDst dst;
  memset(&dst, 0, sizeof(dst));
  dst.out = out;
  dst.key_bytes = merged->key_bits / 8;
  dst.cfeat = merged->channels[OCNN_PROP_FEATURE];
  for (int d = 0; d <= merged->depth; ++d) {
    dst.key[d] = ocnn_prop_offset(merged, OCNN_PROP_KEY, d);
    dst.child[d] = ocnn_prop_offset(merged, OCNN_PROP_CHILD, d);
    dst.feat[d] = at_level(merged, OCNN_PROP_FEATURE, d) ? ocnn_prop_offset(merged, OCNN_PROP_FEATURE, d) : -1;
    dst.label[d] = at_level(merged, OCNN_PROP_LABEL, d) ? ocnn_prop_offset(merged, OCNN_PROP_LABEL, d) : -1;
    dst.split[d] = at_level(merged, OCNN_PROP_SPLIT, d) ? ocnn_prop_offset(merged, OCNN_PROP_SPLIT, d) : -1;
    dst.nnum[d] = merged->nnum[d];
  }
  return dst;
}

// Enqueue the merge of `ne` table entries already resident at table_dev.
int launch_merge(const MergeEntry* table_dev, int ne, int max_n, const MergeDst& dst,
                 cudaStream_t st, const char* what) {
  dim3 grid(ceil_div(max_n, 256) < 64 ? ceil_div(max_n, 256) : 64, ne < 4096 ? ne : 4096);
  merge_kernel<<<grid, 256, 0, st>>>(table_dev, ne, dst);
  OCNN_LAUNCH_OK(what);
  return OCNN_OK;
}

}  // namespace
}  // namespace ocnn

extern "C" {

int ocnn_octree_batch_meta(const ocnn_octree_meta* in, int batch, ocnn_octree_meta* merged) {
  using namespace ocnn;
  OCNN_REQUIRE(in && merged && batch >= 1, "ocnn_octree_batch_meta: empty input");
  const ocnn_octree_meta& f = in[0];
  OCNN_REQUIRE(batch <= (f.key_bits == 64 ? 65535 : 255),
               "ocnn_octree_batch_meta: batch %d does not fit the batch lane of a %d-bit key",
               batch, f.key_bits);
  for (int i = 0; i < batch; ++i) {
    const ocnn_octree_meta& m = in[i];
    // OctreeInfo::is_consistent, octree_info.cpp:118-129
    bool same = m.key_bits == f.key_bits && m.depth == f.depth && m.full_depth == f.full_depth &&
                m.batch_size == f.batch_size && m.is_adaptive == f.is_adaptive &&
                m.key2xyz == f.key2xyz && m.has_node_dis == f.has_node_dis;
    for (int p = 0; p < OCNN_PROP_COUNT; ++p)
      same = same && m.channels[p] == f.channels[p] &&
             (m.channels[p] == 0 || m.locations[p] == f.locations[p]);
    OCNN_REQUIRE(same, "The formats of input octrees are not consistent (octree %d)", i);
  }
  *merged = f;
  merged->batch_size = batch;
  merged->channels[OCNN_PROP_NEIGH] = 8;
  merged->locations[OCNN_PROP_NEIGH] = -1;
  for (int d = 0; d <= f.depth; ++d) {
    long long nn = 0, ne = 0;
    for (int i = 0; i < batch; ++i) { nn += in[i].nnum[d]; ne += in[i].nnum_nempty[d]; }
    OCNN_REQUIRE(nn < (1LL << 28), "ocnn_octree_batch_meta: merged level %d too large", d);
    merged->nnum[d] = (int)nn;
    merged->nnum_nempty[d] = (int)ne;
  }
  finish_meta(merged);
  OCNN_REQUIRE(merged->ptr_dis[OCNN_PROP_COUNT] < (1LL << 31),
               "ocnn_octree_batch_meta: merged octree exceeds the format's 2 GiB limit");
  return OCNN_OK;
}

size_t ocnn_octree_batch_workspace_bytes(int batch, int depth) {
  if (batch < 1 || depth < 1) return 0;
  return sizeof(ocnn::MergeEntry) * (size_t)batch * (size_t)(depth + 1) + 256;
}

int ocnn_octree_batch(const void* const* octrees_dev, const ocnn_octree_meta* in,
                      const void* first_header_host, int batch, const ocnn_octree_meta* merged,
                      void* workspace, size_t workspace_bytes, void* out, void* header_host_out,
                      void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(octrees_dev && in && first_header_host && merged && workspace && out && batch >= 1,
               "ocnn_octree_batch: null argument");
  const int depth = merged->depth;
  const size_t need = ocnn_octree_batch_workspace_bytes(batch, depth);
  if (workspace_bytes < need)
    return fail(OCNN_ERR_CAPACITY, "ocnn_octree_batch: workspace of %zu bytes, need %zu",
                workspace_bytes, need);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* o = static_cast<uint8_t*>(out);

  uint8_t hdr[OCNN_HEADER_BYTES];
  merged_header(first_header_host, merged, hdr);
  if (header_host_out) memcpy(header_host_out, hdr, OCNN_HEADER_BYTES);
  OCNN_CUDA_OK(cudaMemcpyAsync(o, hdr, OCNN_HEADER_BYTES, cudaMemcpyHostToDevice, st));

  std::vector<MergeEntry> entries((size_t)batch * (depth + 1));
  int max_n = 1;
  const int ne = merge_table(octrees_dev, in, batch, depth, entries.data(), &max_n);
  if (ne > 0) {
    // the staging vector is pageable memory: the runtime has copied it out before returning
    OCNN_CUDA_OK(cudaMemcpyAsync(workspace, entries.data(), sizeof(MergeEntry) * (size_t)ne,
                                 cudaMemcpyHostToDevice, st));
    if (int rc = launch_merge(static_cast<const MergeEntry*>(workspace), ne, max_n,
                              merge_destination(merged, o), st, "merge_kernel"))
      return rc;
  }
  return ocnn_calc_neigh(out, merged, stream);
}


}  // extern "C"

// ---- octree_batch without any caller-provided or allocated scratch ----------------------------
// The (octree, level) table that merge_kernel reads lives in a fixed array inside this library's
// device image instead of in a workspace the caller hands over.  Meant for callers that cannot get
// device memory at the moment of the call, e.g. a process whose framework allocator has already
// claimed the whole GPU so that a fresh cudaMalloc fails.
namespace ocnn {
namespace {

constexpr int kStaticMergeEntries = 2048;   // (octree, level) pairs: batch * (depth + 1) <= 2048
static __device__ __align__(256) unsigned char g_merge_scratch[kStaticMergeEntries * sizeof(MergeEntry)];

std::mutex g_static_mutex;
MergeEntry g_static_stage[kStaticMergeEntries];   // host staging of the table, guarded by the mutex
void* g_static_dev_ptr[64] = {};                  // device address of g_merge_scratch, per device

}  // namespace
}  // namespace ocnn

extern "C" int ocnn_octree_batch_noalloc(const void* const* octrees_dev, const ocnn_octree_meta* in,
                                         const void* first_header_host, int batch,
                                         const ocnn_octree_meta* merged, void* out,
                                         void* header_host_out, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(octrees_dev && in && first_header_host && merged && out && batch >= 1,
               "ocnn_octree_batch_noalloc: null argument");
  const int depth = merged->depth;
  const long long pairs = (long long)batch * (depth + 1);
  if (pairs > kStaticMergeEntries)
    return fail(OCNN_ERR_CAPACITY,
                "ocnn_octree_batch_noalloc: batch %d x (depth %d + 1) = %lld (octree, level) pairs "
                "exceeds the built-in scratch of %d pairs; use ocnn_octree_batch with a workspace",
                batch, depth, pairs, kStaticMergeEntries);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* o = static_cast<uint8_t*>(out);

  // In host code the name g_merge_scratch is only a handle for the device array; the address a
  // kernel can use comes from the runtime, once per device, with that device current.
  int device = -1;
  OCNN_CUDA_OK(cudaGetDevice(&device));
  OCNN_REQUIRE(device >= 0 && device < 64, "ocnn_octree_batch_noalloc: device ordinal %d out of range",
               device);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_dev_ptr[device] == nullptr) {
    void* ptr = nullptr;
    OCNN_CUDA_OK(cudaGetSymbolAddress(&ptr, g_merge_scratch));
    OCNN_REQUIRE(ptr != nullptr, "ocnn_octree_batch_noalloc: no device address for the scratch array");
    g_static_dev_ptr[device] = ptr;
  }
  MergeEntry* table_dev = static_cast<MergeEntry*>(g_static_dev_ptr[device]);

  uint8_t hdr[OCNN_HEADER_BYTES];
  merged_header(first_header_host, merged, hdr);
  if (header_host_out) memcpy(header_host_out, hdr, OCNN_HEADER_BYTES);
  OCNN_CUDA_OK(cudaMemcpyAsync(o, hdr, OCNN_HEADER_BYTES, cudaMemcpyHostToDevice, st));

  int max_n = 1;
  const int ne = merge_table(octrees_dev, in, batch, depth, g_static_stage, &max_n);
  if (ne > 0) {
    // Only the first `ne` entries are read by the kernel and all of them are rewritten here, so
    // nothing left over from an earlier call needs clearing.  The staging array is pageable
    // memory: the runtime has copied it out when cudaMemcpyAsync returns, which is what lets the
    // mutex be released at the end of this function.
    OCNN_CUDA_OK(cudaMemcpyAsync(table_dev, g_static_stage, sizeof(MergeEntry) * (size_t)ne,
                                 cudaMemcpyHostToDevice, st));
    if (int rc = launch_merge(table_dev, ne, max_n, merge_destination(merged, o), st,
                              "merge_kernel (built-in scratch)"))
      return rc;
  }
  return ocnn_calc_neigh(out, merged, stream);
}
