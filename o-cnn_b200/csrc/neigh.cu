// Neighbour table: for every sibling group of a level, the 4x4x4 block of node indices around it.
//
// Algorithmic traffic of a split level d: read child[d-1] (4 B/node) and neigh[d-1] (32 B/node),
// write neigh[d] (32 B/node): the kernels below are HBM-bound integer kernels; each warp writes
// 128 contiguous bytes, every lookup inside a parent's block hits one 256-byte line.
#include "common.cuh"

namespace ocnn {
namespace {

__device__ __forceinline__ unsigned spread3(unsigned v) {
  // bit i of v -> bit 3i (v < 2^10 is enough: full levels never exceed depth 10 in practice)
  unsigned r = 0;
#pragma unroll
  for (int i = 0; i < 10; ++i) r |= ((v >> i) & 1u) << (3 * i);
  return r;
}

__device__ __forceinline__ unsigned gather3(unsigned key) {
  unsigned r = 0;
#pragma unroll
  for (int i = 0; i < 10; ++i) r |= ((key >> (3 * i)) & 1u) << i;
  return r;
}

// Full level: one thread per output int; out[(n*per + g)*8 + j], j = (X<<4)|(Y<<2)|Z.
// Restates calc_neigh_cpu(neigh, depth, batch), octree/octree/octree_nn.cpp:382-424.
__global__ void neigh_full_kernel(int* __restrict__ out, int depth, long long per,
                                  long long total) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  const int side = 1 << depth;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i & 63);
    const long long blk = i >> 6;                  // sibling group over the whole batch
    const long long n = (blk << 3) / per;          // batch item
    const unsigned g = (unsigned)((blk << 3) - n * per);   // first node of the group
    const int x = (int)gather3(g >> 2) + (j >> 4) - 1;
    const int y = (int)gather3(g >> 1) + ((j >> 2) & 3) - 1;
    const int z = (int)gather3(g) + (j & 3) - 1;
    int v = -1;
    if (x >= 0 && y >= 0 && z >= 0 && x < side && y < side && z < side)
      v = (int)((spread3(x) << 2) | (spread3(y) << 1) | spread3(z)) + (int)(n * per);
    out[i] = v;
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

// Split level, one warp per sibling group of PARENT nodes.  The eight parents of a group share one
// 4x4x4 neighbour block at their own level, and every entry any of their children's blocks needs
// is "the child group of one of those 64 cells".  So the warp reads the group's 64 neighbour
// entries (256 contiguous bytes) and the 64 child pointers behind them ONCE (two gathers per
// lane), keeps them in shared memory, and then writes the 64-int block of each non-empty parent
// with two coalesced 128-byte stores: 8 child gathers per parent instead of the 64 of the
// one-thread-per-output formulation.  Restates calc_neigh_cpu(neigh_split, neigh, children,
// node_num), octree/octree/octree_nn.cpp:357-380, with the parent/displacement tables
// (octree_nn.cpp:53-81) in arithmetic form.
constexpr int kNeighWarps = 8;

__global__ void __launch_bounds__(kNeighWarps * 32) neigh_split_kernel(
    int* __restrict__ out, const int* __restrict__ neigh, const int* __restrict__ child,
    long long ngroups) {
  grid_dependency_wait();       // launched as a programmatic dependent: see common.cuh
  __shared__ int cblk[kNeighWarps][64];     // child group of each cell of the parents' block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // child-level block position j = (x,y,z) in 0..3 -> which parent-level cell (tap, as a
  // (tx<<4)|(ty<<2)|tz code relative to the parent) and which octant inside it; two per lane
  int tapcode[2], oct[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int j = lane + 32 * k;
    const int x = (j >> 4) + 1, y = ((j >> 2) & 3) + 1, z = (j & 3) + 1;
    tapcode[k] = ((x >> 1) << 4) | ((y >> 1) << 2) | (z >> 1);
    oct[k] = ((x & 1) << 2) | ((y & 1) << 1) | (z & 1);
  }
  for (long long g = blockIdx.x * (long long)kNeighWarps + warp; g < ngroups;
       g += (long long)gridDim.x * kNeighWarps) {
    const int* blk = neigh + (g << 6);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int cell = blk[lane + 32 * k];
      cblk[warp][lane + 32 * k] = cell >= 0 ? child[cell] : -1;
    }
    // the eight parents themselves: lanes 0..7 read their child pointers
    const int mine = lane < 8 ? child[(g << 3) + lane] : -1;
    __syncwarp();
#pragma unroll
    for (int o = 0; o < 8; ++o) {
      const int l0 = __shfl_sync(0xffffffffu, mine, o);
      if (l0 < 0) continue;                                     // empty parent: no block
      const int octcode = ((o & 4) << 2) | ((o & 2) << 1) | (o & 1);
      int* dst = out + ((long long)l0 << 6);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int c = cblk[warp][tapcode[k] + octcode];
        dst[lane + 32 * k] = c >= 0 ? (c << 3) + oct[k] : -1;
      }
    }
    __syncwarp();
  }
  grid_dependency_trigger();    // at the end: the successor's blocks should not sit on SM slots early
}

}  // namespace
}  // namespace ocnn

extern "C" {

int ocnn_calc_neigh_full(int32_t* neigh, int depth, int batch, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(neigh != nullptr, "ocnn_calc_neigh_full: null output");
  OCNN_REQUIRE(depth >= 1 && depth <= 10 && batch >= 1, "ocnn_calc_neigh_full: depth %d / batch %d "
               "out of range", depth, batch);
  const long long per = 1LL << (3 * depth);
  const long long total = per * batch * 8;
  OCNN_REQUIRE(per * batch < (1LL << 31), "ocnn_calc_neigh_full: level too large for int32 indices");
  OCNN_CUDA_OK(launch_chained(neigh_full_kernel, dim3(grid_for(total, 256)), dim3(256), 0, static_cast<cudaStream_t>(stream), neigh, depth, per, total));
  OCNN_LAUNCH_OK("neigh_full_kernel");
  return OCNN_OK;
}

int ocnn_calc_neigh_split(int32_t* neigh_child, const int32_t* neigh, const int32_t* child,
                          int nnum_parent, void* stream) {
  using namespace ocnn;
  if (nnum_parent == 0) return OCNN_OK;
  OCNN_REQUIRE(neigh_child && neigh && child, "ocnn_calc_neigh_split: null pointer");
  OCNN_REQUIRE(nnum_parent > 0 && nnum_parent % 8 == 0,
               "ocnn_calc_neigh_split: parent level must hold whole sibling groups (got %d nodes)",
               nnum_parent);
  const long long ngroups = nnum_parent / 8;
  OCNN_CUDA_OK(launch_chained(neigh_split_kernel, dim3(grid_for(ngroups, kNeighWarps, 16)), dim3(kNeighWarps * 32), 0, static_cast<cudaStream_t>(stream), neigh_child, neigh, child, ngroups));
  OCNN_LAUNCH_OK("neigh_split_kernel");
  return OCNN_OK;
}

int ocnn_calc_neigh(void* octree_dev, const ocnn_octree_meta* m, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(octree_dev != nullptr && m != nullptr, "ocnn_calc_neigh: null argument");
  OCNN_REQUIRE(m->channels[OCNN_PROP_NEIGH] == 8 && m->locations[OCNN_PROP_NEIGH] == -1,
               "ocnn_calc_neigh: the octree has no neighbour block (not a merged batch)");
  OCNN_REQUIRE(m->channels[OCNN_PROP_CHILD] == 1 && m->locations[OCNN_PROP_CHILD] == -1,
               "ocnn_calc_neigh: the octree has no child block");
  uint8_t* base = static_cast<uint8_t*>(octree_dev);
  // level 0 has no neighbour table; the reference leaves its slot zero-filled
  // (merge_octrees.cpp:108-112 resizes a fresh vector, the loop at :184 starts at d = 1)
  if (m->nnum[0] > 0)
    OCNN_CUDA_OK(cudaMemsetAsync(base + ocnn_prop_offset(m, OCNN_PROP_NEIGH, 0), 0,
                                 (size_t)m->nnum[0] * 8 * sizeof(int32_t),
                                 static_cast<cudaStream_t>(stream)));
  for (int d = 1; d <= m->depth; ++d) {
    int32_t* nd = reinterpret_cast<int32_t*>(base + ocnn_prop_offset(m, OCNN_PROP_NEIGH, d));
    int s;
    if (d <= m->full_depth) {
      s = ocnn_calc_neigh_full(nd, d, m->batch_size, stream);
    } else {
      s = ocnn_calc_neigh_split(
          nd, reinterpret_cast<const int32_t*>(base + ocnn_prop_offset(m, OCNN_PROP_NEIGH, d - 1)),
          reinterpret_cast<const int32_t*>(base + ocnn_prop_offset(m, OCNN_PROP_CHILD, d - 1)),
          m->nnum[d - 1], stream);
    }
    if (s != OCNN_OK) return s;
  }
  return OCNN_OK;
}

}  // extern "C"
