// Shared helpers of the ocnn_b200 CUDA library: status/error plumbing, launch geometry and the
// arithmetic forms of the reference's neighbour lookup tables.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/ocnn_b200.h"

namespace ocnn {

// ---- error reporting -------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);
// Count of kernels this library has launched in this process (ocnn_launch_count()).
void note_launches(int n);

#define OCNN_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t err__ = (expr);                                                         \
    if (err__ != cudaSuccess)                                                           \
      return ::ocnn::fail(OCNN_ERR_CUDA, "%s: %s (%s:%d)", #expr, cudaGetErrorString(err__), \
                          __FILE__, __LINE__);                                          \
  } while (0)

#define OCNN_LAUNCH_OK(what) OCNN_LAUNCHES_OK(what, 1)

#define OCNN_LAUNCHES_OK(what, count)                                                   \
  do {                                                                                  \
    ::ocnn::note_launches(count);                                                       \
    cudaError_t err__ = cudaPeekAtLastError();                                          \
    if (err__ != cudaSuccess)                                                           \
      return ::ocnn::fail(OCNN_ERR_CUDA, "launch of %s failed: %s", what,               \
                          cudaGetErrorString(err__));                                   \
  } while (0)

#define OCNN_REQUIRE(cond, ...)                                  \
  do {                                                           \
    if (!(cond)) return ::ocnn::fail(OCNN_ERR_INVALID, __VA_ARGS__); \
  } while (0)

// ---- launch geometry --------------------------------------------------------------------------
constexpr int kSMs = 148;  // B200: 2 dies x 74 SMs (compile-time sizing of fixed scan grids)
// Streaming multiprocessors of the current device, queried once per device (kSMs if the query
// fails); grid-size decisions taken at launch time use this.
int sm_count();

// "Done once per device" flags for per-function attributes (cudaFuncSetAttribute is per device).
struct PerDeviceOnce {
  std::mutex mutex;
  bool done[64] = {};
};

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Grid for a grid-stride kernel: enough blocks to cover `work` items, capped at a whole number of
// waves over the 148 SMs.
inline int grid_for(long long work, int threads, int blocks_per_sm = 8) {
  long long need = (work + threads - 1) / threads;
  long long cap = (long long)sm_count() * blocks_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

// ---- programmatic dependent launch ------------------------------------------------------------
// The layers of a forward pass are a chain of short dependent kernels.  A kernel launched with
// launch_chained() may be scheduled while its predecessor in the stream is still running its last
// wave: its CTAs do their private set-up (barrier init, TMEM allocation) and then block in
// grid_dependency_wait() until the predecessor has completed and its writes are visible.  Every
// kernel launched this way must call grid_dependency_wait() before its first access to global
// memory, and calls grid_dependency_trigger() first thing so that its own successor can queue up.
__device__ __forceinline__ void grid_dependency_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- 32-byte global accesses ------------------------------------------------------------------
// 256-bit loads and stores exist from sm_100: half as many requests on the SM's load/store path as
// 16-byte ones.  The address must be 32-byte aligned.
__device__ __forceinline__ void ld_global_32B(const void* p, uint4& lo, uint4& hi) {
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z),
                 "=r"(hi.w)
               : "l"(p));
}
__device__ __forceinline__ void st_global_32B(void* p, const uint4& lo, const uint4& hi) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(lo.x), "r"(lo.y),
               "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
               : "memory");
}

// ---- two 16-bit floats in one 32-bit word ------------------------------------------------------
// `half` selects fp16 (true) or bf16 (false); kernels that serve both take it as a launch-uniform
// flag, so the branch never diverges.
__device__ __forceinline__ float2 unpack2(uint32_t w, bool half) {
  if (half) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}
__device__ __forceinline__ uint32_t pack2(float a, float b, bool half) {
  uint32_t w;
  if (half) *reinterpret_cast<__half2*>(&w) = __floats2half2_rn(a, b);
  else *reinterpret_cast<__nv_bfloat162*>(&w) = __floats2bfloat162_rn(a, b);
  return w;
}

// ---- neighbour index arithmetic ---------------------------------------------------------------
// Position, inside the 4x4x4 neighbour block of a sibling group, of the cell at offset
// (tx-1, ty-1, tz-1) from octant o of that group, tap = tx*9 + ty*3 + tz.  This is the closed
// form of the reference's ni table for the 3x3x3 kernel
// (NeighHelper::init_neigh_index, octree/octree/octree_nn.cpp:22-37).
__host__ __device__ __forceinline__ int ni333(int octant, int tap) {
  const int ox = octant >> 2, oy = (octant >> 1) & 1, oz = octant & 1;
  const int tx = tap / 9, ty = (tap / 3) % 3, tz = tap % 3;
  return ((tx + ox) << 4) | ((ty + oy) << 2) | (tz + oz);
}

// Stride-2 deconvolution in gather form.  The reference scatters: sibling group h of the finer
// level adds its product to the node at offset (tx-1, ty-1, tz-1) from the group's first cell
// (col2octree_cpu with stride 2, octree/octree/octree_nn.cpp:216-241).  Read from the receiving
// node `node` (group g = node >> 3, octant o): along an axis where the octant bit is 0 only the
// offset 0 of its own group reaches it; where the bit is 1, offset +1 of its own group and offset
// -1 of the group two cells further.  Returns the sending group (= rank of its parent among the
// non-empty nodes of the coarser level) for tap = tx*9 + ty*3 + tz, or -1 when that tap does not
// reach this octant or the group does not exist.  neigh = the finer level's neighbour table.
__device__ __forceinline__ int up_source_group(const int* __restrict__ neigh, int node, int tap) {
  const int o = node & 7;
  const int off[3] = {tap / 9 - 1, (tap / 3) % 3 - 1, tap % 3 - 1};
  int pos = 0;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    const int bit = (o >> (2 - a)) & 1;
    if (bit == 0 ? off[a] != 0 : off[a] == 0) return -1;
    pos = (pos << 2) | ((bit == 1 && off[a] == -1) ? 3 : 1);
  }
  const int q = neigh[((long long)(node >> 3) << 6) + pos];
  return q >= 0 ? (q >> 3) : -1;
}

// The taps of the 3x3x3 neighbourhood that each supported kernel shape uses
// (octree/octree/octree_nn.cpp:7-19).  Returns the tap count or -1.
struct TapList {
  int count;
  signed char tap[27];
};
TapList taps_for_kernel(const int kernel_size[3]);

// Row-count and pointer rules of ocnn_conv_geometry, shared by the CUDA-core and the tensor-core
// route (defined in conv_simt.cu).
int check_conv_geometry(const ocnn_conv_geometry* g, const TapList& tl, const char* who);

}  // namespace ocnn
