// Key arithmetic, key search and the operators built on it: xyz <-> Morton key conversion,
// search of query keys among a level's sorted keys, interpolation of node data at points
// (nearest / trilinear) and alignment of data between two octrees.
//
// Restates xyz2key_cpu / key2xyz_cpu / search_key_cpu (octree/octree/octree_nn.cpp:540-620; GPU
// twins octree_nn.cu:575-660), align_forward / align_backward (octree_nn.cu:711-752) and the
// interpolation the reference assembles in Python from those pieces
// (pytorch/ocnn/modules.py:209-275: octree_nearest_pts, octree_trilinear_pts).
//
// A key packs four lanes (x, y, z, batch id): bytes for 32-bit keys, 16-bit words for 64-bit keys
// (octree/octree/types.h:16-24).  In "xyz" form lanes 0..2 hold the integer coordinates; in "key"
// form the low 3*depth bits hold the Morton interleave (x -> bit 3i+2, y -> 3i+1, z -> 3i) and lane
// 3 still holds the batch id.  Only `depth` bits of each coordinate enter a key
// (compute_key, octree_nn.cpp:551-560): a coordinate outside [0, 2^depth) wraps.
#include "common.cuh"

namespace ocnn {
namespace {

template <typename K> struct Lane;
template <> struct Lane<uint32_t> { static constexpr int bits = 8; };
template <> struct Lane<uint64_t> { static constexpr int bits = 16; };

template <typename K>
__host__ __device__ __forceinline__ K xyz_to_key(K xyz, int depth) {
  constexpr int B = Lane<K>::bits;
  constexpr K lane_mask = (K(1) << B) - 1;
  const K x = xyz & lane_mask, y = (xyz >> B) & lane_mask, z = (xyz >> (2 * B)) & lane_mask;
  K key = 0;
  for (int i = 0; i < depth; ++i) {
    const K m = K(1) << i;
    key |= ((x & m) << (2 * i + 2)) | ((y & m) << (2 * i + 1)) | ((z & m) << (2 * i));
  }
  // lane 3 (the batch id) replaces whatever the interleave put there
  constexpr K low3 = (K(1) << (3 * B)) - 1;
  return (key & low3) | (xyz & ~low3);
}

template <typename K>
__host__ __device__ __forceinline__ K key_to_xyz(K key, int depth) {
  constexpr int B = Lane<K>::bits;
  constexpr K lane_mask = (K(1) << B) - 1;
  K x = 0, y = 0, z = 0;
  for (int i = 0; i < depth; ++i) {
    x |= (key & (K(1) << (3 * i + 2))) >> (2 * i + 2);
    y |= (key & (K(1) << (3 * i + 1))) >> (2 * i + 1);
    z |= (key & (K(1) << (3 * i))) >> (2 * i);
  }
  constexpr K low3 = (K(1) << (3 * B)) - 1;
  return (x & lane_mask) | ((y & lane_mask) << B) | ((z & lane_mask) << (2 * B)) | (key & ~low3);
}

template <typename K, bool TO_KEY>
__global__ void convert_key_kernel(const K* __restrict__ in, K* __restrict__ out, long long num,
                                   int depth) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < num;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = TO_KEY ? xyz_to_key<K>(in[i], depth) : key_to_xyz<K>(in[i], depth);
}

// index of `q` among the n sorted keys, or -1 (std::lower_bound + equality, octree_nn.cpp:540-547)
template <typename K>
__device__ __forceinline__ int find_key(const K* __restrict__ keys, int n, K q) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (keys[mid] < q) lo = mid + 1; else hi = mid;
  }
  return (lo < n && keys[lo] == q) ? lo : -1;
}

template <typename K>
__global__ void search_key_kernel(const K* __restrict__ keys, int n_key, const K* __restrict__ query,
                                  long long n_query, int* __restrict__ idx, int query_is_xyz,
                                  int depth) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_query;
       i += (long long)gridDim.x * blockDim.x) {
    K q = query[i];
    if (query_is_xyz) q = xyz_to_key<K>(q, depth);
    idx[i] = find_key<K>(keys, n_key, q);
  }
}

// keys of the non-empty nodes of a level, in order: out[child[h]] = key[h] (the pad_backward the
// reference runs on the key array, pytorch/cpp/octree_key.cpp:100-108)
template <typename K>
__global__ void key_depad_kernel(const K* __restrict__ key, const int* __restrict__ child, int nnum,
                                 K* __restrict__ out) {
  for (int h = blockIdx.x * blockDim.x + threadIdx.x; h < nnum; h += gridDim.x * blockDim.x) {
    const int c = child[h];
    if (c >= 0) out[c] = key[h];
  }
}

template <typename T> __device__ __forceinline__ float load_f(const T* p, long long i);
template <> __device__ __forceinline__ float load_f<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float load_f<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <> __device__ __forceinline__ float load_f<__half>(const __half* p, long long i) {
  return __half2float(p[i]);
}
template <typename T> __device__ __forceinline__ void store_f(T* p, long long i, float v);
template <> __device__ __forceinline__ void store_f<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void store_f<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16(v);
}
template <> __device__ __forceinline__ void store_f<__half>(__half* p, long long i, float v) {
  p[i] = __float2half(v);
}

// Interpolation of node data at points.  pts: [N, 4] float32 = (x, y, z) in [0, 2^depth] and the
// batch id.  One warp per point: lanes 0..7 (0 for nearest) each look up one corner cell, then the
// whole warp walks the channels.
//   nearest: the cell is trunc(x, y, z) as 16-bit integers; the result is that node's row, or 0.
//   linear:  p = xyz - 0.5 (values sit at cell centres), base = floor(p), frac = p - base; corner
//            (dx,dy,dz) in {0,1}^3 has weight prod(d ? frac : 1 - frac); the result is the weighted
//            sum over the corners that exist, divided by (sum of their weights + 1e-10).
// The corner keys are formed the way the reference does: base cell and batch id packed into the
// four lanes, the corner offset added to the PACKED word (so a lane of -1 carries into the next
// one), then interleaved with only `depth` bits per coordinate.
template <typename T, typename K, bool NODE_MAJOR>
__global__ void __launch_bounds__(256) interp_kernel(const T* __restrict__ data, T* __restrict__ out,
                                                    const float* __restrict__ pts,
                                                    const K* __restrict__ keys, int n_key, int C,
                                                    long long H, long long N, int depth, int linear) {
  constexpr int B = Lane<K>::bits;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long n = warp0; n < N; n += nwarps) {
    const float px = pts[4 * n], py = pts[4 * n + 1], pz = pts[4 * n + 2], pid = pts[4 * n + 3];
    int idx = -1;
    float wgt = 0.f;
    if (lane < (linear ? 8 : 1)) {
      float fx = px, fy = py, fz = pz;
      float frx = 0.f, fry = 0.f, frz = 0.f;
      if (linear) {
        fx = px - 0.5f; fy = py - 0.5f; fz = pz - 0.5f;
        const float bx = floorf(fx), by = floorf(fy), bz = floorf(fz);
        frx = fx - bx; fry = fy - by; frz = fz - bz;
        fx = bx; fy = by; fz = bz;
      }
      // float -> int16 (truncation toward zero, as Tensor.short()), kept as the lane's bit pattern
      constexpr K lane_mask = (K(1) << B) - 1;
      const K kx = (K)(uint16_t)(int16_t)fx & lane_mask, ky = (K)(uint16_t)(int16_t)fy & lane_mask;
      const K kz = (K)(uint16_t)(int16_t)fz & lane_mask, kid = (K)(uint16_t)(int16_t)pid & lane_mask;
      K word = kx | (ky << B) | (kz << (2 * B)) | (kid << (3 * B));
      const int dx = (lane >> 2) & 1, dy = (lane >> 1) & 1, dz = lane & 1;
      if (linear) word += (K)dx + ((K)dy << B) + ((K)dz << (2 * B));
      idx = find_key<K>(keys, n_key, xyz_to_key<K>(word, depth));
      wgt = linear ? fabsf((dx ? -frx : 1.f - frx) * (dy ? -fry : 1.f - fry) * (dz ? -frz : 1.f - frz))
                   : 1.f;
      if (idx < 0) wgt = 0.f;
    }
    float norm = wgt;
#pragma unroll
    for (int o = 4; o >= 1; o >>= 1) norm += __shfl_xor_sync(0xffffffffu, norm, o);   // lanes 0..7
    norm = __shfl_sync(0xffffffffu, norm, 0);
    int cidx[8];
    float cw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      cidx[j] = __shfl_sync(0xffffffffu, idx, j);
      cw[j] = __shfl_sync(0xffffffffu, wgt, j);
    }
    const float inv = linear ? 1.f / (norm + 1e-10f) : 1.f;
    for (int c = lane; c < C; c += 32) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (cidx[j] >= 0 && (linear || j == 0))
          acc += cw[j] * load_f<T>(data, NODE_MAJOR ? (long long)cidx[j] * C + c : (long long)c * H + cidx[j]);
      }
      store_f<T>(out, NODE_MAJOR ? n * C + c : (long long)c * N + n, acc * inv);
    }
  }
}

// align: dst[., idx[h]] = src[., h] where idx[h] >= 0 (dst cleared first)
template <typename T, bool NODE_MAJOR>
__global__ void align_kernel(const T* __restrict__ src, T* __restrict__ dst,
                             const int* __restrict__ idx, int C, long long src_h, long long dst_h,
                             long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long h, c;
    if (NODE_MAJOR) { h = i / C; c = i % C; } else { c = i / src_h; h = i % src_h; }
    const int j = idx[h];
    if (j >= 0) dst[NODE_MAJOR ? (long long)j * C + c : c * dst_h + j] = src[i];
  }
}

// the transpose of align: src[., h] = idx[h] < 0 ? 0 : dst[., idx[h]]
template <typename T, bool NODE_MAJOR>
__global__ void align_back_kernel(T* __restrict__ src, const T* __restrict__ dst,
                                  const int* __restrict__ idx, int C, long long src_h, long long dst_h,
                                  long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long h, c;
    if (NODE_MAJOR) { h = i / C; c = i % C; } else { c = i / src_h; h = i % src_h; }
    const int j = idx[h];
    src[i] = j >= 0 ? dst[NODE_MAJOR ? (long long)j * C + c : c * dst_h + j] : T(0);
  }
}

template <typename K>
int search_impl(const void* keys, int n_key, const void* query, long long n_query, int32_t* idx,
                int query_is_xyz, int depth, cudaStream_t st) {
  search_key_kernel<K><<<grid_for(n_query, 256), 256, 0, st>>>(
      static_cast<const K*>(keys), n_key, static_cast<const K*>(query), n_query, idx, query_is_xyz, depth);
  OCNN_LAUNCH_OK("search_key_kernel");
  return OCNN_OK;
}

template <typename T, typename K>
int interp_impl(const void* data, void* out, const float* pts, const void* keys, int n_key, int C,
                long long H, long long N, int depth, int linear, int layout, cudaStream_t st) {
  const int grid = grid_for(N * 32, 256);
  if (layout == OCNN_NODE_MAJOR)
    interp_kernel<T, K, true><<<grid, 256, 0, st>>>(static_cast<const T*>(data), static_cast<T*>(out), pts,
                                                  static_cast<const K*>(keys), n_key, C, H, N, depth, linear);
  else
    interp_kernel<T, K, false><<<grid, 256, 0, st>>>(static_cast<const T*>(data), static_cast<T*>(out), pts,
                                                   static_cast<const K*>(keys), n_key, C, H, N, depth, linear);
  OCNN_LAUNCH_OK("interp_kernel");
  return OCNN_OK;
}

}  // namespace
}  // namespace ocnn

extern "C" {

int ocnn_convert_key(const void* in, void* out, int64_t num, int depth, int key_bits, int to_key,
                     void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(key_bits == 32 || key_bits == 64, "ocnn_convert_key: key_bits must be 32 or 64");
  OCNN_REQUIRE(depth >= 0 && depth <= (key_bits == 64 ? 16 : 8), "ocnn_convert_key: depth %d out of range", depth);
  OCNN_REQUIRE(num >= 0, "ocnn_convert_key: negative count");
  if (num == 0) return OCNN_OK;
  OCNN_REQUIRE(in && out, "ocnn_convert_key: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(num, 256);
  if (key_bits == 64) {
    if (to_key) convert_key_kernel<uint64_t, true><<<grid, 256, 0, st>>>((const uint64_t*)in, (uint64_t*)out, num, depth);
    else convert_key_kernel<uint64_t, false><<<grid, 256, 0, st>>>((const uint64_t*)in, (uint64_t*)out, num, depth);
  } else {
    if (to_key) convert_key_kernel<uint32_t, true><<<grid, 256, 0, st>>>((const uint32_t*)in, (uint32_t*)out, num, depth);
    else convert_key_kernel<uint32_t, false><<<grid, 256, 0, st>>>((const uint32_t*)in, (uint32_t*)out, num, depth);
  }
  OCNN_LAUNCH_OK("convert_key_kernel");
  return OCNN_OK;
}

int ocnn_search_key(const void* keys, int n_key, const void* query, int64_t n_query, int32_t* idx,
                    int query_is_xyz, int depth, int key_bits, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(key_bits == 32 || key_bits == 64, "ocnn_search_key: key_bits must be 32 or 64");
  OCNN_REQUIRE(n_key >= 0 && n_query >= 0, "ocnn_search_key: negative count");
  if (n_query == 0) return OCNN_OK;
  OCNN_REQUIRE(query && idx && (keys || n_key == 0), "ocnn_search_key: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return key_bits == 64 ? search_impl<uint64_t>(keys, n_key, query, n_query, idx, query_is_xyz, depth, st)
                        : search_impl<uint32_t>(keys, n_key, query, n_query, idx, query_is_xyz, depth, st);
}

int ocnn_key_depad(const void* key, const int32_t* child, int nnum, void* out, int key_bits,
                   void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(key_bits == 32 || key_bits == 64, "ocnn_key_depad: key_bits must be 32 or 64");
  if (nnum == 0) return OCNN_OK;
  OCNN_REQUIRE(key && child && out && nnum > 0, "ocnn_key_depad: null pointer or negative size");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (key_bits == 64)
    key_depad_kernel<uint64_t><<<grid_for(nnum, 256), 256, 0, st>>>((const uint64_t*)key, child, nnum, (uint64_t*)out);
  else
    key_depad_kernel<uint32_t><<<grid_for(nnum, 256), 256, 0, st>>>((const uint32_t*)key, child, nnum, (uint32_t*)out);
  OCNN_LAUNCH_OK("key_depad_kernel");
  return OCNN_OK;
}

int ocnn_octree_interp(const void* data, void* out, const float* pts, const void* keys, int n_key,
                       int channels, int h, int64_t n_pts, int depth, int key_bits, int linear,
                       int dtype, int layout, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(key_bits == 32 || key_bits == 64, "ocnn_octree_interp: key_bits must be 32 or 64");
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16, "ocnn_octree_interp: unknown dtype %d", dtype);
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR, "ocnn_octree_interp: unknown layout %d", layout);
  OCNN_REQUIRE(channels > 0 && h >= 0 && n_pts >= 0 && n_key >= 0 && n_key <= h,
               "ocnn_octree_interp: bad sizes (C=%d, H=%d, keys=%d)", channels, h, n_key);
  OCNN_REQUIRE(depth >= 1 && depth <= (key_bits == 64 ? 16 : 8), "ocnn_octree_interp: depth %d out of range", depth);
  if (n_pts == 0) return OCNN_OK;
  OCNN_REQUIRE(out && pts && (data || h == 0) && (keys || n_key == 0), "ocnn_octree_interp: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define OCNN_INTERP(T)                                                                              \
  (key_bits == 64 ? interp_impl<T, uint64_t>(data, out, pts, keys, n_key, channels, h, n_pts, depth, \
                                             linear, layout, st)                                     \
                  : interp_impl<T, uint32_t>(data, out, pts, keys, n_key, channels, h, n_pts, depth, \
                                             linear, layout, st))
  if (dtype == OCNN_F32) return OCNN_INTERP(float);
  if (dtype == OCNN_F16) return OCNN_INTERP(__half);
  return OCNN_INTERP(__nv_bfloat16);
#undef OCNN_INTERP
}

int ocnn_octree_align(const void* src, void* dst, const int32_t* idx, int channels, int src_h,
                      int dst_h, int dtype, int layout, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16, "ocnn_octree_align: unknown dtype %d", dtype);
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR, "ocnn_octree_align: unknown layout %d", layout);
  OCNN_REQUIRE(channels > 0 && src_h >= 0 && dst_h >= 0, "ocnn_octree_align: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t esize = dtype == OCNN_F32 ? 4 : 2;
  if (dst_h > 0) {
    OCNN_REQUIRE(dst != nullptr, "ocnn_octree_align: null output");
    OCNN_CUDA_OK(cudaMemsetAsync(dst, 0, esize * (size_t)channels * dst_h, st));
  }
  if (src_h == 0 || dst_h == 0) return OCNN_OK;
  OCNN_REQUIRE(src && idx, "ocnn_octree_align: null pointer");
  const long long total = (long long)channels * src_h;
  const int grid = grid_for(total, 256);
  const bool nm = layout == OCNN_NODE_MAJOR;
  if (dtype == OCNN_F32) {
    if (nm) align_kernel<float, true><<<grid, 256, 0, st>>>((const float*)src, (float*)dst, idx, channels, src_h, dst_h, total);
    else align_kernel<float, false><<<grid, 256, 0, st>>>((const float*)src, (float*)dst, idx, channels, src_h, dst_h, total);
  } else {   // both 16-bit types only move bits
    if (nm) align_kernel<uint16_t, true><<<grid, 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, idx, channels, src_h, dst_h, total);
    else align_kernel<uint16_t, false><<<grid, 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, idx, channels, src_h, dst_h, total);
  }
  OCNN_LAUNCH_OK("align_kernel");
  return OCNN_OK;
}

int ocnn_octree_align_backward(const void* dst_grad, void* src_grad, const int32_t* idx, int channels,
                               int src_h, int dst_h, int dtype, int layout, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16,
               "ocnn_octree_align_backward: unknown dtype %d", dtype);
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR,
               "ocnn_octree_align_backward: unknown layout %d", layout);
  OCNN_REQUIRE(channels > 0 && src_h >= 0 && dst_h >= 0, "ocnn_octree_align_backward: bad sizes");
  if (src_h == 0) return OCNN_OK;
  OCNN_REQUIRE(src_grad && idx && (dst_grad || dst_h == 0), "ocnn_octree_align_backward: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long total = (long long)channels * src_h;
  const int grid = grid_for(total, 256);
  const bool nm = layout == OCNN_NODE_MAJOR;
  if (dtype == OCNN_F32) {
    if (nm) align_back_kernel<float, true><<<grid, 256, 0, st>>>((float*)src_grad, (const float*)dst_grad, idx, channels, src_h, dst_h, total);
    else align_back_kernel<float, false><<<grid, 256, 0, st>>>((float*)src_grad, (const float*)dst_grad, idx, channels, src_h, dst_h, total);
  } else {
    if (nm) align_back_kernel<uint16_t, true><<<grid, 256, 0, st>>>((uint16_t*)src_grad, (const uint16_t*)dst_grad, idx, channels, src_h, dst_h, total);
    else align_back_kernel<uint16_t, false><<<grid, 256, 0, st>>>((uint16_t*)src_grad, (const uint16_t*)dst_grad, idx, channels, src_h, dst_h, total);
  }
  OCNN_LAUNCH_OK("align_back_kernel");
  return OCNN_OK;
}

}  // extern "C"
