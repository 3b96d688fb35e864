// octree_pad, octree_depad and octree_max_pool: pure bandwidth kernels.
//
// Channel-major fp32 is the reference's tensor layout ([1,C,H,1] contiguous); node-major
// ([H,C], fp32 or bf16) is what the tensor-core convolution consumes.  Both layouts are served by
// the same entry points.  All kernels are grid-stride over 16-byte vectors where the shapes allow,
// with grids sized in whole waves over the SMs.
#include <type_traits>

#include "common.cuh"

namespace ocnn {
namespace {

// ---- channel-major: y[c*Hy + h] = child[h] < 0 ? val : x[c*Hx + child[h]] --------------------
// One thread per 4 consecutive h of one channel (Hy is a multiple of 8 at every octree level
// d >= 1, so rows stay 16-byte aligned); falls back to scalars when Hy % 4 != 0.
template <typename T>
__global__ void pad_cm_kernel(const T* __restrict__ x, T* __restrict__ y,
                              const int* __restrict__ child, int C, int Hx, int Hy, T val) {
  const long long total = (long long)C * Hy;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i / Hy), h = (int)(i % Hy);
    const int l = child[h];
    y[i] = l < 0 ? val : x[(long long)c * Hx + l];
  }
}

__global__ void pad_cm_f32x4_kernel(const float* __restrict__ x, float* __restrict__ y,
                                    const int* __restrict__ child, int C, int Hx, int Hy,
                                    float val) {
  const int hv = Hy >> 2;
  const long long total = (long long)C * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i / hv), h4 = (int)(i % hv);
    const int4 l = reinterpret_cast<const int4*>(child)[h4];
    const float* xr = x + (long long)c * Hx;
    float4 v;
    v.x = l.x < 0 ? val : xr[l.x];
    v.y = l.y < 0 ? val : xr[l.y];
    v.z = l.z < 0 ? val : xr[l.z];
    v.w = l.w < 0 ? val : xr[l.w];
    reinterpret_cast<float4*>(y + (long long)c * Hy)[h4] = v;
  }
}

template <typename T>
__global__ void depad_cm_kernel(const T* __restrict__ y, T* __restrict__ x,
                                const int* __restrict__ child, int C, int Hx, int Hy) {
  const long long total = (long long)C * Hy;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i / Hy), h = (int)(i % Hy);
    const int l = child[h];
    if (l >= 0) x[(long long)c * Hx + l] = y[i];
  }
}

// fp32 channel-major depad, four consecutive h per thread (16-byte reads of y and child); the
// grid's y dimension is the channel, so no division per element
__global__ void depad_cm_f32x4_kernel(const float* __restrict__ y, float* __restrict__ x,
                                      const int* __restrict__ child, int Hx, int Hy) {
  const int hv = Hy >> 2;
  const float* yr = y + (long long)blockIdx.y * Hy;
  float* xr = x + (long long)blockIdx.y * Hx;
  for (int h4 = blockIdx.x * blockDim.x + threadIdx.x; h4 < hv; h4 += gridDim.x * blockDim.x) {
    const int4 l = reinterpret_cast<const int4*>(child)[h4];
    const float4 v = reinterpret_cast<const float4*>(yr)[h4];
    if (l.x >= 0) xr[l.x] = v.x;
    if (l.y >= 0) xr[l.y] = v.y;
    if (l.z >= 0) xr[l.z] = v.z;
    if (l.w >= 0) xr[l.w] = v.w;
  }
}

// ---- node-major: rows of C elements; one thread per 16-byte chunk of a row ---------------------
// row_bytes must be a multiple of 16 for the vector kernels.
__global__ void pad_nm_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y,
                                  const int* __restrict__ child, int Hy, int chunks, uint4 fill) {
  // four independent child -> row chains per thread and iteration: one chain per iteration makes
  // the grid-stride loop wait for two dependent reads every time round
  const long long total = (long long)Hy * chunks;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
    int l[4], q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      l[u] = -1; q[u] = 0;
      if (i < total) {
        const int h = (int)(i / chunks);
        q[u] = (int)(i - (long long)h * chunks);
        l[u] = child[h];
      }
    }
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = l[u] < 0 ? fill : x[(long long)l[u] * chunks + q[u]];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) y[i] = v[u];
    }
  }
}

__global__ void depad_nm_vec_kernel(const uint4* __restrict__ y, uint4* __restrict__ x,
                                    const int* __restrict__ child, int Hy, int chunks) {
  const long long total = (long long)Hy * chunks;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
    int l[4], q[4];
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {                    // all reads of the four items first
      const long long i = i0 + u * stride;
      l[u] = -1; q[u] = 0; v[u] = make_uint4(0, 0, 0, 0);
      if (i < total) {
        const int h = (int)(i / chunks);
        q[u] = (int)(i - (long long)h * chunks);
        l[u] = child[h];
        v[u] = y[i];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (l[u] >= 0) x[(long long)l[u] * chunks + q[u]] = v[u];
  }
}

template <typename T>
__global__ void pad_nm_kernel(const T* __restrict__ x, T* __restrict__ y,
                              const int* __restrict__ child, int Hy, int C, T val) {
  const long long total = (long long)Hy * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(i / C), c = (int)(i % C);
    const int l = child[h];
    y[i] = l < 0 ? val : x[(long long)l * C + c];
  }
}

template <typename T>
__global__ void depad_nm_kernel(const T* __restrict__ y, T* __restrict__ x,
                                const int* __restrict__ child, int Hy, int C) {
  const long long total = (long long)Hy * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(i / C), c = (int)(i % C);
    const int l = child[h];
    if (l >= 0) x[(long long)l * C + c] = y[i];
  }
}

// ---- tile: nearest-neighbour upsampling, depad followed by "repeat each row for its 8 children" ---
// out[., 8*child[h] + j] = y[., h] for child[h] >= 0, j = 0..7.  Every row of the finer level is
// written (each of its nodes has a non-empty parent).
__global__ void tile_nm_vec_kernel(const uint4* __restrict__ y, uint4* __restrict__ out,
                                   const int* __restrict__ child, int Hy, int chunks) {
  const long long total = (long long)Hy * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(i / chunks), q = (int)(i - (long long)h * chunks);
    const int l = child[h];
    if (l < 0) continue;
    const uint4 v = y[i];
    uint4* dst = out + (long long)l * 8 * chunks + q;
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[(long long)j * chunks] = v;
  }
}

template <typename T>
__global__ void tile_kernel(const T* __restrict__ y, T* __restrict__ out,
                            const int* __restrict__ child, int C, int Hy, long long Hout,
                            int node_major) {
  const long long total = (long long)C * Hy;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int c, h;
    if (node_major) { h = (int)(i / C); c = (int)(i % C); } else { c = (int)(i / Hy); h = (int)(i % Hy); }
    const int l = child[h];
    if (l < 0) continue;
    const T v = y[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long row = (long long)l * 8 + j;
      out[node_major ? row * C + c : (long long)c * Hout + row] = v;
    }
  }
}

// ---- max pool ------------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

// channel-major: one thread per (channel, group): 8 consecutive values = two 16-byte loads (fp32).
__global__ void max_pool_cm_f32_kernel(const float* __restrict__ btm, float* __restrict__ top,
                                       int* __restrict__ mask, int top_h, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    // btm row stride is 8*top_h and top row stride is top_h, so the flat group index i maps to
    // the 8 flat bottom values 8i .. 8i+7 whatever the channel is.
    const float4 a = reinterpret_cast<const float4*>(btm)[2 * i];
    const float4 b = reinterpret_cast<const float4*>(btm)[2 * i + 1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float best = v[0];
    int at = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (v[j] > best) { best = v[j]; at = j; }
    top[i] = best;
    mask[i] = 8 * (int)(i % top_h) + at;  // row inside the channel
  }
}

template <typename T>
__global__ void max_pool_cm_kernel(const T* __restrict__ btm, T* __restrict__ top,
                                   int* __restrict__ mask, int top_h, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const T* v = btm + 8 * i;
    int at = 0;
    float best = to_f32(v[0]);
#pragma unroll
    for (int j = 1; j < 8; ++j) {
      const float f = to_f32(v[j]);
      if (f > best) { best = f; at = j; }
    }
    top[i] = v[at];
    mask[i] = 8 * (int)(i % top_h) + at;
  }
}

// node-major: one thread per (group, channel); consecutive threads walk consecutive channels, so
// each of the 8 row reads is coalesced across the warp.
template <typename T>
__global__ void max_pool_nm_kernel(const T* __restrict__ btm, T* __restrict__ top,
                                   int* __restrict__ mask, int C, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long g = i / C;
    const int c = (int)(i % C);
    const T* v = btm + g * 8 * C + c;
    int at = 0;
    float best = to_f32(v[0]);
#pragma unroll
    for (int j = 1; j < 8; ++j) {
      const float f = to_f32(v[(long long)j * C]);
      if (f > best) { best = f; at = j; }
    }
    top[i] = v[(long long)at * C];
    mask[i] = (int)(8 * g) + at;
  }
}

// bf16 node-major, C a multiple of 8: one thread per (sibling group, 8-channel chunk).  The eight
// children's chunks are eight 16-byte loads in flight at once; the result is one 16-byte store
// (plus two for the argmax rows when the caller wants them).
// PADDED: the output has one row per node of the parent level; child[p] gives the sibling group
// of node p (or < 0: the row is zero) — max pool and the pad that follows it in one pass.
// HALF: the 16-bit elements are fp16 instead of bf16.
template <bool PADDED, bool HALF>
__global__ void __launch_bounds__(256) max_pool_nm_bf16x8_kernel(
    const uint4* __restrict__ btm, uint4* __restrict__ top, int* __restrict__ mask,
    const int* __restrict__ child, int chunks, long long total) {
  grid_dependency_trigger();
  grid_dependency_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / chunks;
    const int q = (int)(i - row * chunks);
    long long g = row;
    if (PADDED) {
      g = child[row];
      if (g < 0) {
        top[i] = make_uint4(0, 0, 0, 0);
        continue;
      }
    }
    const uint4* src = btm + g * 8 * chunks + q;
    uint4 raw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) raw[j] = src[(long long)j * chunks];
    float best[8];
    int at[8];
    {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&raw[0]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack2(p[k], HALF);
        best[2 * k] = f.x; best[2 * k + 1] = f.y;
        at[2 * k] = 0; at[2 * k + 1] = 0;
      }
    }
#pragma unroll
    for (int j = 1; j < 8; ++j) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&raw[j]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack2(p[k], HALF);
        if (f.x > best[2 * k]) { best[2 * k] = f.x; at[2 * k] = j; }
        if (f.y > best[2 * k + 1]) { best[2 * k + 1] = f.y; at[2 * k + 1] = j; }
      }
    }
    // the winner's own bits (the values are exact 16-bit floats, so the round trip through fp32 is too)
    uint4 out;
    uint32_t* op = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int k = 0; k < 4; ++k) op[k] = pack2(best[2 * k], best[2 * k + 1], HALF);
    top[i] = out;
    if (mask != nullptr) {
      const int base = (int)(8 * g);
      int4* m = reinterpret_cast<int4*>(mask + i * 8);
      m[0] = make_int4(base + at[0], base + at[1], base + at[2], base + at[3]);
      m[1] = make_int4(base + at[4], base + at[5], base + at[6], base + at[7]);
    }
  }
}

template <typename T>
T fill_value(float val);
template <>
float fill_value<float>(float val) { return val; }
template <>
__nv_bfloat16 fill_value<__nv_bfloat16>(float val) { return __float2bfloat16(val); }
template <>
__half fill_value<__half>(float val) { return __float2half(val); }

template <typename T>
int pad_impl(const void* x, void* y, const int* child, int C, int Hx, int Hy, float val,
             int layout, cudaStream_t st) {
  const T fv = fill_value<T>(val);
  const long long total = (long long)C * Hy;
  if (total == 0) return OCNN_OK;
  if (layout == OCNN_CHANNEL_MAJOR) {
    const bool vec = sizeof(T) == 4 && Hy % 4 == 0 && ((uintptr_t)y % 16 == 0) &&
                     ((uintptr_t)child % 16 == 0);
    if (vec) {
      pad_cm_f32x4_kernel<<<grid_for(total / 4, 256), 256, 0, st>>>(
          (const float*)x, (float*)y, child, C, Hx, Hy, val);
    } else {
      pad_cm_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)x, (T*)y, child, C, Hx, Hy, fv);
    }
  } else {
    const size_t row = (size_t)C * sizeof(T);
    if (row % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
      const int chunks = (int)(row / 16);
      union { uint4 v; T e[16 / sizeof(T)]; } f;
      for (size_t k = 0; k < 16 / sizeof(T); ++k) f.e[k] = fv;
      pad_nm_vec_kernel<<<grid_for(((long long)Hy * chunks + 3) / 4, 256), 256, 0, st>>>(
          (const uint4*)x, (uint4*)y, child, Hy, chunks, f.v);
    } else {
      pad_nm_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)x, (T*)y, child, Hy, C, fv);
    }
  }
  OCNN_LAUNCH_OK("octree_pad");
  return OCNN_OK;
}

template <typename T>
int depad_impl(const void* y, void* x, const int* child, int C, int Hx, int Hy, int layout,
               cudaStream_t st) {
  const long long total = (long long)C * Hy;
  if (total == 0) return OCNN_OK;
  if (layout == OCNN_CHANNEL_MAJOR) {
    if (sizeof(T) == 4 && Hy % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)child % 16 == 0 && C <= 65535) {
      const int gx = grid_for(Hy / 4, 256, 8);
      depad_cm_f32x4_kernel<<<dim3(gx, C), 256, 0, st>>>((const float*)y, (float*)x, child, Hx, Hy);
    } else {
      depad_cm_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)y, (T*)x, child, C, Hx, Hy);
    }
  } else {
    const size_t row = (size_t)C * sizeof(T);
    if (row % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
      const int chunks = (int)(row / 16);
      depad_nm_vec_kernel<<<grid_for(((long long)Hy * chunks + 3) / 4, 256), 256, 0, st>>>(
          (const uint4*)y, (uint4*)x, child, Hy, chunks);
    } else {
      depad_nm_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)y, (T*)x, child, Hy, C);
    }
  }
  OCNN_LAUNCH_OK("octree_depad");
  return OCNN_OK;
}

template <typename T>
int pool_impl(const void* btm, void* top, int* mask, int C, int top_h, int layout,
              cudaStream_t st) {
  const long long total = (long long)C * top_h;
  if (total == 0) return OCNN_OK;
  if (layout == OCNN_CHANNEL_MAJOR) {
    if (sizeof(T) == 4 && (uintptr_t)btm % 16 == 0) {
      max_pool_cm_f32_kernel<<<grid_for(total, 256), 256, 0, st>>>((const float*)btm, (float*)top,
                                                                   mask, top_h, total);
    } else {
      max_pool_cm_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)btm, (T*)top, mask,
                                                                  top_h, total);
    }
  } else if (sizeof(T) == 2 && C % 8 == 0 && (uintptr_t)btm % 16 == 0 && (uintptr_t)top % 16 == 0 &&
             (uintptr_t)mask % 16 == 0) {
    const long long vec_total = total / 8;
    constexpr bool kHalf = std::is_same<T, __half>::value;
    OCNN_CUDA_OK(launch_chained(max_pool_nm_bf16x8_kernel<false, kHalf>, dim3(grid_for(vec_total, 256, 8)),
                                dim3(256), 0, st, (const uint4*)btm, (uint4*)top, mask,
                                (const int*)nullptr, C / 8, vec_total));
  } else {
    max_pool_nm_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)btm, (T*)top, mask, C,
                                                                total);
  }
  OCNN_LAUNCH_OK("octree_max_pool");
  return OCNN_OK;
}

int check_common(const char* op, const void* a, const void* b, const void* c, int C, int dtype,
                 int layout) {
  OCNN_REQUIRE(a != nullptr && b != nullptr && c != nullptr, "%s: null pointer", op);
  OCNN_REQUIRE(C > 0, "%s: channels must be positive (got %d)", op, C);
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16, "%s: unknown dtype %d", op,
               dtype);
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR, "%s: unknown layout %d",
               op, layout);
  return OCNN_OK;
}

}  // namespace
}  // namespace ocnn

extern "C" {

int ocnn_octree_pad(const void* x, void* y, const int32_t* child, int C, int hx, int hy, float val,
                    int dtype, int layout, void* stream) {
  using namespace ocnn;
  if (hy == 0) return OCNN_OK;
  if (int s = check_common("ocnn_octree_pad", hx > 0 ? x : y, y, child, C, dtype, layout)) return s;
  OCNN_REQUIRE(hx >= 0 && hy > 0 && hx <= hy, "ocnn_octree_pad: need 0 <= hx (%d) <= hy (%d)", hx, hy);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == OCNN_F32) return pad_impl<float>(x, y, child, C, hx, hy, val, layout, st);
  if (dtype == OCNN_F16) return pad_impl<__half>(x, y, child, C, hx, hy, val, layout, st);
  return pad_impl<__nv_bfloat16>(x, y, child, C, hx, hy, val, layout, st);
}

int ocnn_octree_max_pool_pad(const void* btm, void* top, const int32_t* child, int C, int btm_h,
                             int top_h, int dtype, int layout, void* stream) {
  using namespace ocnn;
  if (top_h == 0) return OCNN_OK;
  if (int s = check_common("ocnn_octree_max_pool_pad", btm_h > 0 ? btm : top, top, child, C, dtype, layout))
    return s;
  OCNN_REQUIRE(btm_h >= 0 && btm_h % 8 == 0 && top_h >= btm_h / 8,
               "ocnn_octree_max_pool_pad: need btm_h (%d) = 8 * groups and top_h (%d) >= groups",
               btm_h, top_h);
  OCNN_REQUIRE(dtype != OCNN_F32 && layout == OCNN_NODE_MAJOR && C % 8 == 0,
               "ocnn_octree_max_pool_pad: bf16 / fp16 node-major data with C %% 8 == 0 only (C = %d); "
               "use ocnn_octree_max_pool + ocnn_octree_pad otherwise", C);
  OCNN_REQUIRE((uintptr_t)btm % 16 == 0 && (uintptr_t)top % 16 == 0,
               "ocnn_octree_max_pool_pad: data pointers must be 16-byte aligned");
  const long long total = (long long)top_h * (C / 8);
  auto kernel = dtype == OCNN_F16 ? max_pool_nm_bf16x8_kernel<true, true>
                                  : max_pool_nm_bf16x8_kernel<true, false>;
  OCNN_CUDA_OK(launch_chained(kernel, dim3(grid_for(total, 256, 8)), dim3(256),
                              0, static_cast<cudaStream_t>(stream), (const uint4*)btm, (uint4*)top,
                              (int*)nullptr, (const int*)child, C / 8, total));
  OCNN_LAUNCH_OK("octree_max_pool_pad");
  return OCNN_OK;
}

int ocnn_octree_depad(const void* y, void* x, const int32_t* child, int C, int hx, int hy,
                      int dtype, int layout, void* stream) {
  using namespace ocnn;
  if (hy == 0 || hx == 0) return OCNN_OK;
  if (int s = check_common("ocnn_octree_depad", y, x, child, C, dtype, layout)) return s;
  OCNN_REQUIRE(hx > 0 && hx <= hy, "ocnn_octree_depad: need 0 < hx (%d) <= hy (%d)", hx, hy);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // a depad only moves elements: both 16-bit types take the same kernels
  return dtype == OCNN_F32 ? depad_impl<float>(y, x, child, C, hx, hy, layout, st)
                           : depad_impl<__nv_bfloat16>(y, x, child, C, hx, hy, layout, st);
}

int ocnn_octree_tile(const void* y, void* out, const int32_t* child, int C, int hy, int hout,
                     int dtype, int layout, void* stream) {
  using namespace ocnn;
  if (hy == 0 || hout == 0) return OCNN_OK;
  if (int s = check_common("ocnn_octree_tile", y, out, child, C, dtype, layout)) return s;
  OCNN_REQUIRE(hy > 0 && hout > 0 && hout % 8 == 0, "ocnn_octree_tile: need hy (%d) > 0 and hout (%d) "
               "a multiple of 8", hy, hout);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t esize = dtype == OCNN_F32 ? 4 : 2;
  const size_t row = (size_t)C * esize;
  if (layout == OCNN_NODE_MAJOR && row % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0) {
    const int chunks = (int)(row / 16);
    tile_nm_vec_kernel<<<grid_for((long long)hy * chunks, 256), 256, 0, st>>>(
        (const uint4*)y, (uint4*)out, child, hy, chunks);
  } else if (dtype == OCNN_F32) {
    tile_kernel<float><<<grid_for((long long)C * hy, 256), 256, 0, st>>>(
        (const float*)y, (float*)out, child, C, hy, hout, layout == OCNN_NODE_MAJOR);
  } else {
    tile_kernel<__nv_bfloat16><<<grid_for((long long)C * hy, 256), 256, 0, st>>>(
        (const __nv_bfloat16*)y, (__nv_bfloat16*)out, child, C, hy, hout, layout == OCNN_NODE_MAJOR);
  }
  OCNN_LAUNCH_OK("octree_tile");
  return OCNN_OK;
}

int ocnn_octree_max_pool(const void* btm, void* top, int32_t* mask, int C, int top_h, int dtype,
                         int layout, void* stream) {
  using namespace ocnn;
  if (top_h == 0) return OCNN_OK;
  if (int s = check_common("ocnn_octree_max_pool", btm, top, mask, C, dtype, layout)) return s;
  OCNN_REQUIRE(top_h > 0, "ocnn_octree_max_pool: negative height");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == OCNN_F32) return pool_impl<float>(btm, top, mask, C, top_h, layout, st);
  if (dtype == OCNN_F16) return pool_impl<__half>(btm, top, mask, C, top_h, layout, st);
  return pool_impl<__nv_bfloat16>(btm, top, mask, C, top_h, layout, st);
}

}  // extern "C"
