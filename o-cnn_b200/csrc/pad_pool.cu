// octree_pad, octree_depad and octree_max_pool: pure bandwidth kernels.
//
// Channel-major fp32 is the reference's tensor layout ([1,C,H,1] contiguous); node-major
// ([H,C], fp32 or bf16) is what the tensor-core convolution consumes.  Both layouts are served by
// the same entry points.  All kernels are grid-stride over 16-byte vectors where the shapes allow,
// with grids sized in whole waves over the SMs.
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

// ---- node-major: rows of C elements; one thread per 16-byte chunk of a row ---------------------
// row_bytes must be a multiple of 16 for the vector kernels.
__global__ void pad_nm_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y,
                                  const int* __restrict__ child, int Hy, int chunks, uint4 fill) {
  const long long total = (long long)Hy * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(i / chunks), q = (int)(i % chunks);
    const int l = child[h];
    y[i] = l < 0 ? fill : x[(long long)l * chunks + q];
  }
}

__global__ void depad_nm_vec_kernel(const uint4* __restrict__ y, uint4* __restrict__ x,
                                    const int* __restrict__ child, int Hy, int chunks) {
  const long long total = (long long)Hy * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(i / chunks), q = (int)(i % chunks);
    const int l = child[h];
    if (l >= 0) x[(long long)l * chunks + q] = y[i];
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

// ---- max pool ------------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

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

template <typename T>
T fill_value(float val);
template <>
float fill_value<float>(float val) { return val; }
template <>
__nv_bfloat16 fill_value<__nv_bfloat16>(float val) { return __float2bfloat16(val); }

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
      pad_nm_vec_kernel<<<grid_for((long long)Hy * chunks, 256), 256, 0, st>>>(
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
    depad_cm_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)y, (T*)x, child, C, Hx, Hy);
  } else {
    const size_t row = (size_t)C * sizeof(T);
    if (row % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
      const int chunks = (int)(row / 16);
      depad_nm_vec_kernel<<<grid_for((long long)Hy * chunks, 256), 256, 0, st>>>(
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
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16, "%s: unknown dtype %d", op, dtype);
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
  return dtype == OCNN_F32 ? pad_impl<float>(x, y, child, C, hx, hy, val, layout, st)
                           : pad_impl<__nv_bfloat16>(x, y, child, C, hx, hy, val, layout, st);
}

int ocnn_octree_depad(const void* y, void* x, const int32_t* child, int C, int hx, int hy,
                      int dtype, int layout, void* stream) {
  using namespace ocnn;
  if (hy == 0 || hx == 0) return OCNN_OK;
  if (int s = check_common("ocnn_octree_depad", y, x, child, C, dtype, layout)) return s;
  OCNN_REQUIRE(hx > 0 && hx <= hy, "ocnn_octree_depad: need 0 < hx (%d) <= hy (%d)", hx, hy);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == OCNN_F32 ? depad_impl<float>(y, x, child, C, hx, hy, layout, st)
                           : depad_impl<__nv_bfloat16>(y, x, child, C, hx, hy, layout, st);
}

int ocnn_octree_max_pool(const void* btm, void* top, int32_t* mask, int C, int top_h, int dtype,
                         int layout, void* stream) {
  using namespace ocnn;
  if (top_h == 0) return OCNN_OK;
  if (int s = check_common("ocnn_octree_max_pool", btm, top, mask, C, dtype, layout)) return s;
  OCNN_REQUIRE(top_h > 0, "ocnn_octree_max_pool: negative height");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == OCNN_F32 ? pool_impl<float>(btm, top, mask, C, top_h, layout, st)
                           : pool_impl<__nv_bfloat16>(btm, top, mask, C, top_h, layout, st);
}

}  // extern "C"
