// octree2col as a stand-alone operator (the reference exposes it; the convolution here never
// materialises the column matrix).  col[(c*K + k)*H + h] = data[c*octree_h + nbr(h,k)] or 0,
// restating octree2col_cpu, octree/octree/octree_nn.cpp:188-214.
#include "common.cuh"

namespace ocnn {
namespace {

struct TapsArg { int count; signed char tap[27]; };

__global__ void octree2col_kernel(const float* __restrict__ data, float* __restrict__ col,
                                  const int* __restrict__ neigh, int K, int H, long long octree_h,
                                  int stride, TapsArg taps, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(i % H);
    const long long ck = i / H;
    const int k = (int)(ck % K);
    const long long c = ck / K;
    const int tap = taps.tap[k];
    const long long at = stride == 2 ? ((long long)h << 6) + ni333(0, tap)
                                     : ((long long)(h >> 3) << 6) + ni333(h & 7, tap);
    const int p = neigh[at];
    col[i] = p < 0 ? 0.0f : data[c * octree_h + p];
  }
}

// On the non-empty nodes only (octree2colP_cpu, octree/octree/octree_nn.cpp:244-271): data holds
// octree_h rows (the non-empty nodes); at stride 1 column row h is the h-th non-empty node
// (node ichild[h]), at stride 2 it is sibling group h; the gathered node goes through child.
// SCATTER = the transpose (col2octree_cpu / col2octreeP_cpu, octree_nn.cpp:216-241, 273-298):
// data[c, p] += col[c, k, h], with atomic additions as the reference's GPU kernel does
// (octree_nn.cu:130-147, 203-228).
template <bool SCATTER>
__global__ void col_general_kernel(float* __restrict__ data, float* __restrict__ col,
                                   const int* __restrict__ neigh, const int* __restrict__ child,
                                   const int* __restrict__ ichild, int K, int H, long long octree_h,
                                   int stride, TapsArg taps, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(i % H);
    const long long ck = i / H;
    const int k = (int)(ck % K);
    const long long c = ck / K;
    const int tap = taps.tap[k];
    long long at;
    if (stride == 2) {
      at = ((long long)h << 6) + ni333(0, tap);
    } else {
      const int hp = ichild != nullptr ? ichild[h] : h;
      at = ((long long)(hp >> 3) << 6) + ni333(hp & 7, tap);
    }
    int p = neigh[at];
    if (child != nullptr && p >= 0) p = child[p];
    if (SCATTER) {
      if (p >= 0) atomicAdd(data + c * octree_h + p, col[i]);
    } else {
      col[i] = p < 0 ? 0.0f : data[c * octree_h + p];
    }
  }
}

int col_general(bool scatter, float* data, float* col, const int32_t* neigh, const int32_t* child,
                const int32_t* ichild, int channels, int h_col, int octree_h,
                const int kernel_size[3], int stride, void* stream, const char* who) {
  OCNN_REQUIRE(data && col && neigh && kernel_size, "%s: null pointer", who);
  OCNN_REQUIRE(stride == 1 || stride == 2, "%s: stride must be 1 or 2 (got %d)", who, stride);
  OCNN_REQUIRE(child == nullptr || stride == 2 || ichild != nullptr,
               "%s: ichild is required with child at stride 1", who);
  const TapList tl = taps_for_kernel(kernel_size);
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "%s: unsupported kernel size %dx%dx%d", who, kernel_size[0],
                kernel_size[1], kernel_size[2]);
  OCNN_REQUIRE(channels >= 0 && h_col >= 0 && octree_h >= 0, "%s: negative size", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (scatter && channels > 0 && octree_h > 0)
    OCNN_CUDA_OK(cudaMemsetAsync(data, 0, sizeof(float) * (size_t)channels * octree_h, st));
  if (h_col == 0 || channels == 0) return OCNN_OK;
  TapsArg ta;
  ta.count = tl.count;
  for (int i = 0; i < 27; ++i) ta.tap[i] = i < tl.count ? tl.tap[i] : 0;
  const long long total = (long long)channels * tl.count * h_col;
  if (scatter)
    col_general_kernel<true><<<grid_for(total, 256), 256, 0, st>>>(
        data, col, neigh, child, child ? ichild : nullptr, tl.count, h_col, octree_h, stride, ta, total);
  else
    col_general_kernel<false><<<grid_for(total, 256), 256, 0, st>>>(
        data, col, neigh, child, child ? ichild : nullptr, tl.count, h_col, octree_h, stride, ta, total);
  OCNN_LAUNCH_OK("col_general_kernel");
  return OCNN_OK;
}

}  // namespace
}  // namespace ocnn

extern "C" int ocnn_octree2col_general(const float* data, float* col, const int32_t* neigh,
                                       const int32_t* child, const int32_t* ichild, int channels,
                                       int h_col, int octree_h, const int kernel_size[3], int stride,
                                       void* stream) {
  return ocnn::col_general(false, const_cast<float*>(data), col, neigh, child, ichild, channels, h_col,
                           octree_h, kernel_size, stride, stream, "ocnn_octree2col_general");
}

extern "C" int ocnn_col2octree(const float* col, float* data, const int32_t* neigh,
                               const int32_t* child, const int32_t* ichild, int channels, int h_col,
                               int octree_h, const int kernel_size[3], int stride, void* stream) {
  return ocnn::col_general(true, data, const_cast<float*>(col), neigh, child, ichild, channels, h_col,
                           octree_h, kernel_size, stride, stream, "ocnn_col2octree");
}

extern "C" int ocnn_octree2col(const float* data, float* col, const int32_t* neigh, int channels,
                               int h_out, const int kernel_size[3], int stride, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(data && col && neigh && kernel_size, "ocnn_octree2col: null pointer");
  OCNN_REQUIRE(stride == 1 || stride == 2, "ocnn_octree2col: stride must be 1 or 2 (got %d)", stride);
  const TapList tl = taps_for_kernel(kernel_size);
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "ocnn_octree2col: unsupported kernel size %dx%dx%d",
                kernel_size[0], kernel_size[1], kernel_size[2]);
  if (h_out == 0 || channels == 0) return OCNN_OK;
  TapsArg ta;
  ta.count = tl.count;
  for (int i = 0; i < 27; ++i) ta.tap[i] = i < tl.count ? tl.tap[i] : 0;
  const long long octree_h = stride == 2 ? (long long)h_out * 8 : h_out;
  const long long total = (long long)channels * tl.count * h_out;
  octree2col_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      data, col, neigh, tl.count, h_out, octree_h, stride, ta, total);
  OCNN_LAUNCH_OK("octree2col_kernel");
  return OCNN_OK;
}
