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

}  // namespace
}  // namespace ocnn

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
