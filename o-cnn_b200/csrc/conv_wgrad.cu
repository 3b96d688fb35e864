// Weight gradient of the octree convolution / deconvolution and the pooling transposes (training
// support; not on the inference path).
//
// The reference forms the column matrix and multiplies (OctreeBaseConv::weight_gpu_gemm,
// octree/octree/octree_conv.cpp:332-360: octree2col_gpu + GEMM with the top gradient).  Here the
// product is one implicit-GEMM kernel whose reduction runs over the nodes:
//     dW[m, c*K + k] = sum_h A[m, h] * X[c, nbr(h, k)]
// with nbr the convolution's gather (stride 1 or 2, optionally on non-empty nodes).  For the
// convolution A is the output gradient and X the layer's input; for the deconvolution the roles
// swap (pytorch/cpp/octree_conv.cpp:219-253).  The node range is split over CTAs, each adds its
// partial tile to dW with fp32 atomics, so dW must start at zero (the entry point clears it) and the
// summation order is not fixed.
#include "common.cuh"

namespace ocnn {
namespace {

constexpr int WM = 64, WN = 64, WK = 16, WTHREADS = 256;

struct WgradArgs {
  const float* a;       // [M, h_a]
  const float* x;       // [C, h_x]
  float* dw;            // [M, C*K]
  const int* neigh;
  const int* child;
  const int* ichild;
  int M, C, K, h_a, h_x, stride, identity, node_major;
  int rows_per_cta;
  signed char tap[27];
};

__global__ void __launch_bounds__(WTHREADS) conv_wgrad_kernel(const WgradArgs a) {
  __shared__ float As[WK][WM + 4];
  __shared__ float Bs[WK][WN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * WM, n0 = blockIdx.y * WN;
  const int KD = a.C * a.K;
  const long long h_begin = (long long)blockIdx.z * a.rows_per_cta;
  const long long h_end = min((long long)a.h_a, h_begin + a.rows_per_cta);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int tm = tid % 16, tn = tid / 16;
  for (long long h0 = h_begin; h0 < h_end; h0 += WK) {
#pragma unroll
    for (int r = 0; r < (WK * WM) / WTHREADS; ++r) {
      const int e = tid + WTHREADS * r;
      // channel-major A: consecutive threads walk h; node-major: consecutive threads walk m
      const int hl = a.node_major ? e / WM : e % WK;
      const int m = a.node_major ? e % WM : e / WK;
      const long long h = h0 + hl;
      float v = 0.f;
      if (h < h_end && m0 + m < a.M)
        v = a.node_major ? a.a[h * a.M + m0 + m] : a.a[(long long)(m0 + m) * a.h_a + h];
      As[hl][m] = v;
    }
#pragma unroll
    for (int r = 0; r < (WK * WN) / WTHREADS; ++r) {
      const int e = tid + WTHREADS * r;
      const int hl = e % WK, n = e / WK;
      const long long h = h0 + hl;
      const int kd = n0 + n;
      float v = 0.f;
      if (h < h_end && kd < KD) {
        const int c = kd / a.K, k = kd % a.K;
        long long p;
        if (a.identity) {
          p = h;
        } else {
          const int hn = (a.ichild && a.stride == 1) ? a.ichild[h] : (int)h;
          const int tap = a.tap[k];
          const long long at = a.stride == 2 ? ((long long)hn << 6) + ni333(0, tap)
                                             : ((long long)(hn >> 3) << 6) + ni333(hn & 7, tap);
          p = a.neigh[at];
          if (a.child && p >= 0) p = a.child[p];
        }
        if (p >= 0) v = a.node_major ? a.x[p * a.C + c] : a.x[(long long)c * a.h_x + p];
      }
      Bs[hl][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int hl = 0; hl < WK; ++hl) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[hl][tm * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[hl][tn * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm * 4 + i;
    if (m >= a.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kd = n0 + tn * 4 + j;
      if (kd < KD && acc[i][j] != 0.f) atomicAdd(a.dw + (long long)m * KD + kd, acc[i][j]);
    }
  }
}

// octree_max_unpool: btm[., mask] = top (octree_max_unpool_gpu, octree/octree/octree_nn.cu:293-310);
// octree_mask_pool: top = btm[., mask] (:312-329).  mask holds the row inside the channel.
template <bool UNPOOL>
__global__ void mask_pool_kernel(float* __restrict__ top, float* __restrict__ btm,
                                 const int* __restrict__ mask, int C, long long top_h, long long btm_h,
                                 int node_major, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long c, at_btm;
    if (node_major) { c = i % C; at_btm = (long long)mask[i] * C + c; }
    else { c = i / top_h; at_btm = c * btm_h + mask[i]; }
    if (UNPOOL) btm[at_btm] = top[i]; else top[i] = btm[at_btm];
  }
}

}  // namespace
}  // namespace ocnn

extern "C" {

int ocnn_octree_conv_weight_grad(const float* a, const float* x, float* dw,
                                 const ocnn_conv_geometry* g, int m_channels, int x_channels,
                                 const int kernel_size[3], int layout, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(kernel_size != nullptr && g != nullptr, "ocnn_octree_conv_weight_grad: null argument");
  const TapList tl = taps_for_kernel(kernel_size);
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "ocnn_octree_conv_weight_grad: unsupported kernel size %dx%dx%d",
                kernel_size[0], kernel_size[1], kernel_size[2]);
  OCNN_REQUIRE(!g->transposed, "ocnn_octree_conv_weight_grad: pass the convolution-type geometry of the "
               "column matrix (for a deconvolution: swap the operands, see the header)");
  OCNN_REQUIRE(m_channels > 0 && x_channels > 0, "ocnn_octree_conv_weight_grad: channel counts must be positive");
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR,
               "ocnn_octree_conv_weight_grad: unknown layout %d", layout);
  if (int rc = check_conv_geometry(g, tl, "ocnn_octree_conv_weight_grad")) return rc;
  OCNN_REQUIRE(dw != nullptr, "ocnn_octree_conv_weight_grad: null output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long kd = (long long)x_channels * tl.count;
  OCNN_CUDA_OK(cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)m_channels * kd, st));
  if (g->h_out == 0 || g->h_in == 0) return OCNN_OK;
  OCNN_REQUIRE(a && x, "ocnn_octree_conv_weight_grad: null data pointer");
  const bool identity = tl.count == 1 && g->stride == 1;
  WgradArgs w;
  w.a = a; w.x = x; w.dw = dw;
  w.neigh = identity ? nullptr : g->neigh_dev;
  w.child = (g->nempty && !identity) ? g->child_dev : nullptr;
  w.ichild = (g->nempty && !identity && g->stride == 1) ? g->ichild_dev : nullptr;
  w.M = m_channels; w.C = x_channels; w.K = tl.count;
  w.h_a = g->h_out; w.h_x = g->h_in; w.stride = g->stride; w.identity = identity ? 1 : 0;
  w.node_major = layout == OCNN_NODE_MAJOR ? 1 : 0;
  for (int i = 0; i < 27; ++i) w.tap[i] = i < tl.count ? tl.tap[i] : 0;
  const int gx = ceil_div(m_channels, WM), gy = ceil_div(kd, WN);
  // enough node splits to fill the GPU a few times over, each a multiple of the 16-node step
  long long splits = (4LL * sm_count() + (long long)gx * gy - 1) / ((long long)gx * gy);
  const long long max_splits = (g->h_out + 255) / 256;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  w.rows_per_cta = (int)(((g->h_out + splits - 1) / splits + WK - 1) / WK * WK);
  const int gz = ceil_div(g->h_out, w.rows_per_cta);
  conv_wgrad_kernel<<<dim3(gx, gy, gz), WTHREADS, 0, st>>>(w);
  OCNN_LAUNCH_OK("conv_wgrad_kernel");
  return OCNN_OK;
}

int ocnn_octree_max_unpool(const float* top, const int32_t* mask, float* btm, int channels, int top_h,
                           int layout, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(channels > 0 && top_h >= 0, "ocnn_octree_max_unpool: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long total = (long long)channels * top_h;
  if (total == 0) return OCNN_OK;
  OCNN_REQUIRE(top && mask && btm, "ocnn_octree_max_unpool: null pointer");
  OCNN_CUDA_OK(cudaMemsetAsync(btm, 0, sizeof(float) * (size_t)total * 8, st));
  mask_pool_kernel<true><<<grid_for(total, 256), 256, 0, st>>>(
      const_cast<float*>(top), btm, mask, channels, top_h, 8LL * top_h, layout == OCNN_NODE_MAJOR, total);
  OCNN_LAUNCH_OK("mask_pool_kernel");
  return OCNN_OK;
}

int ocnn_octree_mask_pool(const float* btm, const int32_t* mask, float* top, int channels, int top_h,
                          int layout, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(channels > 0 && top_h >= 0, "ocnn_octree_mask_pool: bad sizes");
  const long long total = (long long)channels * top_h;
  if (total == 0) return OCNN_OK;
  OCNN_REQUIRE(top && mask && btm, "ocnn_octree_mask_pool: null pointer");
  mask_pool_kernel<false><<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      top, const_cast<float*>(btm), mask, channels, top_h, 8LL * top_h, layout == OCNN_NODE_MAJOR, total);
  OCNN_LAUNCH_OK("mask_pool_kernel");
  return OCNN_OK;
}

}  // extern "C"
