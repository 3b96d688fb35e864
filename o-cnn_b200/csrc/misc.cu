// Small layout-conversion kernels between the octree's stored feature block and the node-major
// tensors the tensor-core convolution reads.
#include "common.cuh"

namespace ocnn {
namespace {

// feature [C, nnum] fp32 channel-major -> out [nnum, c_pad] node-major (zeros in the padding
// channels).  One thread per output element; reads are coalesced along nodes for each channel.
template <typename T>
__global__ void feature_to_nm_kernel(const float* __restrict__ f, T* __restrict__ out, int C,
                                     int c_pad, long long nnum) {
  const long long total = nnum * c_pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long h = i / c_pad;
    const int c = (int)(i % c_pad);
    const float v = c < C ? f[(long long)c * nnum + h] : 0.f;
    out[i] = (T)v;
  }
}

// c_pad == 8, bf16 or fp16: one thread per node — up to 8 coalesced plane reads, one 16-byte row
// store.
__global__ void __launch_bounds__(256) feature_to_nm_bf16x8_kernel(const float* __restrict__ f,
                                                                   uint4* __restrict__ out, int C,
                                                                   long long nnum, bool half) {
  for (long long h = blockIdx.x * (long long)blockDim.x + threadIdx.x; h < nnum;
       h += (long long)gridDim.x * blockDim.x) {
    float v[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = c < C ? f[(long long)c * nnum + h] : 0.f;
    uint4 row;
    uint32_t* p = reinterpret_cast<uint32_t*>(&row);
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = pack2(v[2 * k], v[2 * k + 1], half);
    out[h] = row;
  }
}

// Global average pool over each shape's `per` rows followed by a fully connected layer, one CTA per
// shape: the channel means go to shared memory (threads stride over channels: a warp reads
// consecutive channels of one row), then one warp per output computes its dot product.
template <bool HALF>
__global__ void __launch_bounds__(256) global_pool_fc_kernel(const uint16_t* __restrict__ x,
                                                             const float* __restrict__ w,
                                                             const float* __restrict__ bias,
                                                             float* __restrict__ out, int per, int C,
                                                             int nout) {
  extern __shared__ float s_mean[];
  grid_dependency_wait();
  const int b = blockIdx.x;
  const uint16_t* xb = x + (long long)b * per * C;
  const float inv = 1.f / (float)per;
  for (int c2 = threadIdx.x; 2 * c2 < C; c2 += blockDim.x) {
    float s0 = 0.f, s1 = 0.f;
    // (eight rows requested at a time: one load per iteration left the sum waiting on each)
    int i = 0;
    for (; i + 8 <= per; i += 8) {
      uint32_t r[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) r[k] = *reinterpret_cast<const uint32_t*>(xb + (long long)(i + k) * C + 2 * c2);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float2 v = unpack2(r[k], HALF);
        s0 += v.x;
        s1 += v.y;
      }
    }
    for (; i < per; ++i) {
      const float2 v = unpack2(*reinterpret_cast<const uint32_t*>(xb + (long long)i * C + 2 * c2), HALF);
      s0 += v.x;
      s1 += v.y;
    }
    s_mean[2 * c2] = s0 * inv;
    s_mean[2 * c2 + 1] = s1 * inv;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int o = warp; o < nout; o += blockDim.x >> 5) {
    float acc = 0.f;
    const float* wr = w + (long long)o * C;
    int c = lane;
    for (; c + 7 * 32 < C; c += 8 * 32) {        // eight weight reads in flight
      float wv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) wv[k] = wr[c + 32 * k];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc = fmaf(wv[k], s_mean[c + 32 * k], acc);
    }
    for (; c < C; c += 32) acc = fmaf(wr[c], s_mean[c], acc);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) out[(long long)b * nout + o] = acc + (bias ? bias[o] : 0.f);
  }
}

}  // namespace
}  // namespace ocnn

extern "C" int ocnn_global_pool_fc(const void* x, const float* w, const float* bias, float* out, int batch,
                                   int per, int channels, int nout, int dtype, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(x && w && out, "ocnn_global_pool_fc: null pointer");
  OCNN_REQUIRE(dtype == OCNN_BF16 || dtype == OCNN_F16, "ocnn_global_pool_fc: bf16 or fp16 node-major data");
  OCNN_REQUIRE(batch >= 0 && per > 0 && nout > 0 && channels > 0 && channels % 2 == 0 && channels <= 8192,
               "ocnn_global_pool_fc: bad shape (batch %d, per %d, C %d, nout %d)", batch, per, channels, nout);
  OCNN_REQUIRE((uintptr_t)x % 4 == 0, "ocnn_global_pool_fc: data must be 4-byte aligned");
  if (batch == 0) return OCNN_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)channels * sizeof(float);
  if (dtype == OCNN_F16)
    OCNN_CUDA_OK(launch_chained(global_pool_fc_kernel<true>, dim3(batch), dim3(256), smem, st,
                                static_cast<const uint16_t*>(x), w, bias, out, per, channels, nout));
  else
    OCNN_CUDA_OK(launch_chained(global_pool_fc_kernel<false>, dim3(batch), dim3(256), smem, st,
                                static_cast<const uint16_t*>(x), w, bias, out, per, channels, nout));
  OCNN_LAUNCH_OK("global_pool_fc_kernel");
  return OCNN_OK;
}

extern "C" int ocnn_feature_to_node_major(const float* feature, void* out, int channels, int c_pad,
                                          int nnum, int dtype, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(feature && out, "ocnn_feature_to_node_major: null pointer");
  OCNN_REQUIRE(channels > 0 && c_pad >= channels && nnum >= 0,
               "ocnn_feature_to_node_major: bad shape (C=%d, c_pad=%d, nnum=%d)", channels, c_pad, nnum);
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16,
               "ocnn_feature_to_node_major: unknown dtype");
  if (nnum == 0) return OCNN_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long total = (long long)nnum * c_pad;
  if (dtype != OCNN_F32 && c_pad == 8 && (uintptr_t)out % 16 == 0)
    feature_to_nm_bf16x8_kernel<<<grid_for(nnum, 256), 256, 0, st>>>(feature, static_cast<uint4*>(out),
                                                                    channels, nnum, dtype == OCNN_F16);
  else if (dtype == OCNN_F16)
    feature_to_nm_kernel<__half><<<grid_for(total, 256), 256, 0, st>>>(
        feature, static_cast<__half*>(out), channels, c_pad, nnum);
  else if (dtype == OCNN_BF16)
    feature_to_nm_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, st>>>(
        feature, static_cast<__nv_bfloat16*>(out), channels, c_pad, nnum);
  else
    feature_to_nm_kernel<float><<<grid_for(total, 256), 256, 0, st>>>(
        feature, static_cast<float*>(out), channels, c_pad, nnum);
  OCNN_LAUNCH_OK("feature_to_nm_kernel");
  return OCNN_OK;
}
