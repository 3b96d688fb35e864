// Octree convolution as one implicit-GEMM kernel on the CUDA cores (fp32 FMA accumulation).
//
// This is the parity path (fp32 in/out, rel 1e-5 against the reference's octree2col + SGEMM) and
// the general path for shapes the tensor-core kernel does not take (Cin % 8 != 0, channel-major
// data).  The neighbour gather is done while staging the A tile in shared memory, so the
// 27x-inflated column matrix of the reference (octree/octree/octree_conv.cpp:276-298) never
// exists in HBM.
//
// Tile: 64 nodes x 64 output channels per CTA, 256 threads, 4x4 outputs per thread, K walked in
// slices of 16 over the flattened (channel, tap) index.  Channel-major data walks K as
// ci*K + t (the reference's weight column order); node-major data walks t*Cin + ci so that one
// slice reads 16 contiguous channels of a neighbour row.
#include "common.cuh"

namespace ocnn {

int conv_pointwise_bf16(const void* x, const float* w, void* y, int h, int cin, int cout,
                        const ocnn_conv_epilogue* ep, cudaStream_t st, bool f16);   // conv_pw.cu
int conv_pointwise_pool_bf16(const void* x, const float* w, void* top, const int* child_parent, int h,
                             int top_h, int cin, int cout, const ocnn_conv_epilogue* ep, int* inv,
                             cudaStream_t st, bool f16);                            // conv_pw.cu

int conv_pointwise_chain_bf16(const void* x, const float* w1, void* y1, int h, int cin, int cmid,
                              const ocnn_conv_epilogue* ep1, const float* w2, void* y2, int cout2,
                              const ocnn_conv_epilogue* ep2, cudaStream_t st, bool f16);   // conv_pw.cu

namespace {

constexpr int BK = 16;

struct ConvArgs {
  const void* x;
  const float* w;
  void* y;
  const int* neigh;
  const int* child;    // non-empty-node convolution only: child array of the level, and
  const int* ichild;   // its inverse (node of the i-th non-empty node); NULL for the dense one
  int h_in, h_out, cin, cout, K, stride, identity;
  int transposed;      // deconvolution: weights are [Cin, Cout*K], element (ci, co*K + t)
  int up;              // stride-2 deconvolution: rows are nodes of the finer level, x rows are
                       // their parents' ranks among the non-empty nodes (= sibling-group indices)
  const float* scale;
  const float* bias;
  const void* residual;
  int relu;
  signed char tap[27];
};

__device__ __forceinline__ float ld(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ld(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float ld(const __half* p, long long i) { return __half2float(p[i]); }
__device__ __forceinline__ void st(__half* p, long long i, float v) { p[i] = __float2half(v); }
__device__ __forceinline__ void st(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// Tile BM nodes x BN output channels, BM*BN/16 threads, 4x4 outputs per thread.  64x64 (256
// threads) where the level gives the GPU enough of them; 32x32 (64 threads) on small levels, where
// a 64x64 grid would leave SMs without a CTA and every CTA alone with its latency chain.  The K
// loop is software-pipelined: the global loads of slice k+1 (weights and gathered inputs) are
// issued before the FMAs of slice k and land in the other half of a double-buffered pair of
// shared-memory tiles, so a slice costs one barrier.  A thread's (channel, tap) position advances
// by BK per slice and is kept incrementally (no division in the loop).
template <typename T, int LAYOUT, int BM, int BN>
__global__ void __launch_bounds__(BM* BN / 16) conv_simt_kernel(const ConvArgs a) {
  constexpr int THREADS = BM * BN / 16;
  constexpr int RA = (BK * BM) / THREADS, RB = (BK * BN) / THREADS;
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  __shared__ int nbr[27][BM];

  const T* __restrict__ x = static_cast<const T*>(a.x);
  const int tid = threadIdx.x;
  const int h0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int KD = a.cin * a.K;

  // neighbour rows of this tile's nodes, one entry per (tap, node)
  for (int e = tid; e < a.K * BM; e += THREADS) {
    const int t = e / BM, m = e % BM;
    const int h = h0 + m;
    int p = -1;
    if (h < a.h_out) {
      if (a.identity) {
        p = h;
      } else {
        const int tap = a.tap[t];
        // on non-empty nodes only (octree2colP, octree/octree/octree_nn.cu:179-201): row h is the
        // h-th non-empty node, its neighbours are looked up from the node itself and mapped back
        // to ranks among the non-empty nodes
        const int hn = (a.ichild && (a.stride == 1 || a.up)) ? a.ichild[h] : h;
        if (a.up) {
          p = up_source_group(a.neigh, hn, tap);
        } else {
          const long long at = a.stride == 2 ? ((long long)hn << 6) + ni333(0, tap)
                                             : ((long long)(hn >> 3) << 6) + ni333(hn & 7, tap);
          p = a.neigh[at];
          if (a.child && p >= 0) p = a.child[p];
        }
      }
    }
    nbr[t][m] = p;
  }
  __syncthreads();

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int tm = tid % (BM / 4), tn = tid / (BM / 4);

  // this thread's slots in the A and B tiles: (kl, m) / (kl, n) are fixed, the K position of kl
  // advances by BK per slice; (ci, t) of that position is carried along
  int a_kl[RA], a_m[RA], b_kl[RB], b_n[RB];
#pragma unroll
  for (int r = 0; r < RA; ++r) {
    const int e = tid + THREADS * r;
    if (LAYOUT == OCNN_CHANNEL_MAJOR) { a_m[r] = e % BM; a_kl[r] = e / BM; } else { a_kl[r] = e % BK; a_m[r] = e / BK; }
  }
#pragma unroll
  for (int r = 0; r < RB; ++r) {
    const int e = tid + THREADS * r;
    b_kl[r] = e % BK;
    b_n[r] = e / BK;
  }
  auto split = [&](int kk, int& ci, int& t) {
    if (LAYOUT == OCNN_CHANNEL_MAJOR) { ci = kk / a.K; t = kk - ci * a.K; } else { t = kk / a.cin; ci = kk - t * a.cin; }
  };
  int a_ci[RA], a_t[RA], b_ci[RB], b_t[RB];
#pragma unroll
  for (int r = 0; r < RA; ++r) split(a_kl[r], a_ci[r], a_t[r]);
#pragma unroll
  for (int r = 0; r < RB; ++r) split(b_kl[r], b_ci[r], b_t[r]);
  auto advance = [&](int& ci, int& t) {
    // K position += BK
    if (LAYOUT == OCNN_CHANNEL_MAJOR) {
      t += BK;
      while (t >= a.K) { t -= a.K; ++ci; }
    } else {
      ci += BK;
      while (ci >= a.cin) { ci -= a.cin; ++t; }
    }
  };
  auto in_range = [&](int ci, int t) {
    return LAYOUT == OCNN_CHANNEL_MAJOR ? ci < a.cin : t < a.K;
  };

  float ra[RA], rb[RB];
  auto fetch = [&]() {
#pragma unroll
    for (int r = 0; r < RA; ++r) {
      float v = 0.f;
      if (in_range(a_ci[r], a_t[r])) {
        const int p = nbr[a_t[r]][a_m[r]];
        if (p >= 0)
          v = LAYOUT == OCNN_CHANNEL_MAJOR ? ld(x, (long long)a_ci[r] * a.h_in + p)
                                           : ld(x, (long long)p * a.cin + a_ci[r]);
      }
      ra[r] = v;
      advance(a_ci[r], a_t[r]);
    }
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      float v = 0.f;
      const int co = n0 + b_n[r];
      if (in_range(b_ci[r], b_t[r]) && co < a.cout)
        v = a.transposed ? a.w[((long long)b_ci[r] * a.cout + co) * a.K + b_t[r]]
                         : a.w[(long long)co * KD + b_ci[r] * a.K + b_t[r]];
      rb[r] = v;
      advance(b_ci[r], b_t[r]);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int r = 0; r < RA; ++r) As[buf][a_kl[r]][a_m[r]] = ra[r];
#pragma unroll
    for (int r = 0; r < RB; ++r) Bs[buf][b_kl[r]][b_n[r]] = rb[r];
  };

  fetch();
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < KD; k0 += BK) {
    const bool more = k0 + BK < KD;
    if (more) fetch();                 // in flight during the FMAs below
#pragma unroll
    for (int kl = 0; kl < BK; ++kl) {
      const float4 av4 = *reinterpret_cast<const float4*>(&As[buf][kl][tm * 4]);
      const float4 bv4 = *reinterpret_cast<const float4*>(&Bs[buf][kl][tn * 4]);
      const float av[4] = {av4.x, av4.y, av4.z, av4.w};
      const float bv[4] = {bv4.x, bv4.y, bv4.z, bv4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }

  T* __restrict__ y = static_cast<T*>(a.y);
  const T* __restrict__ res = static_cast<const T*>(a.residual);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int co = n0 + tn * 4 + j;
    if (co >= a.cout) continue;
    const float sc = a.scale ? a.scale[co] : 1.f;
    const float bi = a.bias ? a.bias[co] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int h = h0 + tm * 4 + i;
      if (h >= a.h_out) continue;
      const long long at = LAYOUT == OCNN_CHANNEL_MAJOR ? (long long)co * a.h_out + h
                                                        : (long long)h * a.cout + co;
      float v = acc[i][j] * sc + bi;
      if (res) v += ld(res, at);
      if (a.relu) v = fmaxf(v, 0.f);
      st(y, at, v);
    }
  }
}

}  // namespace
}  // namespace ocnn

namespace ocnn {
namespace {

__global__ void ichild_kernel(const int* __restrict__ child, int* __restrict__ ichild, int nnum) {
  for (int h = blockIdx.x * blockDim.x + threadIdx.x; h < nnum; h += gridDim.x * blockDim.x) {
    const int l = child[h];
    if (l >= 0) ichild[l] = h;
  }
}

int conv_simt_launch(const void* x, const float* w, void* y, const int32_t* neigh,
                     const int32_t* child, const int32_t* ichild, int h_in, int h_out, int cin,
                     int cout, const TapList& tl, int stride, int dtype, int layout,
                     const ocnn_conv_epilogue* ep, void* stream, bool transposed = false) {
  const bool identity = tl.count == 1 && stride == 1;
  ConvArgs a;
  a.x = x; a.w = w; a.y = y; a.neigh = neigh; a.child = child; a.ichild = ichild;
  a.h_in = h_in; a.h_out = h_out; a.cin = cin; a.cout = cout;
  a.K = tl.count; a.stride = stride; a.identity = identity ? 1 : 0;
  a.transposed = transposed ? 1 : 0;
  a.up = (transposed && stride == 2) ? 1 : 0;
  a.scale = ep ? ep->scale_dev : nullptr;
  a.bias = ep ? ep->bias_dev : nullptr;
  a.residual = ep ? ep->residual_dev : nullptr;
  a.relu = ep ? ep->relu : 0;
  // a stride-1 deconvolution gathers from the mirrored offsets: node p receives from the node h
  // with p = h + offset(t), i.e. h = p - offset(t)
  for (int i = 0; i < 27; ++i)
    a.tap[i] = i < tl.count ? (signed char)((transposed && stride == 1) ? 26 - tl.tap[i] : tl.tap[i]) : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 64x64 tiles unless they would not even give every SM one CTA: then 32x32 tiles
  const long long big_ctas = (long long)ceil_div(h_out, 64) * ceil_div(cout, 64);
  const bool small = big_ctas < (long long)sm_count();
#define OCNN_SIMT_LAUNCH(TYPE, LAY)                                                                   \
  do {                                                                                                \
    if (small)                                                                                        \
      conv_simt_kernel<TYPE, LAY, 32, 32><<<dim3(ceil_div(h_out, 32), ceil_div(cout, 32)), 64, 0, s>>>(a); \
    else                                                                                              \
      conv_simt_kernel<TYPE, LAY, 64, 64><<<dim3(ceil_div(h_out, 64), ceil_div(cout, 64)), 256, 0, s>>>(a); \
  } while (0)
  if (dtype == OCNN_F32) {
    if (layout == OCNN_CHANNEL_MAJOR) OCNN_SIMT_LAUNCH(float, OCNN_CHANNEL_MAJOR);
    else OCNN_SIMT_LAUNCH(float, OCNN_NODE_MAJOR);
  } else if (dtype == OCNN_F16) {
    if (layout == OCNN_CHANNEL_MAJOR) OCNN_SIMT_LAUNCH(__half, OCNN_CHANNEL_MAJOR);
    else OCNN_SIMT_LAUNCH(__half, OCNN_NODE_MAJOR);
  } else {
    if (layout == OCNN_CHANNEL_MAJOR) OCNN_SIMT_LAUNCH(__nv_bfloat16, OCNN_CHANNEL_MAJOR);
    else OCNN_SIMT_LAUNCH(__nv_bfloat16, OCNN_NODE_MAJOR);
  }
#undef OCNN_SIMT_LAUNCH
  OCNN_LAUNCH_OK("conv_simt_kernel");
  return OCNN_OK;
}

}  // namespace
}  // namespace ocnn

extern "C" int ocnn_octree_conv(const void* x, const float* w, void* y, const int32_t* neigh,
                                int h_in, int h_out, int cin, int cout, const int kernel_size[3],
                                int stride, int dtype, int layout, const ocnn_conv_epilogue* ep,
                                void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(kernel_size != nullptr, "ocnn_octree_conv: null kernel size");
  OCNN_REQUIRE(stride == 1 || stride == 2, "ocnn_octree_conv: stride must be 1 or 2 (got %d)", stride);
  const TapList tl = taps_for_kernel(kernel_size);
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "ocnn_octree_conv: unsupported kernel size %dx%dx%d",
                kernel_size[0], kernel_size[1], kernel_size[2]);
  OCNN_REQUIRE(cin > 0 && cout > 0, "ocnn_octree_conv: channel counts must be positive");
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16,
               "ocnn_octree_conv: unknown dtype %d", dtype);
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR,
               "ocnn_octree_conv: unknown layout %d", layout);
  OCNN_REQUIRE(h_in >= 0 && h_out >= 0, "ocnn_octree_conv: negative height");
  if (h_out == 0) return OCNN_OK;
  const bool identity = tl.count == 1 && stride == 1;
  OCNN_REQUIRE(x && w && y, "ocnn_octree_conv: null data pointer");
  OCNN_REQUIRE(identity || neigh != nullptr, "ocnn_octree_conv: neighbour table required");
  if (stride == 2) {
    OCNN_REQUIRE((long long)h_out * 8 == h_in,
                 "ocnn_octree_conv: stride 2 needs h_in == 8*h_out (got %d, %d)", h_in, h_out);
  } else {
    OCNN_REQUIRE(h_in == h_out, "ocnn_octree_conv: stride 1 needs h_in == h_out (got %d, %d)",
                 h_in, h_out);
  }
  if (identity && dtype != OCNN_F32 && layout == OCNN_NODE_MAJOR) {
    // few-channel pointwise layers: a dedicated streaming kernel (conv_pw.cu)
    const int s = conv_pointwise_bf16(x, w, y, h_out, cin, cout, ep, static_cast<cudaStream_t>(stream),
                                      dtype == OCNN_F16);
    if (s >= 0) return s;
  }
  return conv_simt_launch(x, w, y, neigh, nullptr, nullptr, h_in, h_out, cin, cout, tl, stride, dtype,
                          layout, ep, stream);
}

extern "C" int ocnn_octree_conv1x1_max_pool_pad(const void* x, const float* w, void* top,
                                                const int32_t* child_parent, int h, int top_h, int cin,
                                                int cout, int dtype, const ocnn_conv_epilogue* ep,
                                                int32_t* group_parent, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(x && w && top && child_parent && group_parent, "ocnn_octree_conv1x1_max_pool_pad: null pointer");
  OCNN_REQUIRE(dtype == OCNN_BF16 || dtype == OCNN_F16,
               "ocnn_octree_conv1x1_max_pool_pad: bf16 or fp16 node-major data");
  OCNN_REQUIRE(h >= 0 && h % 8 == 0 && top_h >= h / 8,
               "ocnn_octree_conv1x1_max_pool_pad: %d rows are not whole sibling groups of %d parents", h, top_h);
  if (top_h == 0) return OCNN_OK;
  const int s = conv_pointwise_pool_bf16(x, w, top, child_parent, h, top_h, cin, cout, ep, group_parent,
                                         static_cast<cudaStream_t>(stream), dtype == OCNN_F16);
  if (s >= 0) return s;
  return fail(OCNN_ERR_UNSUPPORTED,
              "ocnn_octree_conv1x1_max_pool_pad: %d -> %d channels (8, 16, 32 or 64 each, not 64 -> 64; "
              "16-byte aligned data)", cin, cout);
}

extern "C" int ocnn_octree_conv1x1_chain(const void* x, const float* w1, void* y1,
                                         const ocnn_conv_epilogue* ep1, const float* w2, void* y2,
                                         const ocnn_conv_epilogue* ep2, int h, int cin, int cmid,
                                         int cout2, int dtype, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(x && w1 && y1 && w2 && y2, "ocnn_octree_conv1x1_chain: null pointer");
  OCNN_REQUIRE(dtype == OCNN_BF16 || dtype == OCNN_F16, "ocnn_octree_conv1x1_chain: bf16 or fp16 node-major data");
  OCNN_REQUIRE(h >= 0, "ocnn_octree_conv1x1_chain: negative height");
  OCNN_REQUIRE(!(ep2 && ep2->residual_dev), "ocnn_octree_conv1x1_chain: no residual on the second layer");
  if (h == 0) return OCNN_OK;
  const int s = conv_pointwise_chain_bf16(x, w1, y1, h, cin, cmid, ep1, w2, y2, cout2, ep2,
                                          static_cast<cudaStream_t>(stream), dtype == OCNN_F16);
  if (s >= 0) return s;
  return fail(OCNN_ERR_UNSUPPORTED, "ocnn_octree_conv1x1_chain: %d -> %d -> %d channels is not one of "
              "8-32-8, 16-64-16, 16-32-8, 8-16-8 (16-byte aligned data)", cin, cmid, cout2);
}

extern "C" int ocnn_octree_ichild(const int32_t* child, int nnum, int32_t* ichild, void* stream) {
  using namespace ocnn;
  if (nnum == 0) return OCNN_OK;
  OCNN_REQUIRE(child && ichild && nnum > 0, "ocnn_octree_ichild: null pointer or negative size");
  ichild_kernel<<<grid_for(nnum, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(child, ichild, nnum);
  OCNN_LAUNCH_OK("ichild_kernel");
  return OCNN_OK;
}

extern "C" int ocnn_octree_conv_nempty(const void* x, const float* w, void* y, const int32_t* neigh,
                                       const int32_t* child, const int32_t* ichild, int nne, int cin,
                                       int cout, const int kernel_size[3], int dtype, int layout,
                                       const ocnn_conv_epilogue* ep, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(kernel_size != nullptr, "ocnn_octree_conv_nempty: null kernel size");
  const TapList tl = taps_for_kernel(kernel_size);
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "ocnn_octree_conv_nempty: unsupported kernel size %dx%dx%d",
                kernel_size[0], kernel_size[1], kernel_size[2]);
  OCNN_REQUIRE(cin > 0 && cout > 0, "ocnn_octree_conv_nempty: channel counts must be positive");
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16,
               "ocnn_octree_conv_nempty: unknown dtype %d", dtype);
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR,
               "ocnn_octree_conv_nempty: unknown layout %d", layout);
  OCNN_REQUIRE(nne >= 0, "ocnn_octree_conv_nempty: negative height");
  if (nne == 0) return OCNN_OK;
  OCNN_REQUIRE(x && w && y, "ocnn_octree_conv_nempty: null data pointer");
  if (tl.count == 1)      // 1x1x1: no neighbours, the same product as on all nodes
    return ocnn_octree_conv(x, w, y, nullptr, nne, nne, cin, cout, kernel_size, 1, dtype, layout, ep, stream);
  OCNN_REQUIRE(neigh && child && ichild, "ocnn_octree_conv_nempty: neighbour table, child and ichild required");
  return conv_simt_launch(x, w, y, neigh, child, ichild, nne, nne, cin, cout, tl, 1, dtype, layout, ep,
                          stream);
}

// Height rules shared by the CUDA-core and the tensor-core route of the general entry points.
namespace ocnn {
int check_conv_geometry(const ocnn_conv_geometry* g, const TapList& tl, const char* who) {
  OCNN_REQUIRE(g != nullptr, "%s: null geometry", who);
  OCNN_REQUIRE(g->stride == 1 || g->stride == 2, "%s: stride must be 1 or 2 (got %d)", who, g->stride);
  OCNN_REQUIRE(g->h_in >= 0 && g->h_out >= 0, "%s: negative height", who);
  const bool identity = tl.count == 1 && g->stride == 1;
  OCNN_REQUIRE(identity || g->neigh_dev != nullptr, "%s: neighbour table required", who);
  if (g->nempty && !identity) {
    const bool need_child = !(g->transposed && g->stride == 2);
    const bool need_ichild = !(g->stride == 2 && !g->transposed);
    OCNN_REQUIRE(!need_child || g->child_dev != nullptr, "%s: child array required (nempty)", who);
    OCNN_REQUIRE(!need_ichild || g->ichild_dev != nullptr, "%s: ichild array required (nempty)", who);
  }
  if (g->stride == 1) {
    OCNN_REQUIRE(g->h_in == g->h_out, "%s: stride 1 needs h_in == h_out (got %d, %d)", who, g->h_in,
                 g->h_out);
  } else if (!g->transposed) {
    if (!g->nempty)
      OCNN_REQUIRE((long long)g->h_out * 8 == g->h_in, "%s: stride 2 needs h_in == 8*h_out (got %d, %d)",
                   who, g->h_in, g->h_out);
  } else {
    if (!g->nempty)
      OCNN_REQUIRE((long long)g->h_in * 8 == g->h_out,
                   "%s: a stride-2 deconvolution needs h_out == 8*h_in (got %d, %d)", who, g->h_in,
                   g->h_out);
    else
      OCNN_REQUIRE((long long)g->h_in * 8 >= g->h_out,
                   "%s: a stride-2 deconvolution on non-empty nodes needs h_out <= 8*h_in (got %d, %d)",
                   who, g->h_in, g->h_out);
  }
  return OCNN_OK;
}
}  // namespace ocnn

extern "C" int ocnn_octree_conv_general(const void* x, const float* w, void* y,
                                        const ocnn_conv_geometry* g, int cin, int cout,
                                        const int kernel_size[3], int dtype, int layout,
                                        const ocnn_conv_epilogue* ep, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(kernel_size != nullptr, "ocnn_octree_conv_general: null kernel size");
  const TapList tl = taps_for_kernel(kernel_size);
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "ocnn_octree_conv_general: unsupported kernel size %dx%dx%d",
                kernel_size[0], kernel_size[1], kernel_size[2]);
  OCNN_REQUIRE(cin > 0 && cout > 0, "ocnn_octree_conv_general: channel counts must be positive");
  OCNN_REQUIRE(dtype == OCNN_F32 || dtype == OCNN_BF16 || dtype == OCNN_F16,
               "ocnn_octree_conv_general: unknown dtype %d", dtype);
  OCNN_REQUIRE(layout == OCNN_CHANNEL_MAJOR || layout == OCNN_NODE_MAJOR,
               "ocnn_octree_conv_general: unknown layout %d", layout);
  if (int rc = check_conv_geometry(g, tl, "ocnn_octree_conv_general")) return rc;
  if (g->h_out == 0) return OCNN_OK;
  OCNN_REQUIRE(x && w && y, "ocnn_octree_conv_general: null data pointer");
  const bool identity = tl.count == 1 && g->stride == 1;
  const int32_t* child = (g->nempty && !identity && !(g->transposed && g->stride == 2)) ? g->child_dev : nullptr;
  const int32_t* ichild = (g->nempty && !identity && !(g->stride == 2 && !g->transposed)) ? g->ichild_dev : nullptr;
  return conv_simt_launch(x, w, y, identity ? nullptr : g->neigh_dev, child, ichild, g->h_in, g->h_out,
                          cin, cout, tl, g->stride, dtype, layout, ep, stream, g->transposed != 0);
}
