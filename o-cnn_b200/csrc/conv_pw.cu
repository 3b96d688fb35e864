// 1x1x1 octree convolution (a per-node matrix product) for node-major bf16 data with few
// channels: the pointwise layers of the reference's bottleneck blocks
// (pytorch/ocnn/modules.py:71-83, a torch Conv1d there).  With Cin, Cout <= 64 the arithmetic
// intensity is a few flops per byte, so the kernel is a pure HBM stream: every thread owns ROWS
// whole node rows (16-byte loads), keeps Cout fp32 accumulators per row in registers, reads the
// fp32 weights as shared-memory broadcasts, applies the fused epilogue and writes 16-byte pieces.
// Algorithmic bytes per node: (Cin + Cout [+ Cout residual]) * 2.
#include "common.cuh"

namespace ocnn {
namespace {

struct PwArgs {
  const __nv_bfloat16* x;
  const float* w;          // [cout, cin], the reference layout
  __nv_bfloat16* y;
  int h, cin;
  int y_stride;            // output channels of the whole layer (row stride of y / residual)
  int co_base;             // first output channel this launch produces
  const float* scale;
  const float* bias;
  const __nv_bfloat16* residual;
  int relu;
  int f16;                 // the 16-bit elements are fp16 instead of bf16
  int wide;                // x, y and the residual start on 32-byte boundaries
  // conv_pw_mma_pool_kernel: the layer's output is max-pooled over sibling groups (8 consecutive
  // rows) and the group's row written to row pool_inv[group] of y (OctreeMaxPool's pad: the parent
  // node of the group); the un-pooled output is not stored at all
  const int* pool_inv;
  // conv_pw_mma_kernel<.., C2 > 0>: a second 1x1x1 layer (the next block's conv1x1a) applied to the
  // rows this one has just produced, while they are still in registers: y2 = act(scale2 * (w2 * y)
  // + bias2), w2 fp32 [C2, COUT]
  const float* w2;
  const float* scale2;
  const float* bias2;
  __nv_bfloat16* y2;
  int relu2;
};

// CIN > 0: the channel count is a compile-time constant and a thread requests its whole rows
// (and the residual rows) before it starts on the arithmetic, 32 bytes per load where the row
// allows: with one 16-byte piece in flight per thread the kernel waited on memory latency (42 %
// of the HBM copy rate).  CIN == 0: any Cin % 8 == 0, one 16-byte piece at a time.
template <int CIN, int COUT, int ROWS, bool HALF>
__global__ void __launch_bounds__(256) conv_pw_kernel(const PwArgs a) {
  extern __shared__ float ws[];                      // [cin][COUT]
  grid_dependency_trigger();
  grid_dependency_wait();
  for (int i = threadIdx.x; i < a.cin * COUT; i += blockDim.x) {
    const int co = i / a.cin, ci = i % a.cin;        // coalesced read of w[co][ci], transposed store
    ws[ci * COUT + co] = a.w[(long long)a.co_base * a.cin + i];
  }
  __syncthreads();
  const long long stride = (long long)gridDim.x * blockDim.x;
  // thread t of the grid handles rows t, t + stride, ... in packets of ROWS rows spaced by the
  // grid size, so that a warp always touches 32 consecutive rows
  for (long long h0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; h0 < a.h; h0 += stride * ROWS) {
    float acc[ROWS][COUT];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
      for (int co = 0; co < COUT; ++co) acc[r][co] = 0.f;
    constexpr int kResPieces = COUT / 8;
    uint4 rres[ROWS][kResPieces];
    auto load_residual = [&]() {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const long long h = h0 + r * stride;
#pragma unroll
        for (int q = 0; q < kResPieces; ++q) rres[r][q] = make_uint4(0, 0, 0, 0);
        if (a.residual == nullptr || h >= a.h) continue;
        const __nv_bfloat16* rp = a.residual + h * a.y_stride + a.co_base;
        if constexpr (COUT % 16 == 0) {
          if (a.wide) {
#pragma unroll
            for (int q = 0; q < kResPieces; q += 2) ld_global_32B(rp + 8 * q, rres[r][q], rres[r][q + 1]);
            continue;
          }
        }
#pragma unroll
        for (int q = 0; q < kResPieces; ++q) rres[r][q] = *reinterpret_cast<const uint4*>(rp + 8 * q);
      }
    };
    auto fma_piece = [&](const uint4 (&raw)[ROWS], int c8) {
      float xv[ROWS][8];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(&raw[r]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack2(p[k], HALF);
          xv[r][2 * k] = f.x;
          xv[r][2 * k + 1] = f.y;
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4* wrow = reinterpret_cast<const float4*>(ws + (c8 * 8 + k) * COUT);
#pragma unroll
        for (int q = 0; q < COUT / 4; ++q) {
          const float4 wv = wrow[q];
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            acc[r][4 * q + 0] = fmaf(xv[r][k], wv.x, acc[r][4 * q + 0]);
            acc[r][4 * q + 1] = fmaf(xv[r][k], wv.y, acc[r][4 * q + 1]);
            acc[r][4 * q + 2] = fmaf(xv[r][k], wv.z, acc[r][4 * q + 2]);
            acc[r][4 * q + 3] = fmaf(xv[r][k], wv.w, acc[r][4 * q + 3]);
          }
        }
      }
    };
    if constexpr (CIN > 0) {
      constexpr int kPieces = CIN / 8;
      uint4 xr[kPieces][ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const long long h = h0 + r * stride;
#pragma unroll
        for (int c8 = 0; c8 < kPieces; ++c8) xr[c8][r] = make_uint4(0, 0, 0, 0);
        if (h >= a.h) continue;
        const __nv_bfloat16* xp = a.x + h * CIN;
        if constexpr (CIN % 16 == 0) {
          if (a.wide) {
#pragma unroll
            for (int c8 = 0; c8 < kPieces; c8 += 2) ld_global_32B(xp + 8 * c8, xr[c8][r], xr[c8 + 1][r]);
            continue;
          }
        }
#pragma unroll
        for (int c8 = 0; c8 < kPieces; ++c8) xr[c8][r] = reinterpret_cast<const uint4*>(xp)[c8];
      }
      load_residual();
#pragma unroll
      for (int c8 = 0; c8 < kPieces; ++c8) fma_piece(xr[c8], c8);
    } else {
      load_residual();
      const int chunks = a.cin >> 3;
      for (int c8 = 0; c8 < chunks; ++c8) {
        uint4 raw[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const long long h = h0 + r * stride;
          raw[r] = make_uint4(0, 0, 0, 0);
          if (h < a.h) raw[r] = reinterpret_cast<const uint4*>(a.x + h * a.cin)[c8];
        }
        fma_piece(raw, c8);
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const long long h = h0 + r * stride;
      if (h >= a.h) continue;
      uint4 ov[kResPieces];
#pragma unroll
      for (int q = 0; q < COUT / 8; ++q) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          f[j] = acc[r][8 * q + j];
          if (a.scale) f[j] *= a.scale[a.co_base + 8 * q + j];
          if (a.bias) f[j] += a.bias[a.co_base + 8 * q + j];
        }
        if (a.residual) {
          const uint32_t* rp = reinterpret_cast<const uint32_t*>(&rres[r][q]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 rf = unpack2(rp[j], HALF);
            f[2 * j] += rf.x;
            f[2 * j + 1] += rf.y;
          }
        }
        if (a.relu) {
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
        }
        uint32_t* op = reinterpret_cast<uint32_t*>(&ov[q]);
#pragma unroll
        for (int j = 0; j < 4; ++j) op[j] = pack2(f[2 * j], f[2 * j + 1], HALF);
      }
      __nv_bfloat16* yp = a.y + h * a.y_stride + a.co_base;
      if constexpr (COUT % 16 == 0) {
        if (a.wide) {
#pragma unroll
          for (int q = 0; q < kResPieces; q += 2) st_global_32B(yp + 8 * q, ov[q], ov[q + 1]);
          continue;
        }
      }
#pragma unroll
      for (int q = 0; q < kResPieces; ++q) *reinterpret_cast<uint4*>(yp + 8 * q) = ov[q];
    }
  }
}

template <int CIN, int COUT, int ROWS, bool HALF>
int launch_pw_t(const PwArgs& a, cudaStream_t st) {
  const size_t smem = (size_t)a.cin * COUT * sizeof(float);
  static PerDeviceOnce attr_once;      // one per template instance
  int device = 0;
  OCNN_CUDA_OK(cudaGetDevice(&device));
  if (smem > 48 * 1024) {
    std::lock_guard<std::mutex> lock(attr_once.mutex);
    const bool known = device >= 0 && device < 64;
    if (!known || !attr_once.done[device]) {
      OCNN_CUDA_OK(cudaFuncSetAttribute(conv_pw_kernel<CIN, COUT, ROWS, HALF>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
      if (known) attr_once.done[device] = true;
    }
  }
  const int grid = grid_for(((long long)a.h + ROWS - 1) / ROWS, 256, 4);
  OCNN_CUDA_OK(launch_chained(conv_pw_kernel<CIN, COUT, ROWS, HALF>, dim3(grid), dim3(256), smem, st, a));
  OCNN_LAUNCH_OK("conv_pw_kernel");
  return OCNN_OK;
}

template <int COUT, int ROWS>
int launch_pw(const PwArgs& a, cudaStream_t st) {
  // the channel counts of the reference's bottleneck blocks get the whole-row variant
  switch (a.cin) {
    case 8:
      return a.f16 ? launch_pw_t<8, COUT, ROWS, true>(a, st) : launch_pw_t<8, COUT, ROWS, false>(a, st);
    case 16:
      return a.f16 ? launch_pw_t<16, COUT, ROWS, true>(a, st) : launch_pw_t<16, COUT, ROWS, false>(a, st);
    case 32:
      return a.f16 ? launch_pw_t<32, COUT, ROWS, true>(a, st) : launch_pw_t<32, COUT, ROWS, false>(a, st);
    default:
      return a.f16 ? launch_pw_t<0, COUT, ROWS, true>(a, st) : launch_pw_t<0, COUT, ROWS, false>(a, st);
  }
}

// ---- the same layer on warp-level tensor-core instructions ------------------------------------
// With 8..64 channels the CUDA-core kernel above is bound by instruction issue (Cin*Cout FMAs and
// Cin*Cout/4 shared-memory reads per node), not by memory.  Here a warp owns 16 consecutive node
// rows at a time and multiplies them with mma.sync (m16n8k16, or m16n8k8 for 8 input channels;
// bf16 or fp16 operands, fp32 accumulation): the A fragments come straight from the node-major
// rows (consecutive rows are consecutive memory), the weights live in registers for the whole
// launch as a (hi, lo) pair of 16-bit values per element, so the product is that of the fp32
// weights to about 2^-17, and output and shortcut are accessed from the accumulator fragments.
// What is left per node is the memory traffic.
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                          bool half) {
  if (half)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, bool half) {
  if (half)
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
  else
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

// (hi, lo) 16-bit split of two fp32 weights, packed as the low / high half of a register each
__device__ __forceinline__ void split2(float w0, float w1, bool half, uint32_t& hi, uint32_t& lo) {
  hi = pack2(w0, w1, half);
  const float2 h = unpack2(hi, half);
  lo = pack2(w0 - h.x, w1 - h.y, half);
}

// W consecutive 32-bit words, as the widest accesses their count allows (W = 1, 2, 4, 8)
template <int W>
__device__ __forceinline__ void load_words(const uint32_t* p, uint32_t (&v)[W]) {
  if constexpr (W == 1) {
    v[0] = *p;
  } else if constexpr (W == 2) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = t.x; v[1] = t.y;
  } else {
#pragma unroll
    for (int i = 0; i < W; i += 4) {
      const uint4 t = *reinterpret_cast<const uint4*>(p + i);
      v[i] = t.x; v[i + 1] = t.y; v[i + 2] = t.z; v[i + 3] = t.w;
    }
  }
}
template <int W>
__device__ __forceinline__ void store_words(uint32_t* p, const uint32_t (&v)[W]) {
  if constexpr (W == 1) {
    *p = v[0];
  } else if constexpr (W == 2) {
    *reinterpret_cast<uint2*>(p) = make_uint2(v[0], v[1]);
  } else {
#pragma unroll
    for (int i = 0; i < W; i += 4)
      *reinterpret_cast<uint4*>(p + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  }
}

// Which channel an MMA operand element stands for is free as long as A and B agree on k and B and
// D agree on n.  Here lane q of a quad owns a CONTIGUOUS quarter of the node's input row and of
// its output row: logical k = 2q + {0, 1} (+ 8) of slice s is input channel q*CIN/4 + 4s + {0, 1}
// (+ 2), logical column 2q + e of accumulator tile j is output channel q*COUT/4 + 2j + e.  A
// lane then reads its CIN/4 input channels and writes its COUT/4 output channels (and reads the
// shortcut's) of a row as one vector each, and a warp instruction covers 8 whole consecutive rows.
template <int CIN, int COUT, bool HALF, int C2 = 0>
__global__ void __launch_bounds__(256) conv_pw_mma_kernel(const PwArgs a) {
  static_assert(C2 == 0 || (COUT % 16 == 0 && C2 % 8 == 0), "second layer: whole K slices");
  constexpr int KS2 = C2 > 0 ? COUT / 16 : 1, NT2 = C2 > 0 ? C2 / 8 : 1;   // second layer's slices, tiles
  constexpr int CQ2 = C2 > 0 ? C2 / 4 : 2, YW2 = CQ2 / 2;
  constexpr int PAIRS2 = C2 > 0 ? C2 * COUT / 2 : 1;
  __shared__ uint32_t s2_hi[PAIRS2], s2_lo[PAIRS2];
  constexpr int KS = CIN >= 16 ? CIN / 16 : 1;     // 16-wide (8-wide for CIN = 8) K slices
  constexpr int NT = COUT / 8;                      // 8-column accumulator tiles
  constexpr int BR = CIN >= 16 ? 2 : 1;             // B registers per (slice, tile)
  constexpr int KQ = CIN / 4, CQ = COUT / 4;        // channels per lane of a row: input, output
  constexpr int XW = KQ / 2, YW = CQ / 2;           // ... in 32-bit words (YW == NT)
  constexpr int PAIRS = COUT * CIN / 2;             // weight pairs (w[co][2p], w[co][2p + 1])
  // the (hi, lo) split of the layer's weights, made once per CTA
  __shared__ uint32_t s_hi[PAIRS], s_lo[PAIRS];
  grid_dependency_trigger();
  grid_dependency_wait();
  for (int p = threadIdx.x; p < PAIRS; p += blockDim.x) {
    const float2 w2 = *reinterpret_cast<const float2*>(a.w + 2 * p);
    split2(w2.x, w2.y, HALF, s_hi[p], s_lo[p]);
  }
  if constexpr (C2 > 0) {
    for (int p = threadIdx.x; p < PAIRS2; p += blockDim.x) {
      const float2 w2 = *reinterpret_cast<const float2*>(a.w2 + 2 * p);
      split2(w2.x, w2.y, HALF, s2_hi[p], s2_lo[p]);
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  // this lane's elements of every (slice, tile): column g of tile j, rows 2q + {0, 1} (+ 8)
  uint32_t bh[KS][NT][BR], bl[KS][NT][BR];
#pragma unroll
  for (int s = 0; s < KS; ++s)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int r = 0; r < BR; ++r) {
        const int co = (g >> 1) * CQ + 2 * j + (g & 1);
        const int ci = q * KQ + (CIN >= 16 ? 4 * s + 2 * r : 0);
        const int p = (co * CIN + ci) >> 1;
        bh[s][j][r] = s_hi[p];
        bl[s][j][r] = s_lo[p];
      }
  float sc[NT][2], bi[NT][2];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      sc[j][e] = a.scale ? a.scale[q * CQ + 2 * j + e] : 1.f;
      bi[j][e] = a.bias ? a.bias[q * CQ + 2 * j + e] : 0.f;
    }
  // The second layer's A operand is this layer's packed output: the pair (2q, 2q + 1) of
  // accumulator tile 2s is K pair 2q of slice s, that of tile 2s + 1 is K pair 2q + 8, i.e. logical
  // k of (slice s, register r) is output channel q*CQ + 2*(2s + r) + {0, 1}; its B fragments and
  // its own output follow the same lane-contiguous scheme.
  uint32_t b2h[KS2][NT2][2], b2l[KS2][NT2][2];
  float sc2[NT2][2], bi2[NT2][2];
  if constexpr (C2 > 0) {
#pragma unroll
    for (int s = 0; s < KS2; ++s)
#pragma unroll
      for (int j = 0; j < NT2; ++j)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int co = (g >> 1) * CQ2 + 2 * j + (g & 1);
          const int ci = q * CQ + 2 * (2 * s + r);
          const int p = (co * COUT + ci) >> 1;
          b2h[s][j][r] = s2_hi[p];
          b2l[s][j][r] = s2_lo[p];
        }
#pragma unroll
    for (int j = 0; j < NT2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sc2[j][e] = a.scale2 ? a.scale2[q * CQ2 + 2 * j + e] : 1.f;
        bi2[j][e] = a.bias2 ? a.bias2[q * CQ2 + 2 * j + e] : 0.f;
      }
  }
  const long long tiles = ((long long)a.h + 15) >> 4;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const uint32_t* x32 = reinterpret_cast<const uint32_t*>(a.x) + q * XW;
  const uint32_t* r32 = a.residual ? reinterpret_cast<const uint32_t*>(a.residual) + q * YW : nullptr;
  uint32_t* y32 = reinterpret_cast<uint32_t*>(a.y) + q * YW;
  // this lane's quarter of rows 16*tile + g and + 8, and of the shortcut's: the next tile's are
  // requested before the current one is multiplied
  uint32_t xa[XW], xb[XW], ra[YW], rb[YW];
  auto load_tile = [&](long long tile, uint32_t (&pa)[XW], uint32_t (&pb)[XW], uint32_t (&qa)[YW],
                       uint32_t (&qb)[YW]) {
    const long long r0 = (tile << 4) + g, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < XW; ++i) pa[i] = pb[i] = 0u;
#pragma unroll
    for (int i = 0; i < YW; ++i) qa[i] = qb[i] = 0u;
    if (tile >= tiles) return;
    if (r0 < a.h) load_words<XW>(x32 + r0 * (CIN / 2), pa);
    if (r1 < a.h) load_words<XW>(x32 + r1 * (CIN / 2), pb);
    if (r32 && r0 < a.h) load_words<YW>(r32 + r0 * (COUT / 2), qa);
    if (r32 && r1 < a.h) load_words<YW>(r32 + r1 * (COUT / 2), qb);
  };
  load_tile(warp0, xa, xb, ra, rb);
  for (long long tile = warp0; tile < tiles; tile += nwarps) {
    const long long r0 = (tile << 4) + g, r1 = r0 + 8;
    const bool ok0 = r0 < a.h, ok1 = r1 < a.h;
    uint32_t nxa[XW], nxb[XW], nra[YW], nrb[YW];
    load_tile(tile + nwarps, nxa, nxb, nra, nrb);
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        if constexpr (CIN >= 16) {
          const uint32_t af[4] = {xa[2 * s], xb[2 * s], xa[2 * s + 1], xb[2 * s + 1]};
          mma_16816(acc[j], af, bl[s][j][0], bl[s][j][BR - 1], HALF);
          mma_16816(acc[j], af, bh[s][j][0], bh[s][j][BR - 1], HALF);
        } else {
          mma_1688(acc[j], xa[0], xb[0], bl[s][j][0], HALF);
          mma_1688(acc[j], xa[0], xb[0], bh[s][j][0], HALF);
        }
      }
    }
    uint32_t oa[YW], ob[YW];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float v0 = fmaf(acc[j][0], sc[j][0], bi[j][0]), v1 = fmaf(acc[j][1], sc[j][1], bi[j][1]);
      float v2 = fmaf(acc[j][2], sc[j][0], bi[j][0]), v3 = fmaf(acc[j][3], sc[j][1], bi[j][1]);
      if (r32) {
        const float2 fa = unpack2(ra[j], HALF), fb = unpack2(rb[j], HALF);
        v0 += fa.x; v1 += fa.y; v2 += fb.x; v3 += fb.y;
      }
      if (a.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); v2 = fmaxf(v2, 0.f); v3 = fmaxf(v3, 0.f); }
      oa[j] = pack2(v0, v1, HALF);
      ob[j] = pack2(v2, v3, HALF);
    }
    if (ok0) store_words<YW>(y32 + r0 * (COUT / 2), oa);
    if (ok1) store_words<YW>(y32 + r1 * (COUT / 2), ob);
    if constexpr (C2 > 0) {
      uint32_t* y2 = reinterpret_cast<uint32_t*>(a.y2) + q * YW2;
      uint32_t pa[YW2], pb[YW2];
#pragma unroll
      for (int j = 0; j < NT2; ++j) {
        float c2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < KS2; ++s) {
          const uint32_t af[4] = {oa[2 * s], ob[2 * s], oa[2 * s + 1], ob[2 * s + 1]};
          mma_16816(c2, af, b2l[s][j][0], b2l[s][j][1], HALF);
          mma_16816(c2, af, b2h[s][j][0], b2h[s][j][1], HALF);
        }
        float u0 = fmaf(c2[0], sc2[j][0], bi2[j][0]), u1 = fmaf(c2[1], sc2[j][1], bi2[j][1]);
        float u2 = fmaf(c2[2], sc2[j][0], bi2[j][0]), u3 = fmaf(c2[3], sc2[j][1], bi2[j][1]);
        if (a.relu2) { u0 = fmaxf(u0, 0.f); u1 = fmaxf(u1, 0.f); u2 = fmaxf(u2, 0.f); u3 = fmaxf(u3, 0.f); }
        pa[j] = pack2(u0, u1, HALF);
        pb[j] = pack2(u2, u3, HALF);
      }
      if (ok0) store_words<YW2>(y2 + r0 * (C2 / 2), pa);
      if (ok1) store_words<YW2>(y2 + r1 * (C2 / 2), pb);
    }
#pragma unroll
    for (int i = 0; i < XW; ++i) { xa[i] = nxa[i]; xb[i] = nxb[i]; }
#pragma unroll
    for (int i = 0; i < YW; ++i) { ra[i] = nra[i]; rb[i] = nrb[i]; }
  }
}

// The two-input layer (a residual block's conv1x1b + shortcut conv1x1c over [xa | xb]) on the same
// scheme: K slices first over xa's channels, then over xb's, lane q owning a contiguous quarter of
// each input row.  The weights are the 16-bit values of the tensor-core kernel's packed image
// (element (k, n) of K-block kb sits at kb*npad*64 + (n>>3)*512 + (n&7)*64 + (((kk>>3)^(n&7))<<3)
// + (kk&7), kk = k - 64*kb), so both kernels multiply the same numbers.
struct PwPairArgs {
  const __nv_bfloat16* xa;
  const __nv_bfloat16* xb;
  const uint16_t* packed;
  __nv_bfloat16* y;
  int h, npad;
  const float* scale;
  const float* bias;
  const __nv_bfloat16* residual;
  int relu;
};

template <int CA, int CB, int COUT, bool HALF>
__global__ void __launch_bounds__(256) conv_pw_pair_kernel(const PwPairArgs a) {
  constexpr int KA = CA / 16, KB = CB / 16, KS = KA + KB;
  constexpr int NT = COUT / 8;
  constexpr int AQ = CA / 4, BQ = CB / 4, CQ = COUT / 4;      // channels per lane of a row
  constexpr int AW = AQ / 2, BW = BQ / 2, YW = CQ / 2;        // ... in 32-bit words
  constexpr int CIN = CA + CB;
  __shared__ uint32_t s_w[COUT * CIN / 2];                    // [co][k pair], 16-bit values as packed
  grid_dependency_trigger();
  grid_dependency_wait();
  for (int p = threadIdx.x; p < COUT * CIN / 2; p += blockDim.x) {
    const int n = p / (CIN / 2), k = 2 * (p % (CIN / 2));
    const int kb = k >> 6, kk = k & 63;
    const long long off = (long long)kb * a.npad * 64 + (n >> 3) * 512 + (n & 7) * 64 +
                          (((kk >> 3) ^ (n & 7)) << 3) + (kk & 7);
    s_w[p] = *reinterpret_cast<const uint32_t*>(a.packed + off);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  uint32_t bw[KS][NT][2];
#pragma unroll
  for (int s = 0; s < KS; ++s)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int co = (g >> 1) * CQ + 2 * j + (g & 1);
        const int ci = s < KA ? q * AQ + 4 * s + 2 * r : CA + q * BQ + 4 * (s - KA) + 2 * r;
        bw[s][j][r] = s_w[(co * CIN + ci) >> 1];
      }
  float sc[NT][2], bi[NT][2];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      sc[j][e] = a.scale ? a.scale[q * CQ + 2 * j + e] : 1.f;
      bi[j][e] = a.bias ? a.bias[q * CQ + 2 * j + e] : 0.f;
    }
  const long long tiles = ((long long)a.h + 15) >> 4;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const uint32_t* xa32 = reinterpret_cast<const uint32_t*>(a.xa) + q * AW;
  const uint32_t* xb32 = reinterpret_cast<const uint32_t*>(a.xb) + q * BW;
  const uint32_t* r32 = a.residual ? reinterpret_cast<const uint32_t*>(a.residual) + q * YW : nullptr;
  uint32_t* y32 = reinterpret_cast<uint32_t*>(a.y) + q * YW;
  // rows 16*tile + g (0) and + 8 (1) of both inputs and of the residual
  uint32_t a0[AW], a1[AW], b0[BW], b1[BW], ra[YW], rb[YW];
  auto load_tile = [&](long long tile, uint32_t (&pa0)[AW], uint32_t (&pa1)[AW], uint32_t (&pb0)[BW],
                       uint32_t (&pb1)[BW], uint32_t (&qa)[YW], uint32_t (&qb)[YW]) {
    const long long r0 = (tile << 4) + g, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < AW; ++i) pa0[i] = pa1[i] = 0u;
#pragma unroll
    for (int i = 0; i < BW; ++i) pb0[i] = pb1[i] = 0u;
#pragma unroll
    for (int i = 0; i < YW; ++i) qa[i] = qb[i] = 0u;
    if (tile >= tiles) return;
    if (r0 < a.h) {
      load_words<AW>(xa32 + r0 * (CA / 2), pa0);
      load_words<BW>(xb32 + r0 * (CB / 2), pb0);
      if (r32) load_words<YW>(r32 + r0 * (COUT / 2), qa);
    }
    if (r1 < a.h) {
      load_words<AW>(xa32 + r1 * (CA / 2), pa1);
      load_words<BW>(xb32 + r1 * (CB / 2), pb1);
      if (r32) load_words<YW>(r32 + r1 * (COUT / 2), qb);
    }
  };
  load_tile(warp0, a0, a1, b0, b1, ra, rb);
  for (long long tile = warp0; tile < tiles; tile += nwarps) {
    const long long r0 = (tile << 4) + g, r1 = r0 + 8;
    uint32_t na0[AW], na1[AW], nb0[BW], nb1[BW], nra[YW], nrb[YW];
    load_tile(tile + nwarps, na0, na1, nb0, nb1, nra, nrb);
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        uint32_t af[4];
        if (s < KA) {
          af[0] = a0[2 * s]; af[1] = a1[2 * s]; af[2] = a0[2 * s + 1]; af[3] = a1[2 * s + 1];
        } else {
          af[0] = b0[2 * (s - KA)]; af[1] = b1[2 * (s - KA)];
          af[2] = b0[2 * (s - KA) + 1]; af[3] = b1[2 * (s - KA) + 1];
        }
        mma_16816(acc[j], af, bw[s][j][0], bw[s][j][1], HALF);
      }
    }
    uint32_t oa[YW], ob[YW];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float v0 = fmaf(acc[j][0], sc[j][0], bi[j][0]), v1 = fmaf(acc[j][1], sc[j][1], bi[j][1]);
      float v2 = fmaf(acc[j][2], sc[j][0], bi[j][0]), v3 = fmaf(acc[j][3], sc[j][1], bi[j][1]);
      if (r32) {
        const float2 fa = unpack2(ra[j], HALF), fb = unpack2(rb[j], HALF);
        v0 += fa.x; v1 += fa.y; v2 += fb.x; v3 += fb.y;
      }
      if (a.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); v2 = fmaxf(v2, 0.f); v3 = fmaxf(v3, 0.f); }
      oa[j] = pack2(v0, v1, HALF);
      ob[j] = pack2(v2, v3, HALF);
    }
    if (r0 < a.h) store_words<YW>(y32 + r0 * (COUT / 2), oa);
    if (r1 < a.h) store_words<YW>(y32 + r1 * (COUT / 2), ob);
#pragma unroll
    for (int i = 0; i < AW; ++i) { a0[i] = na0[i]; a1[i] = na1[i]; }
#pragma unroll
    for (int i = 0; i < BW; ++i) { b0[i] = nb0[i]; b1[i] = nb1[i]; }
#pragma unroll
    for (int i = 0; i < YW; ++i) { ra[i] = nra[i]; rb[i] = nrb[i]; }
  }
}

// The pooled form without any exchange between lanes.  Which NODE an MMA row stands for is free
// too: a warp takes 16 sibling groups at a time and runs eight MMA passes over them, pass t on
// sibling t of every group (row g of the pass = node 8*(G0 + g) + t, row g + 8 = node
// 8*(G0 + g + 8) + t).  A lane then sees all eight siblings of its two groups one after the other
// and keeps a running maximum of its accumulator values; after the eighth pass it writes its
// quarter of the two pooled rows.  The next sibling's rows are requested before the current
// ones are multiplied.
template <int CIN, int COUT, bool HALF>
__global__ void __launch_bounds__(256) conv_pw_mma_pool_kernel(const PwArgs a) {
  constexpr int KS = CIN >= 16 ? CIN / 16 : 1;
  constexpr int NT = COUT / 8;
  constexpr int BR = CIN >= 16 ? 2 : 1;
  constexpr int KQ = CIN / 4, CQ = COUT / 4;
  constexpr int XW = KQ / 2, YW = CQ / 2;
  constexpr int PAIRS = COUT * CIN / 2;
  __shared__ uint32_t s_hi[PAIRS], s_lo[PAIRS];
  grid_dependency_trigger();
  grid_dependency_wait();
  for (int p = threadIdx.x; p < PAIRS; p += blockDim.x) {
    const float2 w2 = *reinterpret_cast<const float2*>(a.w + 2 * p);
    split2(w2.x, w2.y, HALF, s_hi[p], s_lo[p]);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  uint32_t bh[KS][NT][BR], bl[KS][NT][BR];
#pragma unroll
  for (int s = 0; s < KS; ++s)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int r = 0; r < BR; ++r) {
        const int co = (g >> 1) * CQ + 2 * j + (g & 1);
        const int ci = q * KQ + (CIN >= 16 ? 4 * s + 2 * r : 0);
        const int p = (co * CIN + ci) >> 1;
        bh[s][j][r] = s_hi[p];
        bl[s][j][r] = s_lo[p];
      }
  float sc[NT][2], bi[NT][2];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      sc[j][e] = a.scale ? a.scale[q * CQ + 2 * j + e] : 1.f;
      bi[j][e] = a.bias ? a.bias[q * CQ + 2 * j + e] : 0.f;
    }
  const long long groups = (long long)a.h >> 3;
  const long long supers = (groups + 15) >> 4;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const uint32_t* x32 = reinterpret_cast<const uint32_t*>(a.x) + q * XW;
  const uint32_t* r32 = a.residual ? reinterpret_cast<const uint32_t*>(a.residual) + q * YW : nullptr;
  uint32_t* y32 = reinterpret_cast<uint32_t*>(a.y) + q * YW;
  for (long long sup = warp0; sup < supers; sup += nwarps) {
    const long long ga = (sup << 4) + g, gb = ga + 8;          // this lane's two groups
    const bool oka = ga < groups, okb = gb < groups;
    auto load_pass = [&](int t, uint32_t (&pa)[XW], uint32_t (&pb)[XW], uint32_t (&qa)[YW],
                         uint32_t (&qb)[YW]) {
#pragma unroll
      for (int i = 0; i < XW; ++i) pa[i] = pb[i] = 0u;
#pragma unroll
      for (int i = 0; i < YW; ++i) qa[i] = qb[i] = 0u;
      if (t >= 8) return;
      const long long ra = (ga << 3) + t, rb = (gb << 3) + t;
      if (oka) load_words<XW>(x32 + ra * (CIN / 2), pa);
      if (okb) load_words<XW>(x32 + rb * (CIN / 2), pb);
      if (r32 && oka) load_words<YW>(r32 + ra * (COUT / 2), qa);
      if (r32 && okb) load_words<YW>(r32 + rb * (COUT / 2), qb);
    };
    uint32_t xa[XW], xb[XW], ra_[YW], rb_[YW];
    load_pass(0, xa, xb, ra_, rb_);
    float m[NT][4];
#pragma unroll(NT >= 8 ? 1 : 8)
    for (int t = 0; t < 8; ++t) {
      uint32_t nxa[XW], nxb[XW], nra[YW], nrb[YW];
      load_pass(t + 1, nxa, nxb, nra, nrb);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < KS; ++s) {
          if constexpr (CIN >= 16) {
            const uint32_t af[4] = {xa[2 * s], xb[2 * s], xa[2 * s + 1], xb[2 * s + 1]};
            mma_16816(acc, af, bl[s][j][0], bl[s][j][BR - 1], HALF);
            mma_16816(acc, af, bh[s][j][0], bh[s][j][BR - 1], HALF);
          } else {
            mma_1688(acc, xa[0], xb[0], bl[s][j][0], HALF);
            mma_1688(acc, xa[0], xb[0], bh[s][j][0], HALF);
          }
        }
        float v0 = fmaf(acc[0], sc[j][0], bi[j][0]), v1 = fmaf(acc[1], sc[j][1], bi[j][1]);
        float v2 = fmaf(acc[2], sc[j][0], bi[j][0]), v3 = fmaf(acc[3], sc[j][1], bi[j][1]);
        if (r32) {
          const float2 fa = unpack2(ra_[j], HALF), fb = unpack2(rb_[j], HALF);
          v0 += fa.x; v1 += fa.y; v2 += fb.x; v3 += fb.y;
        }
        if (a.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); v2 = fmaxf(v2, 0.f); v3 = fmaxf(v3, 0.f); }
        if (t == 0) {
          m[j][0] = v0; m[j][1] = v1; m[j][2] = v2; m[j][3] = v3;
        } else {                       // fmaxf drops a NaN operand, like the pool kernel
          m[j][0] = fmaxf(m[j][0], v0); m[j][1] = fmaxf(m[j][1], v1);
          m[j][2] = fmaxf(m[j][2], v2); m[j][3] = fmaxf(m[j][3], v3);
        }
      }
#pragma unroll
      for (int i = 0; i < XW; ++i) { xa[i] = nxa[i]; xb[i] = nxb[i]; }
#pragma unroll
      for (int i = 0; i < YW; ++i) { ra_[i] = nra[i]; rb_[i] = nrb[i]; }
    }
    uint32_t oa[YW], ob[YW];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      oa[j] = pack2(m[j][0], m[j][1], HALF);
      ob[j] = pack2(m[j][2], m[j][3], HALF);
    }
    if (oka) store_words<YW>(y32 + (long long)a.pool_inv[ga] * (COUT / 2), oa);
    if (okb) store_words<YW>(y32 + (long long)a.pool_inv[gb] * (COUT / 2), ob);
  }
}

template <int CIN, int COUT>
int launch_pw_mma(const PwArgs& a, cudaStream_t st) {
  const long long warps = ((long long)a.h + 15) / 16;
  // about six 16-row tiles per warp (a warp's set-up -- its weight fragments, scale and bias -- is
  // then a small part of its life), up to eight CTAs per SM
  const long long want = (warps + 47) / 48;
  const long long cap = (long long)sm_count() * 8;
  const int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  if (a.pool_inv != nullptr) {
    // one pass over 16 sibling groups (eight MMA passes) per warp and iteration
    const long long supers = ((long long)a.h / 8 + 15) / 16;
    const long long pwant = (supers + 7) / 8;
    const int pgrid = (int)(pwant < 1 ? 1 : (pwant > cap ? cap : pwant));
    if (a.f16)
      OCNN_CUDA_OK(launch_chained(conv_pw_mma_pool_kernel<CIN, COUT, true>, dim3(pgrid), dim3(256), 0, st, a));
    else
      OCNN_CUDA_OK(launch_chained(conv_pw_mma_pool_kernel<CIN, COUT, false>, dim3(pgrid), dim3(256), 0, st, a));
  } else if (a.f16) {
    OCNN_CUDA_OK(launch_chained(conv_pw_mma_kernel<CIN, COUT, true>, dim3(grid), dim3(256), 0, st, a));
  } else {
    OCNN_CUDA_OK(launch_chained(conv_pw_mma_kernel<CIN, COUT, false>, dim3(grid), dim3(256), 0, st, a));
  }
  OCNN_LAUNCH_OK("conv_pw_mma_kernel");
  return OCNN_OK;
}

// Before the pooled layer: for every node p of the parent level, inv[child[p]] = p for a non-empty
// node (its sibling group's pooled row goes to row p), a zero row p for a leaf.  One thread per
// (node, 16-byte piece of the row).
__global__ void __launch_bounds__(256) pool_prepare_kernel(const int* __restrict__ child, int top_h,
                                                           int* __restrict__ inv, uint4* __restrict__ top,
                                                           int chunks) {
  grid_dependency_wait();
  const long long total = (long long)top_h * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i / chunks), c = (int)(i % chunks);
    const int ch = child[p];
    if (ch < 0) top[i] = make_uint4(0, 0, 0, 0);
    else if (c == 0) inv[ch] = p;
  }
}

// -1: not a shape the mma kernel is built for
int try_pw_mma(const PwArgs& a, int cout, cudaStream_t st) {
  if (a.y_stride != cout || a.co_base != 0) return -1;
  if ((uintptr_t)a.w % 8 != 0) return -1;          // the weights are read two at a time
#define OCNN_PW_CASE(CI, CO) if (a.cin == CI && cout == CO) return launch_pw_mma<CI, CO>(a, st);
  OCNN_PW_CASE(8, 8) OCNN_PW_CASE(8, 16) OCNN_PW_CASE(8, 32) OCNN_PW_CASE(8, 64)
  OCNN_PW_CASE(16, 8) OCNN_PW_CASE(16, 16) OCNN_PW_CASE(16, 32) OCNN_PW_CASE(16, 64)
  OCNN_PW_CASE(32, 8) OCNN_PW_CASE(32, 16) OCNN_PW_CASE(32, 32) OCNN_PW_CASE(32, 64)
  OCNN_PW_CASE(64, 8) OCNN_PW_CASE(64, 16) OCNN_PW_CASE(64, 32)
#undef OCNN_PW_CASE
  return -1;
}

}  // namespace

// Used by ocnn_octree_conv for 1x1x1 stride-1 bf16 node-major convolutions.  Returns -1 when the
// shape is not one this kernel takes (the caller then uses the general kernel).
int conv_pointwise_bf16(const void* x, const float* w, void* y, int h, int cin, int cout,
                        const ocnn_conv_epilogue* ep, cudaStream_t st, bool f16) {
  if (cin % 8 != 0 || cin > 256 || (long long)cin * cout > 16384) return -1;
  if (cout != 8 && cout != 16 && cout != 32 && cout != 64) return -1;
  if (((uintptr_t)x % 16) != 0 || ((uintptr_t)y % 16) != 0) return -1;
  if (ep && ep->residual_dev && ((uintptr_t)ep->residual_dev % 16) != 0) return -1;
  PwArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.w = w;
  a.y = static_cast<__nv_bfloat16*>(y);
  a.h = h; a.cin = cin;
  a.y_stride = cout; a.co_base = 0;
  a.scale = ep ? ep->scale_dev : nullptr;
  a.bias = ep ? ep->bias_dev : nullptr;
  a.residual = ep ? static_cast<const __nv_bfloat16*>(ep->residual_dev) : nullptr;
  a.relu = ep ? ep->relu : 0;
  a.f16 = f16 ? 1 : 0;
  a.pool_inv = nullptr;
  a.w2 = nullptr; a.scale2 = nullptr; a.bias2 = nullptr; a.y2 = nullptr; a.relu2 = 0;
  a.wide = (((uintptr_t)x % 32) == 0 && ((uintptr_t)y % 32) == 0 &&
            (!(ep && ep->residual_dev) || ((uintptr_t)ep->residual_dev % 32) == 0)) ? 1 : 0;
  {
    static const int use_mma = [] { const char* e = getenv("OCNN_PW_MMA"); return e ? atoi(e) : 1; }();
    if (use_mma) {
      const int rc = try_pw_mma(a, cout, st);
      if (rc != -1) return rc;
    }
  }
  switch (cout) {
    case 8: return launch_pw<8, 2>(a, st);
    case 16: return launch_pw<16, 2>(a, st);
    case 32: return launch_pw<32, 1>(a, st);
    case 64: {
      // 64 accumulators per thread leave too little occupancy: two passes of 32 channels (the
      // input row is 1/4 of the traffic or less, so reading it twice is cheap)
      if (int s0 = launch_pw<32, 1>(a, st)) return s0;
      a.co_base = 32;
      return launch_pw<32, 1>(a, st);
    }
    default: return -1;
  }
}

// 1x1x1 convolution + OctreeMaxPool (max over sibling groups, pad to the parent level) in one pass
// over the data: the streaming kernel's 16-row tiles are two sibling groups.  -1: not a shape that
// kernel takes.
int conv_pointwise_pool_bf16(const void* x, const float* w, void* top, const int* child_parent, int h,
                             int top_h, int cin, int cout, const ocnn_conv_epilogue* ep, int* inv,
                             cudaStream_t st, bool f16) {
  if (h % 8 != 0 || cout % 8 != 0) return -1;
  if (((uintptr_t)x % 16) != 0 || ((uintptr_t)top % 16) != 0) return -1;
  if (ep && ep->residual_dev && ((uintptr_t)ep->residual_dev % 16) != 0) return -1;
  PwArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.w = w;
  a.y = static_cast<__nv_bfloat16*>(top);
  a.h = h; a.cin = cin;
  a.y_stride = cout; a.co_base = 0;
  a.scale = ep ? ep->scale_dev : nullptr;
  a.bias = ep ? ep->bias_dev : nullptr;
  a.residual = ep ? static_cast<const __nv_bfloat16*>(ep->residual_dev) : nullptr;
  a.relu = ep ? ep->relu : 0;
  a.f16 = f16 ? 1 : 0;
  a.wide = 0;
  a.pool_inv = inv;
  a.w2 = nullptr; a.scale2 = nullptr; a.bias2 = nullptr; a.y2 = nullptr; a.relu2 = 0;
  // is it a shape of the mma kernel?  (decided before anything is launched)
  bool known = false;
  for (int ci : {8, 16, 32, 64})
    for (int co : {8, 16, 32, 64})
      if (cin == ci && cout == co && !(ci == 64 && co == 64)) known = true;
  if (!known || (uintptr_t)w % 8 != 0) return -1;
  const int chunks = cout / 8;
  OCNN_CUDA_OK(launch_chained(pool_prepare_kernel, dim3(grid_for((long long)top_h * chunks, 256, 8)), dim3(256), 0,
                              st, child_parent, top_h, inv, static_cast<uint4*>(top), chunks));
  OCNN_LAUNCH_OK("pool_prepare_kernel");
  return try_pw_mma(a, cout, st);
}

// Two 1x1x1 layers in a row (a block's conv1x1b with its shortcut, then the next block's conv1x1a)
// as one pass: the second reads the first's rows from registers.  -1: not a shape it is built for.
int conv_pointwise_chain_bf16(const void* x, const float* w1, void* y1, int h, int cin, int cmid,
                              const ocnn_conv_epilogue* ep1, const float* w2, void* y2, int cout2,
                              const ocnn_conv_epilogue* ep2, cudaStream_t st, bool f16) {
  if (((uintptr_t)x % 16) || ((uintptr_t)y1 % 16) || ((uintptr_t)y2 % 16)) return -1;
  if (((uintptr_t)w1 % 8) || ((uintptr_t)w2 % 8)) return -1;
  if (ep1 && ep1->residual_dev && ((uintptr_t)ep1->residual_dev % 16) != 0) return -1;
  if (ep2 && ep2->residual_dev) return -1;
  PwArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.w = w1;
  a.y = static_cast<__nv_bfloat16*>(y1);
  a.h = h; a.cin = cin;
  a.y_stride = cmid; a.co_base = 0;
  a.scale = ep1 ? ep1->scale_dev : nullptr;
  a.bias = ep1 ? ep1->bias_dev : nullptr;
  a.residual = ep1 ? static_cast<const __nv_bfloat16*>(ep1->residual_dev) : nullptr;
  a.relu = ep1 ? ep1->relu : 0;
  a.f16 = f16 ? 1 : 0;
  a.wide = 0;
  a.pool_inv = nullptr;
  a.w2 = w2;
  a.scale2 = ep2 ? ep2->scale_dev : nullptr;
  a.bias2 = ep2 ? ep2->bias_dev : nullptr;
  a.y2 = static_cast<__nv_bfloat16*>(y2);
  a.relu2 = ep2 ? ep2->relu : 0;
  const long long warps = ((long long)h + 15) / 16;
  const long long want = (warps + 47) / 48;
  const long long cap = (long long)sm_count() * 8;
  const int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
#define OCNN_CHAIN_CASE(CI, CM, CO)                                                                     \
  if (cin == CI && cmid == CM && cout2 == CO) {                                                         \
    if (f16)                                                                                            \
      OCNN_CUDA_OK(launch_chained(conv_pw_mma_kernel<CI, CM, true, CO>, dim3(grid), dim3(256), 0,        \
                                  st, a));                                                              \
    else                                                                                                \
      OCNN_CUDA_OK(launch_chained(conv_pw_mma_kernel<CI, CM, false, CO>, dim3(grid), dim3(256), 0,       \
                                  st, a));                                                              \
    OCNN_LAUNCH_OK("conv_pw_mma_kernel");                                                               \
    return OCNN_OK;                                                                                     \
  }
  OCNN_CHAIN_CASE(8, 32, 8) OCNN_CHAIN_CASE(16, 64, 16) OCNN_CHAIN_CASE(16, 32, 8) OCNN_CHAIN_CASE(8, 16, 8)
#undef OCNN_CHAIN_CASE
  return -1;
}

// The two-input 1x1x1 layer on the streaming kernel, for the shapes and sizes where it beats the
// tensor-core kernels (a big level, few channels).  -1: not one of them.
int conv_pointwise_pair_packed(const void* xa, int ca, const void* xb, int cb, const void* packed,
                               int npad, void* y, int h, int cout, const ocnn_conv_epilogue* ep,
                               cudaStream_t st, bool f16) {
  static const int enabled = [] { const char* e = getenv("OCNN_PW_MMA"); return e ? atoi(e) : 1; }();
  if (!enabled || h < 100000) return -1;
  if (!(ca == 16 && cb == 32 && cout == 64)) return -1;
  if (((uintptr_t)xa % 16) || ((uintptr_t)xb % 16) || ((uintptr_t)y % 16) || ((uintptr_t)packed % 4)) return -1;
  if (ep && ep->residual_dev && ((uintptr_t)ep->residual_dev % 16) != 0) return -1;
  PwPairArgs a;
  a.xa = static_cast<const __nv_bfloat16*>(xa);
  a.xb = static_cast<const __nv_bfloat16*>(xb);
  a.packed = static_cast<const uint16_t*>(packed);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.h = h; a.npad = npad;
  a.scale = ep ? ep->scale_dev : nullptr;
  a.bias = ep ? ep->bias_dev : nullptr;
  a.residual = ep ? static_cast<const __nv_bfloat16*>(ep->residual_dev) : nullptr;
  a.relu = ep ? ep->relu : 0;
  const long long warps = ((long long)h + 15) / 16;
  const long long want = (warps + 47) / 48;
  const long long cap = (long long)sm_count() * 8;
  const int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  if (f16)
    OCNN_CUDA_OK(launch_chained(conv_pw_pair_kernel<16, 32, 64, true>, dim3(grid), dim3(256), 0, st, a));
  else
    OCNN_CUDA_OK(launch_chained(conv_pw_pair_kernel<16, 32, 64, false>, dim3(grid), dim3(256), 0, st, a));
  OCNN_LAUNCH_OK("conv_pw_pair_kernel");
  return OCNN_OK;
}

}  // namespace ocnn
