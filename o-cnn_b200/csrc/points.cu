// Point-cloud preparation on the device, the steps the reference runs on the CPU in its DataLoader
// workers before points2octree: transform_points (displace along normals, rotate, translate,
// scale, orient normals), normalize_points, clip_points and the bounding box behind
// bounding_sphere(method = "box").  Restates PointsParser::displace / rotate / translate / scale /
// orient_normal / clip (octree/octree/points_parser.cpp:42-259) and bounding_box
// (octree/octree/math_functions.cpp:113-128); bindings pytorch/cpp/transform_points.cpp:7-125.
//
// Compiled without fused multiply-add so that every coordinate rounds as the reference's scalar
// CPU loops do (the cells a point falls into must not depend on where the transform ran).
#include "common.cuh"

namespace ocnn {
namespace {

struct TransformArgs {
  float* xyz;        // [n, 3]
  float* normal;     // [n, 3] or NULL
  long long n;
  float offset;      // displacement along the normal (applied when > 1e-10 and normals exist)
  int rotate;
  float rot[9];      // column-major as the reference's rotation_matrix: out[m] = sum_k rot[k*3+m]*in[k]
  int translate;
  float shift[3];
  int scale;         // 0: none, 1: uniform, 2: per axis (normals are divided and renormalised)
  float s[3];
  int orient;        // 0: none, 1..3: flip normals whose x / y / z is negative, 4: absolute values
};

__global__ void transform_kernel(const TransformArgs a) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    float p[3] = {a.xyz[3 * i], a.xyz[3 * i + 1], a.xyz[3 * i + 2]};
    float q[3] = {0.f, 0.f, 0.f};
    const bool has_n = a.normal != nullptr;
    if (has_n) { q[0] = a.normal[3 * i]; q[1] = a.normal[3 * i + 1]; q[2] = a.normal[3 * i + 2]; }
    if (has_n && a.offset > 1.0e-10f) {
#pragma unroll
      for (int m = 0; m < 3; ++m) p[m] += q[m] * a.offset;
    }
    if (a.rotate) {
      float t[3], u[3];
#pragma unroll
      for (int m = 0; m < 3; ++m) {
        // matrix_prod's order: C = 0, then += A[k*M + m] * B[k] for k = 0, 1, 2
        float c = 0.f, d = 0.f;
#pragma unroll
        for (int k = 0; k < 3; ++k) { c += a.rot[k * 3 + m] * p[k]; d += a.rot[k * 3 + m] * q[k]; }
        t[m] = c; u[m] = d;
      }
#pragma unroll
      for (int m = 0; m < 3; ++m) { p[m] = t[m]; q[m] = u[m]; }
    }
    if (a.translate) {
#pragma unroll
      for (int m = 0; m < 3; ++m) p[m] += a.shift[m];
    }
    if (a.scale) {
#pragma unroll
      for (int m = 0; m < 3; ++m) p[m] *= a.s[m];
      if (a.scale == 2 && has_n) {
#pragma unroll
        for (int m = 0; m < 3; ++m) q[m] *= 1.0f / a.s[m];
        float len = 0.f;
#pragma unroll
        for (int m = 0; m < 3; ++m) len += q[m] * q[m];
        const float inv = 1.0f / (sqrtf(len) + 1.0e-15f);
#pragma unroll
        for (int m = 0; m < 3; ++m) q[m] = q[m] * inv;
      }
    }
    if (has_n && a.orient >= 1 && a.orient <= 3) {
      if (q[a.orient - 1] < 0) { q[0] = -q[0]; q[1] = -q[1]; q[2] = -q[2]; }
    } else if (has_n && a.orient == 4) {
#pragma unroll
      for (int m = 0; m < 3; ++m) if (q[m] < 0) q[m] = -q[m];
    }
    a.xyz[3 * i] = p[0]; a.xyz[3 * i + 1] = p[1]; a.xyz[3 * i + 2] = p[2];
    if (has_n) { a.normal[3 * i] = q[0]; a.normal[3 * i + 1] = q[1]; a.normal[3 * i + 2] = q[2]; }
  }
}

// ---- clip: keep the points strictly inside the box, in order --------------------------------------
constexpr int kClipThreads = 256;
constexpr int kClipItems = 8;                       // points per thread
constexpr int kClipTile = kClipThreads * kClipItems;

__device__ __forceinline__ int inside(const float* __restrict__ xyz, long long i, const float* lo,
                                      const float* hi) {
  const float x = xyz[3 * i], y = xyz[3 * i + 1], z = xyz[3 * i + 2];
  return (lo[0] < x && x < hi[0] && lo[1] < y && y < hi[1] && lo[2] < z && z < hi[2]) ? 1 : 0;
}

struct Box { float lo[3], hi[3]; };

// pass 1: mask and the number of kept points per tile
__global__ void __launch_bounds__(kClipThreads) clip_count_kernel(const float* __restrict__ xyz,
                                                                 long long n, Box box,
                                                                 int* __restrict__ mask,
                                                                 int* __restrict__ tile_count) {
  __shared__ int warp_sum[kClipThreads / 32];
  const long long base = (long long)blockIdx.x * kClipTile;
  int mine = 0;
#pragma unroll
  for (int j = 0; j < kClipItems; ++j) {
    const long long i = base + (long long)j * kClipThreads + threadIdx.x;
    if (i < n) {
      const int in = inside(xyz, i, box.lo, box.hi);
      mask[i] = in;
      mine += in;
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < kClipThreads / 32; ++w) s += warp_sum[w];
    tile_count[blockIdx.x] = s;
  }
}

// pass 2: exclusive scan of the tile counts by one block (tiles <= a few thousand for any cloud the
// octree format can hold); total -> tile_count[tiles]
__global__ void __launch_bounds__(1024) clip_scan_kernel(int* __restrict__ tile_count, int tiles) {
  __shared__ int part[1024];
  const int per = (tiles + 1023) / 1024;
  const int lo = threadIdx.x * per, hi = min(tiles, lo + per);
  int s = 0;
  for (int t = lo; t < hi; ++t) s += tile_count[t];
  part[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int t = 0; t < 1024; ++t) { const int v = part[t]; part[t] = run; run += v; }
    tile_count[tiles] = run;
  }
  __syncthreads();
  int run = part[threadIdx.x];
  for (int t = lo; t < hi; ++t) { const int v = tile_count[t]; tile_count[t] = run; run += v; }
}

struct ClipProps {
  const float* src[4];
  float* dst[4];
  int channels[4];
};

// pass 3: every kept point moves to its rank; the header's point count is rewritten; an empty
// result keeps one point at the box's lower corner (points_parser.cpp:169-175)
__global__ void __launch_bounds__(kClipThreads) clip_move_kernel(long long n, ClipProps pr, Box box,
                                                                int* __restrict__ mask,
                                                                const int* __restrict__ tile_offset,
                                                                int tiles, int* __restrict__ pt_num_out) {
  __shared__ int warp_base[kClipThreads / 32];
  __shared__ int carry;
  const int total = tile_offset[tiles];
  if (total == 0) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      for (int m = 0; m < 3; ++m) pr.dst[0][m] = box.lo[m];
      for (int t = 1; t < 4; ++t)
        for (int c = 0; c < pr.channels[t]; ++c) pr.dst[t][c] = pr.src[t][c];
      mask[0] = 1;
      *pt_num_out = 1;
    }
    return;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *pt_num_out = total;
  if (threadIdx.x == 0) carry = tile_offset[blockIdx.x];
  const long long base = (long long)blockIdx.x * kClipTile;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // items are visited round by round (j), inside a round in thread order: the same order as i
  for (int j = 0; j < kClipItems; ++j) {
    const long long i = base + (long long)j * kClipThreads + threadIdx.x;
    const int in = (i < n) ? mask[i] : 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, in);
    if (lane == 0) warp_base[warp] = __popc(ballot);
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_base[w];
    int round_total = 0;
    for (int w = 0; w < kClipThreads / 32; ++w) round_total += warp_base[w];
    const int rank = carry + before + __popc(ballot & ((1u << lane) - 1u));
    if (in) {
      for (int t = 0; t < 4; ++t) {
        const int ch = pr.channels[t];
        for (int c = 0; c < ch; ++c) pr.dst[t][(long long)rank * ch + c] = pr.src[t][i * ch + c];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) carry += round_total;
    __syncthreads();
  }
}

// ---- bounding box -----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bbox_kernel(const float* __restrict__ xyz, long long n,
                                                  float* __restrict__ part /* [grid, 6] */) {
  float lo[3] = {INFINITY, INFINITY, INFINITY}, hi[3] = {-INFINITY, -INFINITY, -INFINITY};
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
#pragma unroll
    for (int m = 0; m < 3; ++m) {
      const float v = xyz[3 * i + m];
      lo[m] = fminf(lo[m], v);
      hi[m] = fmaxf(hi[m], v);
    }
  }
  __shared__ float s[256 / 32][6];
#pragma unroll
  for (int m = 0; m < 3; ++m) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
      lo[m] = fminf(lo[m], __shfl_xor_sync(0xffffffffu, lo[m], o));
      hi[m] = fmaxf(hi[m], __shfl_xor_sync(0xffffffffu, hi[m], o));
    }
  }
  if ((threadIdx.x & 31) == 0) {
    for (int m = 0; m < 3; ++m) { s[threadIdx.x >> 5][m] = lo[m]; s[threadIdx.x >> 5][3 + m] = hi[m]; }
  }
  __syncthreads();
  if (threadIdx.x < 6) {
    float v = s[0][threadIdx.x];
    for (int w = 1; w < 256 / 32; ++w)
      v = threadIdx.x < 3 ? fminf(v, s[w][threadIdx.x]) : fmaxf(v, s[w][threadIdx.x]);
    part[blockIdx.x * 6 + threadIdx.x] = v;
  }
}

__global__ void bbox_final_kernel(const float* __restrict__ part, int blocks, float* __restrict__ out) {
  if (threadIdx.x < 6) {
    float v = part[threadIdx.x];
    for (int b = 1; b < blocks; ++b)
      v = threadIdx.x < 3 ? fminf(v, part[b * 6 + threadIdx.x]) : fmaxf(v, part[b * 6 + threadIdx.x]);
    out[threadIdx.x] = v;
  }
}

}  // namespace
}  // namespace ocnn

extern "C" {

int ocnn_points_transform(float* xyz, float* normal, int64_t n, float offset, const float* rot9,
                          const float* shift3, const float* scale3, int orient, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(n >= 0, "ocnn_points_transform: negative point count");
  OCNN_REQUIRE(orient >= 0 && orient <= 4, "ocnn_points_transform: orient must be 0..4 (got %d)", orient);
  if (n == 0) return OCNN_OK;
  OCNN_REQUIRE(xyz != nullptr, "ocnn_points_transform: null points");
  TransformArgs a;
  a.xyz = xyz; a.normal = normal; a.n = n; a.offset = offset;
  a.rotate = rot9 != nullptr;
  for (int i = 0; i < 9; ++i) a.rot[i] = rot9 ? rot9[i] : 0.f;
  a.translate = shift3 != nullptr;
  for (int i = 0; i < 3; ++i) a.shift[i] = shift3 ? shift3[i] : 0.f;
  a.scale = 0;
  for (int i = 0; i < 3; ++i) a.s[i] = 1.f;
  if (scale3 != nullptr) {
    // PointsParser::scale: nothing for (1,1,1) or when any factor is 0
    const bool unit = scale3[0] == 1.f && scale3[1] == 1.f && scale3[2] == 1.f;
    const bool zero = scale3[0] == 0.f || scale3[1] == 0.f || scale3[2] == 0.f;
    if (!unit && !zero) {
      for (int i = 0; i < 3; ++i) a.s[i] = scale3[i];
      a.scale = (scale3[0] == scale3[1] && scale3[0] == scale3[2]) ? 1 : 2;
    }
  }
  a.orient = orient;
  transform_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  OCNN_LAUNCH_OK("transform_kernel");
  return OCNN_OK;
}

size_t ocnn_points_clip_workspace_bytes(int64_t n) {
  if (n < 0) return 0;
  const long long tiles = (n + ocnn::kClipTile - 1) / ocnn::kClipTile;
  return (size_t)(tiles + 2) * sizeof(int);
}

int ocnn_points_clip(const float* const src[4], float* const dst[4], const int channels[4], int64_t n,
                     const float bbmin[3], const float bbmax[3], int32_t* mask, int32_t* pt_num_out,
                     void* workspace, size_t workspace_bytes, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(src && dst && channels && bbmin && bbmax && mask && pt_num_out, "ocnn_points_clip: null argument");
  OCNN_REQUIRE(n > 0, "ocnn_points_clip: the cloud must hold at least one point");
  OCNN_REQUIRE(channels[0] == 3 && src[0] && dst[0], "ocnn_points_clip: property 0 must be the xyz block");
  const long long tiles = (n + kClipTile - 1) / kClipTile;
  if (workspace_bytes < ocnn_points_clip_workspace_bytes(n) || workspace == nullptr)
    return fail(OCNN_ERR_CAPACITY, "ocnn_points_clip: workspace of %zu bytes, need %zu", workspace_bytes,
                ocnn_points_clip_workspace_bytes(n));
  Box box;
  ClipProps pr;
  for (int m = 0; m < 3; ++m) { box.lo[m] = bbmin[m]; box.hi[m] = bbmax[m]; }
  for (int t = 0; t < 4; ++t) {
    pr.channels[t] = channels[t];
    pr.src[t] = src[t]; pr.dst[t] = dst[t];
    OCNN_REQUIRE(channels[t] >= 0 && (channels[t] == 0 || (src[t] && dst[t] && src[t] != dst[t])),
                 "ocnn_points_clip: property %d needs distinct source and destination blocks", t);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* counts = static_cast<int*>(workspace);
  clip_count_kernel<<<(int)tiles, kClipThreads, 0, st>>>(src[0], n, box, mask, counts);
  clip_scan_kernel<<<1, 1024, 0, st>>>(counts, (int)tiles);
  clip_move_kernel<<<(int)tiles, kClipThreads, 0, st>>>(n, pr, box, mask, counts, (int)tiles, pt_num_out);
  OCNN_LAUNCHES_OK("clip kernels", 3);
  return OCNN_OK;
}

size_t ocnn_points_bbox_workspace_bytes(void) { return (size_t)ocnn::kSMs * 4 * 6 * sizeof(float); }

int ocnn_points_bbox(const float* xyz, int64_t n, float* out6, void* workspace, size_t workspace_bytes,
                     void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(xyz && out6 && n > 0, "ocnn_points_bbox: null pointer or empty cloud");
  if (workspace == nullptr || workspace_bytes < ocnn_points_bbox_workspace_bytes())
    return fail(OCNN_ERR_CAPACITY, "ocnn_points_bbox: workspace of %zu bytes, need %zu", workspace_bytes,
                ocnn_points_bbox_workspace_bytes());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int blocks = grid_for(n, 256, 4);
  if (blocks > kSMs * 4) blocks = kSMs * 4;
  bbox_kernel<<<blocks, 256, 0, st>>>(xyz, n, static_cast<float*>(workspace));
  bbox_final_kernel<<<1, 32, 0, st>>>(static_cast<const float*>(workspace), blocks, out6);
  OCNN_LAUNCHES_OK("bbox kernels", 2);
  return OCNN_OK;
}

}  // extern "C"
