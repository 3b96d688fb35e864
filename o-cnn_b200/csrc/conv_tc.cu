// Octree convolution on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 in, fp32 accumulate.
//
// One CTA computes a tile of 128 output nodes x all output channels as an implicit GEMM
//     D[128, Cout] = A[128, K] * B[K, Cout],     K = taps * Cin walked tap-major (k = t*Cin + ci),
// where row r of A is the concatenation, over the taps, of the Cin-channel rows of node r's
// neighbours (zeros where a neighbour does not exist).  A is never materialised in HBM: each
// K-block of 64 (128 bytes per row) is gathered straight into the 128B-swizzled K-major shared
// memory layout the UMMA smem descriptor expects, 16 bytes per cp.async, zero-filled for missing
// neighbours.  B comes from weights packed once per layer into the same swizzled image, one
// contiguous chunk per K-block, fetched with one bulk async copy.  Accumulators live in TMEM and
// are read back by the four epilogue warps with tcgen05.ld.
//
// Sibling-group mode (stride 1, more than one tap, Cin <= 32, Cout <= 32): the eight nodes of a
// sibling group share one 4x4x4 neighbour block, so gathering per node reads each of its 64 rows
// 3.4 times (8 x 27 = 216 reads).  Here a tile ROW is a whole group: A row = the group's 64
// neighbour rows back to back (K = 64*Cin, read once, indices straight from the neighbour block),
// B = the weights expanded to [64*Cin, 8*Cout] with zeros where a block position is outside an
// octant's 3x3x3 window, D row = the group's 8 output nodes x Cout, which is exactly the group's
// contiguous stretch of the node-major output.  2.4x the flops (the tensor core idles anyway at
// these channel counts) for 3.4x fewer gathers and a tile of 1024 nodes instead of 128.
//
// Warp roles (192 threads): warps 0-3 gather A (one tile row per thread, or four tile rows per
// warp instruction for the few-channel group layers) and later run the epilogue (TMEM lane
// quarter = warp id); warp 4 allocates TMEM and its lane 0 issues the MMAs; lane 0 of warp 5
// streams the weight tiles.  A ring of 2-7 {A tile, B tile} stages is handed between them with
// mbarriers: full[s] (128 gather arrivals, each fired by cp.async.mbarrier.arrive.noinc when the
// thread's copies have landed, + the weight copy's bytes), empty[s] (tcgen05.commit when the MMAs
// that read the stage have retired).  A level too small to fill the SMs runs 64- or 32-row tiles:
// the MMA is still 128 rows, the rows a tile does not have are neither gathered nor stored.
//
// Every wait is bounded: a wait that runs out sets *status (and a CTA-wide abort flag); the other
// roles see the flag at their next wait and stop issuing.  Before the CTA frees its TMEM and
// returns, the gather threads wait for their own cp.async copies, the MMA thread commits what it
// has issued and waits (bounded) for that commit, and the weight thread gives the bulk copies it
// has in flight a bounded time to land — the launch never hangs the GPU.
#include "common.cuh"

namespace ocnn {
// conv_pw.cu
int conv_pointwise_pair_packed(const void* xa, int ca, const void* xb, int cb, const void* packed,
                               int npad, void* y, int h, int cout, const ocnn_conv_epilogue* ep,
                               cudaStream_t st, bool f16);
namespace {

constexpr int kTileM = 128;          // nodes per CTA = TMEM lanes
constexpr int kBlockK = 64;          // bf16 elements per K-block = one 128-byte swizzle row
constexpr int kStageA = kTileM * 128;  // bytes of one A stage
constexpr int kThreads = 192;
constexpr int kGroupTableStride = 132;   // ints between positions in the group-mode index table:
                                         // 4*position + slot spreads a 16-byte read over all banks
constexpr unsigned kSpinLimit = 1u << 20;

enum : int { kErrFullWait = 1, kErrEmptyWait = 2, kErrAccumWait = 3, kErrWeightWait = 4 };

struct TcArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* x2;   // two-input 1x1x1 layer: the K row of node h is x[h] followed by x2[h]
  int cpt_a;                 // ... and x's share of it in 16-byte chunks (0: one input)
  const uint8_t* wpacked;
  __nv_bfloat16* y;
  const int* neigh;
  const int* child;    // convolution on non-empty nodes only: the level's child array and its
  const int* ichild;   // inverse (node of the i-th non-empty node); NULL otherwise
  int h_in, h_out, cin, cout, npad, T, stride, identity, nkb, stages, tmem_cols;
  int group;        // 1: tile rows are sibling groups (see the header comment), 0: nodes
  int rows;         // number of tile rows in total: h_out, or h_out / 8 in group mode
  int row_elems;    // output elements per tile row: cout, or 8 * cout in group mode
  int y_stride;     // elements between consecutive output rows (= row_elems unless the layer's
                    // output channels are produced in several launches)
  int tile_rows;    // tile rows a CTA actually computes (128, 64 or 32): small levels are cut into
                    // more, emptier tiles so that every SM gets one; the MMA is always 128 rows
  int wide;         // output (and residual) rows can be accessed 32 bytes at a time
  int rowsplit;     // gather mapping: 0 = one tile row per thread; four tile rows per warp
                    // instruction: 1 = group mode with 8 or 16 channels (indices from global memory),
                    // 2 = node mode, Cin % 64 == 0, 3 = group mode through the shared index table,
                    // 4 = node mode, any other Cin with more than one tap (index table with the
                    // padded stride, two 16-byte index reads per K-block)
  int up;           // stride-2 deconvolution in gather form: tile rows are nodes of the finer level,
                    // the gathered rows are their source sibling groups (common.cuh: up_source_group)
  int f16;          // the 16-bit elements are fp16 instead of bf16
  int expand_cout;  // > 0: the kernel-2 stride-2 deconvolution as a dense product: tile row = a
                    // parent, its row_elems = 8 * expand_cout columns are (octant, channel) pairs
  int fold_cout;    // > 0: a 1x1x1 layer with Cin < 64 run on rows of 64/Cin nodes (one 128-byte
                    // line) against block-diagonal weights: column n is channel n % fold_cout of
                    // node n / fold_cout of the row
  const int* scatter_child;   // with expand_cout: Child block of the finer level; octant o of tile
                              // row h is written to row scatter_child[8h + o] (skipped when < 0)
  const float* scale;
  const float* bias;
  const __nv_bfloat16* residual;
  int relu;
  int* status;
  signed char tap[27];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  for (unsigned it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && *abort_flag != 0) return false;
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

// K-major, 128-byte-swizzled shared memory matrix descriptor (sm_100 format): start address >> 4
// in bits [0,14), leading byte offset (unused for swizzled K-major, 1) in [16,30), stride byte
// offset = 1024 B between 8-row groups in [32,46), descriptor version 1 in [46,48), layout type
// SWIZZLE_128B = 2 in [61,64).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
                 "=r"(v[6]), "=r"(v[7])
               : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
               : "memory");
}

// Gather one K-block (8 chunks of 16 bytes) of this thread's tile row.  CPT = 16-byte chunks per
// tap (Cin / 8) when it is one of the specialised values, 0 = any (running counters).  Chunk c of
// the row lands at position c ^ (row & 7): the 128-byte swizzle.
// nbr_col[t * nbr_stride] is the row to read for tap t: a column of the shared-memory table in
// node mode (stride 128), the group's own 64-int neighbour block in global memory in group mode
// (stride 1).
template <int CPT>
__device__ __forceinline__ void gather_block(const TcArgs& a, const int* __restrict__ nbr_col,
                                             const int nbr_stride, const int T, int kb,
                                             uint32_t dst_row, uint32_t sw, int& t_run,
                                             int& cc_run) {
  const char* xb = reinterpret_cast<const char*>(a.x);
  const uint32_t row_bytes = (uint32_t)a.cin * 2u;
  if constexpr (CPT >= 8) {
    // the whole K-block reads one neighbour row
    constexpr int kBlocksPerTap = CPT / 8;
    const int t = kb / kBlocksPerTap;
    const int p = t < T ? nbr_col[t * nbr_stride] : -1;
    const char* src = xb;
    if (p >= 0) src = xb + (size_t)((uint32_t)p * row_bytes) + (kb % kBlocksPerTap) * 128;
    const uint32_t bytes = p >= 0 ? 16u : 0u;
    const uint32_t step = p >= 0 ? 16u : 0u;
#pragma unroll
    for (int c = 0; c < 8; ++c) cp_async16(dst_row + (((uint32_t)c ^ sw) << 4), src + c * step, bytes);
  } else if constexpr (CPT > 0) {
    constexpr int kTapsPerBlock = 8 / CPT;
    int pj[kTapsPerBlock];
#pragma unroll
    for (int j = 0; j < kTapsPerBlock; ++j) {       // all index loads first, then the copies
      const int t = kb * kTapsPerBlock + j;
      pj[j] = t < T ? nbr_col[t * nbr_stride] : -1;
    }
#pragma unroll
    for (int j = 0; j < kTapsPerBlock; ++j) {
      const int p = pj[j];
      const char* src = xb;
      if (p >= 0) src = xb + (size_t)((uint32_t)p * row_bytes);
      const uint32_t bytes = p >= 0 ? 16u : 0u;
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const int c = j * CPT + cc;
        cp_async16(dst_row + (((uint32_t)c ^ sw) << 4), p >= 0 ? src + cc * 16 : xb, bytes);
      }
    }
  } else {
    const int cpt = a.cin >> 3;
    int p = t_run < T ? nbr_col[t_run * nbr_stride] : -1;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const char* src = p >= 0 ? xb + (size_t)((uint32_t)p * row_bytes) + cc_run * 16 : xb;
      cp_async16(dst_row + (((uint32_t)c ^ sw) << 4), src, p >= 0 ? 16u : 0u);
      if (++cc_run == cpt) {
        cc_run = 0;
        ++t_run;
        p = t_run < T ? nbr_col[t_run * nbr_stride] : -1;
      }
    }
  }
}

// Which tap the 16-byte chunk `chunk` of K-block kb belongs to, and the byte offset inside that
// neighbour's row.  CPT as in gather_block.
template <int CPT>
__device__ __forceinline__ void chunk_src(int cpt, int kb, int chunk, int& t, uint32_t& off) {
  if constexpr (CPT >= 8) {
    t = kb / (CPT / 8);
    off = (uint32_t)(kb % (CPT / 8)) * 128u + (uint32_t)chunk * 16u;
  } else if constexpr (CPT > 0) {
    t = kb * (8 / CPT) + chunk / CPT;
    off = (uint32_t)(chunk % CPT) * 16u;
  } else {
    const int g = kb * 8 + chunk;
    t = g / cpt;
    off = (uint32_t)(g - t * cpt) * 16u;
  }
}

// GENERAL compiles in the rarely used layer kinds (stride-2 deconvolution in gather form, the
// expanded kernel-2 deconvolution with its scattered epilogue); the convolutions of the
// classification networks run the variant without them.
template <int CPT, bool HALF, bool GENERAL>
__global__ void __launch_bounds__(kThreads, 3) conv_tc_kernel(const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern is a function of address bits [4,10)
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stage_b = a.npad * 128;
  uint8_t* sA = smem;
  uint8_t* sB = sA + a.stages * kStageA;
  int* nbr = reinterpret_cast<int*>(sB + a.stages * stage_b);
  // per-column scale and bias of the epilogue, staged once per CTA: read from global memory in
  // the epilogue they were a chain of cold misses (one per 128-byte line of each array) that every
  // thread of a one-wave launch sat through
  float* s_scale = reinterpret_cast<float*>(
      nbr + (a.group ? (a.rowsplit == 3 ? 64 * kGroupTableStride : 0)
                     : a.T * (a.rowsplit == 4 ? kGroupTableStride : kTileM)));
  float* s_bias = s_scale + a.npad;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + a.npad);
  uint64_t* full = bars;
  uint64_t* empty = bars + a.stages;
  uint64_t* accum = bars + 2 * a.stages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h0 = blockIdx.x * a.tile_rows;
  // blockIdx.y = 256-channel slice of the output (layers with more than 256 output channels)
  const int co_base = blockIdx.y * a.cout;
  const uint8_t* wpacked = a.wpacked + (size_t)blockIdx.y * a.nkb * (a.npad * 128);
  grid_dependency_trigger();     // the next layer's CTAs may queue up behind this grid's last wave

  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(&full[s]), kTileM + 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    mbar_init(smem_u32(accum), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_holder)), "r"((uint32_t)a.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // everything above is private to the CTA; from here on global memory is read, so the previous
  // kernel of the stream must have completed
  grid_dependency_wait();
  for (int n = tid; n < a.npad; n += kThreads) {
    // output channel of column n: columns are (octant, channel) pairs in group mode
    int co = a.group ? (n & (a.cout - 1)) : co_base + n;
    if (a.fold_cout) co = n % a.fold_cout;
    if (GENERAL && a.expand_cout) co = (co_base + n) % a.expand_cout;
    const bool live = n < a.row_elems;
    s_scale[n] = (live && a.scale) ? a.scale[co] : 1.f;
    s_bias[n] = (live && a.bias) ? a.bias[co] : 0.f;
  }
  if (tid < kTileM) {
    const int h = h0 + tid;          // node, or sibling group in group mode
    const bool live = tid < a.tile_rows && h < a.rows;
    if (a.group) {
      // The group's neighbour block IS the list of rows to gather, 64 contiguous ints.  The
      // gather either reads them straight from global memory, or (rowsplit == 3) from a shared
      // table [position][slot] that is filled here, 16 reads in flight at a time.
      if (a.rowsplit == 3) {
        const int slot = (tid & ~31) + ((tid & 3) << 3) + ((tid >> 2) & 7);
        const int* blk = a.neigh + ((long long)(live ? h : 0) << 6);
#pragma unroll
        for (int t0 = 0; t0 < 64; t0 += 16) {
          int pv[16];
#pragma unroll
          for (int t = 0; t < 16; ++t) pv[t] = live ? __ldg(blk + t0 + t) : -1;
#pragma unroll
          for (int t = 0; t < 16; ++t) nbr[(t0 + t) * kGroupTableStride + slot] = pv[t];
        }
      }
    } else {
      // on non-empty nodes only (octree2colP): tile row h is the h-th non-empty node; its
      // neighbours are looked up from the node itself and mapped back to non-empty ranks
      const int hn = (a.ichild != nullptr && live) ? a.ichild[h] : h;
      const int oct_code = ((hn & 4) << 2) | ((hn & 2) << 1) | (hn & 1);
      if (a.identity) {
        nbr[a.rowsplit >= 2 ? (tid & ~31) + ((tid & 3) << 3) + ((tid >> 2) & 7) : tid] = live ? h : -1;
      } else {
      // all (up to 27) table reads are issued before the first result is used: a load-then-store
      // loop would expose the L2 latency once per tap
      // with the four-rows-per-instruction mapping a thread serves rows sub + 4*i of its warp: their
      // entries are stored next to each other so that it reads them as two 16-byte words
      const int slot = a.rowsplit >= 2 ? (tid & ~31) + ((tid & 3) << 3) + ((tid >> 2) & 7) : tid;
      const int tstride = a.rowsplit == 4 ? kGroupTableStride : kTileM;
      int pv[27];
#pragma unroll
      for (int t = 0; t < 27; ++t) {
        int p = -1;
        if (t < a.T && live) {
          // a.tap[t] holds (tx<<4)|(ty<<2)|tz; adding the octant's (ox<<4)|(oy<<2)|oz gives the
          // position in the sibling group's 4x4x4 block (no field can carry: each sum is <= 3)
          if (GENERAL && a.up) {
            const int code = a.tap[t];
            p = up_source_group(a.neigh, hn, (code >> 4) * 9 + ((code >> 2) & 3) * 3 + (code & 3));
          } else {
            const long long at = a.stride == 2 ? ((long long)hn << 6) + a.tap[t]
                                               : ((long long)(hn >> 3) << 6) + a.tap[t] + oct_code;
            p = a.neigh[at];
          }
        }
        pv[t] = p;
      }
      if (a.child != nullptr) {
#pragma unroll
        for (int t = 0; t < 27; ++t)
          if (t < a.T && pv[t] >= 0) pv[t] = a.child[pv[t]];
      }
#pragma unroll
      for (int t = 0; t < 27; ++t)
        if (t < a.T) nbr[t * tstride + slot] = pv[t];
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
    // ---------------- A gather ----------------
    const int r = tid;
    bool alive = true;
    if ((CPT >= 8 || CPT == 0) && a.rowsplit == 2) {
      // Node mode with Cin a multiple of 64: a K-block of a tile row is one contiguous 128-byte stretch of a
      // neighbour's row.  A warp instruction copies four whole rows (lane = row within the four,
      // 16-byte chunk): every fetched sector is used in full, where one row per thread fetches
      // each 32-byte sector twice.  The thread's eight row indices of a tap are two 16-byte reads
      // of the shared table, once per tap.
      if constexpr (CPT >= 8 || CPT == 0) {
        const int kBlocksPerTap = CPT >= 8 ? CPT / 8 : a.cin >> 6;
        const int sub = lane >> 3, chunk = lane & 7;
        const int rbase = warp * 32 + sub;
        const char* xb = reinterpret_cast<const char*>(a.x);
        const uint32_t row_bytes = (uint32_t)a.cin * 2u;
        const int* my_idx = nbr + warp * 32 + sub * 8;
        uint32_t row_mask = 0;        // bit i: tile row rbase + 4*i exists
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (rbase + 4 * i < a.tile_rows && h0 + rbase + 4 * i < a.rows) row_mask |= 1u << i;
        int p[8];
        int s = 0;
        uint32_t pe = 1;
        int t = 0, part = 0;
        for (int kb = 0; kb < a.nkb; ++kb) {
          if (part == 0) {
            const int4 lo = *reinterpret_cast<const int4*>(my_idx + t * kTileM);
            const int4 hi = *reinterpret_cast<const int4*>(my_idx + t * kTileM + 4);
            p[0] = lo.x; p[1] = lo.y; p[2] = lo.z; p[3] = lo.w;
            p[4] = hi.x; p[5] = hi.y; p[6] = hi.z; p[7] = hi.w;
          }
          if (alive && kb >= a.stages)
            alive = mbar_wait(smem_u32(&empty[s]), pe, abort_flag, a.status, kErrEmptyWait);
          if (alive) {
            const uint32_t stage_base = smem_u32(sA + s * kStageA);
            const uint32_t off = (uint32_t)part * 128u + (uint32_t)chunk * 16u;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = rbase + 4 * i;
              const uint32_t dst = stage_base + (uint32_t)row * 128u +
                                   (((uint32_t)chunk ^ (uint32_t)(row & 7)) << 4);
              const int pi = p[i];
              const char* src = pi >= 0 ? xb + (size_t)((uint32_t)pi * row_bytes) + off : xb;
              if ((row_mask >> i) & 1u) cp_async16(dst, src, pi >= 0 ? 16u : 0u);
            }
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[s]))
                       : "memory");
          if (++s == a.stages) { s = 0; pe ^= 1u; }
          if (++part == kBlocksPerTap) { part = 0; ++t; }
        }
      }
    } else if (a.rowsplit) {
      // Sibling-group mode with 8 or 16 channels: every 16-byte chunk of a tile row comes from a
      // different node, so "one tile row per thread" makes each warp instruction touch 32
      // unrelated lines.  Here a warp instruction copies the 8 chunks of a K-block for 4 tile rows
      // (lane = row within the four, chunk): the chunks of one row are 8 (or 4) consecutive
      // positions of the group's 4x4x4 block, i.e. whole sibling sets, which are contiguous in
      // memory.  A thread serves chunk position `chunk` of rows rbase + 4*i, i = 0..7.
      const int sub = lane >> 3, chunk = lane & 7;
      const int rbase = warp * 32 + sub;
      const char* xb = reinterpret_cast<const char*>(a.x);
      const uint32_t row_bytes = (uint32_t)a.cin * 2u;
      const int cpt = a.cin >> 3;
      uint32_t row_mask = 0;        // bit i: tile row rbase + 4*i exists
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (rbase + 4 * i < a.tile_rows && h0 + rbase + 4 * i < a.rows) row_mask |= 1u << i;
      const int* my_idx = nbr + warp * 32 + sub * 8;     // rowsplit == 3: this thread's 8 rows
      auto fetch = [&](int kb, int (&p)[8], uint32_t& off) {
        int t;
        chunk_src<CPT>(cpt, kb, chunk, t, off);
        if (a.rowsplit >= 3) {
          if (t < a.T) {
            const int4 lo = *reinterpret_cast<const int4*>(my_idx + t * kGroupTableStride);
            const int4 hi = *reinterpret_cast<const int4*>(my_idx + t * kGroupTableStride + 4);
            p[0] = lo.x; p[1] = lo.y; p[2] = lo.z; p[3] = lo.w;
            p[4] = hi.x; p[5] = hi.y; p[6] = hi.z; p[7] = hi.w;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) p[i] = -1;
          }
          return;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          p[i] = -1;
          if (t < a.T && ((row_mask >> i) & 1u))
            p[i] = __ldg(a.neigh + (((long long)(h0 + rbase + 4 * i)) << 6) + t);
        }
      };
      int s = 0;
      uint32_t pe = 1;
      int p_cur[8];
      uint32_t off_cur;
      fetch(0, p_cur, off_cur);
      for (int kb = 0; kb < a.nkb; ++kb) {
        // the indices of the next block are requested before this block's copies are issued
        int p_nxt[8] = {-1, -1, -1, -1, -1, -1, -1, -1};
        uint32_t off_nxt = 0;
        if (kb + 1 < a.nkb) fetch(kb + 1, p_nxt, off_nxt);
        if (alive && kb >= a.stages)
          alive = mbar_wait(smem_u32(&empty[s]), pe, abort_flag, a.status, kErrEmptyWait);
        if (alive) {
          const uint32_t stage_base = smem_u32(sA + s * kStageA);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = rbase + 4 * i;
            const uint32_t dst = stage_base + (uint32_t)row * 128u +
                                 (((uint32_t)chunk ^ (uint32_t)(row & 7)) << 4);
            const int p = p_cur[i];
            const char* src = p >= 0 ? xb + (size_t)((uint32_t)p * row_bytes) + off_cur : xb;
            // rows the tile does not have are left as they are: their accumulator lanes are
            // never read
            if ((row_mask >> i) & 1u) cp_async16(dst, src, p >= 0 ? 16u : 0u);
          }
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[s]))
                     : "memory");
        if (++s == a.stages) { s = 0; pe ^= 1u; }
#pragma unroll
        for (int i = 0; i < 8; ++i) p_cur[i] = p_nxt[i];
        off_cur = off_nxt;
      }
    } else {
      // one tile row per thread
      const uint32_t row_off = (uint32_t)r * 128u;
      const uint32_t sw = (uint32_t)(r & 7);
      // rows the tile does not have gather nothing: their accumulator lanes are never read
      const bool row_ok = r < a.tile_rows && h0 + r < a.rows;
      const int* nbr_col = a.group ? a.neigh + ((long long)(row_ok ? h0 + r : 0) << 6) : nbr + r;
      const int nbr_stride = a.group ? 1 : kTileM;
      const int T = a.T;
      int s = 0, t_run = 0, cc_run = 0;
      uint32_t pe = 1;                       // parity of the next empty[] wait, flips per ring turn
      for (int kb = 0; kb < a.nkb; ++kb) {
        if (alive && kb >= a.stages)
          alive = mbar_wait(smem_u32(&empty[s]), pe, abort_flag, a.status, kErrEmptyWait);
        bool paired = false;
        if constexpr (CPT == 0) paired = a.x2 != nullptr;
        if (alive && row_ok && paired) {
          // chunk g of the node's K row: the first cpt_a chunks are its row of x, the rest its row
          // of x2, zeros beyond Cin
          const uint32_t cpt_all = (uint32_t)a.cin >> 3, cpt_a = (uint32_t)a.cpt_a;
          const char* row_a = reinterpret_cast<const char*>(a.x) + (size_t)(h0 + r) * (cpt_a * 16u);
          const char* row_b =
              reinterpret_cast<const char*>(a.x2) + (size_t)(h0 + r) * ((cpt_all - cpt_a) * 16u);
          const uint32_t dst_row = smem_u32(sA + s * kStageA) + row_off;
#pragma unroll
          for (uint32_t c = 0; c < 8; ++c) {
            const uint32_t g = (uint32_t)kb * 8u + c;
            const char* src = g < cpt_a ? row_a + g * 16u : row_b + (g - cpt_a) * 16u;
            const bool live = g < cpt_all;
            cp_async16(dst_row + ((c ^ sw) << 4), live ? src : row_a, live ? 16u : 0u);
          }
        } else if (alive && row_ok)
          gather_block<CPT>(a, nbr_col, nbr_stride, T, kb, smem_u32(sA + s * kStageA) + row_off, sw,
                            t_run, cc_run);
        // Arrive on full[s] when this thread's copies of the block have landed; the thread itself
        // moves on, so up to `stages` blocks of gathers are in flight per thread.
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[s]))
                     : "memory");
        if (++s == a.stages) { s = 0; pe ^= 1u; }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of ours in flight past this point

    // ---------------- epilogue: TMEM -> registers -> global ----------------
    // The residual is read 64 bytes (32 channels) of the row at a time, the four 16-byte pieces at
    // once and the next four before the current ones are used; the first are requested before
    // the wait for the accumulator.
    const int h = h0 + r;
    const bool row_ok = r < a.tile_rows && h < a.rows;
    constexpr bool f16 = HALF;
    const __nv_bfloat16* res_row =
        (a.residual && row_ok) ? a.residual + (long long)h * a.y_stride + co_base : nullptr;
    uint4 res_nxt[4];
    auto load_line = [&](int c0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) res_nxt[q] = make_uint4(0, 0, 0, 0);
      if (res_row == nullptr) return;
      if (a.wide) {
#pragma unroll
        for (int q = 0; q < 4; q += 2)
          if (c0 + 8 * q < a.row_elems) ld_global_32B(res_row + c0 + 8 * q, res_nxt[q], res_nxt[q + 1]);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (c0 + 8 * q < a.row_elems)
            res_nxt[q] = *reinterpret_cast<const uint4*>(res_row + c0 + 8 * q);
      }
    };
    load_line(0);
    if (alive) alive = mbar_wait(smem_u32(accum), 0, abort_flag, a.status, kErrAccumWait);
    alive = __all_sync(0xffffffffu, alive);   // tcgen05.ld is warp-collective: decide per warp
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    if (alive) {
      __nv_bfloat16* y_row = a.y + (long long)h * a.y_stride + co_base;
      const bool has_sb = a.scale != nullptr || a.bias != nullptr;
      const bool scatter = GENERAL && a.scatter_child != nullptr;
      for (int c0 = 0; c0 < a.npad; c0 += 32) {
        uint4 res_cur[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) res_cur[q] = res_nxt[q];
        if (c0 + 32 < a.npad) load_line(c0 + 32);
        // both 16-column reads of the line are in flight before the one wait
        uint32_t v2[2][16];
        tmem_ld16(lane_base + (uint32_t)c0, v2[0]);
        if (c0 + 16 < a.npad) tmem_ld16(lane_base + (uint32_t)(c0 + 16), v2[1]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int step = 0; step < 2; ++step) {
          const int n0 = c0 + 16 * step;
          if (n0 >= a.npad) break;
          const uint32_t (&v)[16] = v2[step];
          uint4 ov[2];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int n = n0 + 8 * half;
            if (!row_ok || n >= a.row_elems) continue;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[8 * half + j]);
            if (has_sb) {
              const float4 sc0 = *reinterpret_cast<const float4*>(s_scale + n);
              const float4 sc1 = *reinterpret_cast<const float4*>(s_scale + n + 4);
              const float4 bi0 = *reinterpret_cast<const float4*>(s_bias + n);
              const float4 bi1 = *reinterpret_cast<const float4*>(s_bias + n + 4);
              const float sc[8] = {sc0.x, sc0.y, sc0.z, sc0.w, sc1.x, sc1.y, sc1.z, sc1.w};
              const float bi[8] = {bi0.x, bi0.y, bi0.z, bi0.w, bi1.x, bi1.y, bi1.z, bi1.w};
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], sc[j], bi[j]);
            }
            if (res_row != nullptr) {
              const uint32_t* rp = reinterpret_cast<const uint32_t*>(&res_cur[2 * step + half]);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 rf = unpack2(rp[j], f16);
                f[2 * j] += rf.x;
                f[2 * j + 1] += rf.y;
              }
            }
            if (a.relu) {
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
            }
            uint32_t* op = reinterpret_cast<uint32_t*>(&ov[half]);
#pragma unroll
            for (int j = 0; j < 4; ++j) op[j] = pack2(f[2 * j], f[2 * j + 1], f16);
            if (scatter) {
              // column (co_base + n) = octant * Cout + channel of this parent's children; the child
              // of octant o lives in row scatter_child[8h + o] of the output (if it is non-empty)
              const int ng = co_base + n;
              const int o = ng / a.expand_cout;
              const int dst = a.scatter_child[((long long)h << 3) + o];
              if (dst >= 0)
                *reinterpret_cast<uint4*>(a.y + (long long)dst * a.expand_cout + (ng - o * a.expand_cout)) =
                    ov[half];
            } else if (!a.wide) {
              *reinterpret_cast<uint4*>(y_row + n) = ov[half];
            }
          }
          if (a.wide && !scatter && row_ok && n0 < a.row_elems) st_global_32B(y_row + n0, ov[0], ov[1]);
        }
      }
    }
  } else if (warp == 4) {
    // ---------------- MMA issue: one thread ----------------
    if (lane == 0) {
      // instruction descriptor: D = F32 (bit 4), A = B = BF16 (bits 7, 10), both K-major,
      // N >> 3 at bit 17, M >> 4 at bit 24
      // (A/B format field: 0 = F16, 1 = BF16)
      const uint32_t ab = HALF ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (ab << 7) | (ab << 10) | ((uint32_t)(a.npad >> 3) << 17) |
                             ((uint32_t)(kTileM >> 4) << 24);
      bool alive = true;
      int s = 0;
      uint32_t pf = 0;
      for (int kb = 0; kb < a.nkb && alive; ++kb) {
        alive = mbar_wait(smem_u32(&full[s]), pf, abort_flag, a.status, kErrFullWait);
        if (!alive) break;
        // the gathered bytes were written through the generic proxy (cp.async) and have been
        // observed through the mbarrier; the tensor core reads shared memory through the async
        // proxy, so order the two before issuing
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(sA + s * kStageA);
        const uint32_t b_addr = smem_u32(sB + s * stage_b);
#pragma unroll
        for (int k4 = 0; k4 < kBlockK / 16; ++k4) {
          umma_bf16(tmem_base, smem_desc_sw128(a_addr + k4 * 32), smem_desc_sw128(b_addr + k4 * 32),
                    idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&empty[s]));     // stage reusable once these MMAs retire
        if (++s == a.stages) { s = 0; pf ^= 1u; }
      }
      umma_commit(smem_u32(accum));
      if (!alive) {
        // gave up: nobody may be waiting on `accum` any more; make sure the MMAs already issued have
        // retired before TMEM is freed
        for (unsigned it = 0; it < kSpinLimit; ++it)
          if (mbar_try_wait(smem_u32(accum), 0)) break;
      }
    }
  } else {
    // ---------------- weight tiles: one thread, one bulk copy per K-block ----------------
    // Every CTA streams the same nkb tiles in the same order, so on a cold L2 each tile would be a
    // DRAM miss that all CTAs of the wave wait for, one ring turn after the other.  The CTAs of the
    // first wave therefore start by asking L2 for the whole weight image, each for its own
    // share of the tiles.
    {
      const int wave = gridDim.x < kSMs ? (int)gridDim.x : kSMs;
      if ((int)blockIdx.x < wave) {
        for (int kb = blockIdx.x + lane * wave; kb < a.nkb; kb += 32 * wave)
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(wpacked + (size_t)kb * stage_b),
                       "r"((uint32_t)stage_b)
                       : "memory");
      }
    }
    if (lane == 0) {
      bool alive = true;
      int s = 0;
      uint32_t pe = 1;
      for (int kb = 0; kb < a.nkb && alive; ++kb) {
        if (kb >= a.stages)
          alive = mbar_wait(smem_u32(&empty[s]), pe, abort_flag, a.status, kErrWeightWait);
        if (!alive) break;
        const uint32_t bar = smem_u32(&full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)stage_b);
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
            ::"r"(smem_u32(sB + s * stage_b)), "l"(wpacked + (size_t)kb * stage_b),
              "r"((uint32_t)stage_b), "r"(bar)
            : "memory");
        if (++s == a.stages) { s = 0; pe ^= 1u; }
      }
      if (!alive) {
        // gave up with up to `stages` bulk copies in flight into this CTA's shared memory: they
        // complete on their own; leave them time to (bounded) before the CTA exits
        for (int it = 0; it < 64; ++it) __nanosleep(1000);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)a.tmem_cols)
                 : "memory");
  }
}

// ---- persistent variant ------------------------------------------------------------------------
// For layers whose Cin is a multiple of 64 (whole-row gathers) on levels of many tiles.  While an
// MMA runs it reads its A and B slices from shared memory at about the rate shared memory can
// deliver (M = N = 128, K = 16: 8 KB in 64 cycles), and every byte it reads was written there
// once by the gather or the weight copy, so with one 128-row tile per weight tile the tensor pipe
// cannot be busy more than about half of the time.  This variant computes R = 2 tiles of 128 rows
// against every weight tile (B is written once per 256 rows: a third less shared-memory traffic
// per flop at Cout = 128), which needs all of an SM: one CTA per SM walks many 256-row tiles
// (tile = blockIdx.x, += gridDim.x) and overlaps everything inside itself.  Set-up (barriers,
// TMEM, scale / bias) happens once; the accumulator set is double buffered in TMEM where it fits
// and four extra warps run the epilogue, so tile i's TMEM read-out, scale / bias / residual /
// ReLU and stores run under tile i+1's gathers and MMAs.  Roles (32 * (4R + 6) threads): warps
// 0 .. 4R-1 fill the tile's neighbour table and gather A (warp w: rows 32w .. 32w+31); warp 4R
// lane 0 issues the MMAs; warp 4R+1 lane 0 streams the weight tiles; the last four warps are the
// epilogue (TMEM lane quarter = warp & 3).  The {A, B} ring and its phase bits run on across
// tiles; tfull[b] / tempty[b] hand accumulator set b between the MMA thread and the epilogue.
// Same packed weights and the same whole-row gather mapping as conv_tc_kernel's rowsplit 2.
//
// The sibling-group layers with 8 or 16 channels run here too on levels of many tiles (R = 1: a
// tile is 128 groups): the one-tile kernel's CTA spends most of its life in set-up, the latency of
// its first gathers and weight tiles and its 64- to 256-column epilogue, none of which overlaps
// anything of its own.  Their gather is conv_tc_kernel's rowsplit 1 (lane = row within four,
// chunk; indices straight from the groups' neighbour blocks), the indices of four K-blocks read
// ahead of the copies, across tile boundaries.
template <int R>
__device__ __forceinline__ void gather_bar() {
  asm volatile("bar.sync 1, %0;" ::"n"(128 * R) : "memory");
}

template <int CPT, bool HALF, int R>
__global__ void __launch_bounds__(32 * (4 * R + 6), 1) conv_tc_persist_kernel(const TcArgs a, const int ntiles,
                                                                             const int acc_bufs) {
  constexpr int kRows = kTileM * R;              // rows of one tile
  constexpr int kGatherWarps = 4 * R;
  constexpr int kThreadsP = 32 * (4 * R + 6);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stage_b = a.npad * 128;
  uint8_t* sA = smem;                            // stage s: R sub-tiles of 128 rows back to back
  uint8_t* sB = sA + a.stages * (R * kStageA);
  int* nbr = reinterpret_cast<int*>(sB + a.stages * stage_b);      // [taps][kRows]
  float* s_scale = reinterpret_cast<float*>(nbr + (a.group ? 0 : a.T * kRows));   // group mode: no table
  float* s_bias = s_scale + a.npad;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + a.npad);
  uint64_t* full = bars;
  uint64_t* empty = bars + a.stages;
  uint64_t* tfull = bars + 2 * a.stages;
  uint64_t* tempty = tfull + 2;
  uint64_t* wfull = tempty + 2;                  // single K-block: the one weight tile has landed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(wfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int co_base = blockIdx.y * a.cout;
  const uint8_t* wpacked = a.wpacked + (size_t)blockIdx.y * a.nkb * (a.npad * 128);
  const int acc_cols = R * a.tmem_cols;          // TMEM columns of one accumulator set
  // A layer of one K-block (a 1x1x1 layer on 64 channels) uses the same weight tile for every
  // tile of rows: it is fetched once into slot 0 of the B ring and stays there.
  const bool b_resident = a.nkb == 1;
  grid_dependency_trigger();

  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(&full[s]), b_resident ? kRows : kRows + 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull[b]), 1);
      mbar_init(smem_u32(&tempty[b]), kTileM);
    }
    mbar_init(smem_u32(wfull), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kGatherWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_holder)), "r"((uint32_t)(acc_cols * acc_bufs))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  grid_dependency_wait();
  for (int n = tid; n < a.npad; n += kThreadsP) {
    const bool live = n < a.row_elems;
    const int co = a.group ? (n & (a.cout - 1)) : (a.fold_cout ? n % a.fold_cout : co_base + n);
    s_scale[n] = (live && a.scale) ? a.scale[co] : 1.f;
    s_bias[n] = (live && a.bias) ? a.bias[co] : 0.f;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  if (warp < kGatherWarps) {
    // ---------------- neighbour table + A gather, tile after tile ----------------
    bool alive = true;
    int s = 0;
    uint32_t pe = 1;
    long long gk = 0;                  // K-blocks issued so far by this CTA (all tiles)
    const char* xb = reinterpret_cast<const char*>(a.x);
    const uint32_t row_bytes = (uint32_t)a.cin * 2u;
    const int kBlocksPerTap = CPT >= 8 ? CPT / 8 : a.cin >> 6;
    const int sub = lane >> 3, chunk = lane & 7;
    const int rbase = warp * 32 + sub;             // this thread gathers rows rbase + 4i, i = 0..7
    // table slot of row tid: the eight rows of one gather thread sit side by side
    const int slot = (tid & ~31) + ((tid & 3) << 3) + ((tid >> 2) & 7);
    const int* my_idx = nbr + warp * 32 + sub * 8;
    if (a.group) {
      // Sibling-group mode with 8 or 16 channels: chunk `chunk` of K-block kb of tile row g is (a
      // piece of) the row of the node at one position of group g's 4x4x4 neighbour block.  The
      // indices come straight from the block in global memory, one K-block ahead of the copies,
      // across tile boundaries too: the (tile, K-block) sequence of a CTA is one continuous stream.
      const int cpt = a.cin >> 3;
      // The neighbour blocks stream from HBM, so an index read takes longer than a K-block's
      // copies: the indices are read four K-blocks at a time, one such batch ahead of the copies
      // (the host only sends layers here whose K-block count is a multiple of four).
      constexpr int kAhead = 4;
      auto fetch = [&](int tile, int kb0, int (&p)[kAhead][8], uint32_t (&off)[kAhead]) {
#pragma unroll
        for (int j = 0; j < kAhead; ++j) {
          int t;
          chunk_src<CPT>(cpt, kb0 + j, chunk, t, off[j]);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int g = tile * kRows + rbase + 4 * i;
            p[j][i] = -1;
            if (t < a.T && g < a.rows) p[j][i] = __ldg(a.neigh + ((long long)g << 6) + t);
          }
        }
      };
      int tile = blockIdx.x, kb0 = 0;
      int p_cur[kAhead][8];
      uint32_t off_cur[kAhead];
      if (tile < ntiles) fetch(tile, 0, p_cur, off_cur);
      while (tile < ntiles) {
        int tile_nxt = tile, kb_nxt = kb0 + kAhead;
        if (kb_nxt >= a.nkb) { kb_nxt = 0; tile_nxt += gridDim.x; }
        int p_nxt[kAhead][8];
        uint32_t off_nxt[kAhead];
#pragma unroll
        for (int j = 0; j < kAhead; ++j) {
          off_nxt[j] = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) p_nxt[j][i] = -1;
        }
        if (tile_nxt < ntiles) fetch(tile_nxt, kb_nxt, p_nxt, off_nxt);
#pragma unroll
        for (int j = 0; j < kAhead; ++j) {
          if (alive && gk >= a.stages)
            alive = mbar_wait(smem_u32(&empty[s]), pe, abort_flag, a.status, kErrEmptyWait);
          if (alive) {
            const uint32_t stage_base = smem_u32(sA + s * (R * kStageA));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = rbase + 4 * i;
              const uint32_t dst = stage_base + (uint32_t)row * 128u +
                                   (((uint32_t)chunk ^ (uint32_t)(row & 7)) << 4);
              const int pi = p_cur[j][i];
              const char* src = pi >= 0 ? xb + (size_t)((uint32_t)pi * row_bytes) + off_cur[j] : xb;
              // rows past the level's last group are left as they are: their accumulator lanes
              // are never read
              if (tile * kRows + row < a.rows) cp_async16(dst, src, pi >= 0 ? 16u : 0u);
            }
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[s]))
                       : "memory");
          if (++s == a.stages) { s = 0; pe ^= 1u; }
          ++gk;
        }
#pragma unroll
        for (int j = 0; j < kAhead; ++j) {
          off_cur[j] = off_nxt[j];
#pragma unroll
          for (int i = 0; i < 8; ++i) p_cur[j][i] = p_nxt[j][i];
        }
        tile = tile_nxt;
        kb0 = kb_nxt;
      }
    } else
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
      const int h0 = tile * kRows;
      // 1x1x1: a tile row reads its own row, no table and no barriers
      if (!a.identity) {
      gather_bar<R>();                 // every gather thread has finished reading the previous table
      {
        const int h = h0 + tid;
        const bool live = h < a.rows;
        const int hn = (a.ichild != nullptr && live) ? a.ichild[h] : h;
        const int oct_code = ((hn & 4) << 2) | ((hn & 2) << 1) | (hn & 1);
        {
          int pv[27];
#pragma unroll
          for (int t = 0; t < 27; ++t) {
            int p = -1;
            if (t < a.T && live) {
              const long long at = a.stride == 2 ? ((long long)hn << 6) + a.tap[t]
                                                 : ((long long)(hn >> 3) << 6) + a.tap[t] + oct_code;
              p = a.neigh[at];
            }
            pv[t] = p;
          }
          if (a.child != nullptr) {
#pragma unroll
            for (int t = 0; t < 27; ++t)
              if (t < a.T && pv[t] >= 0) pv[t] = a.child[pv[t]];
          }
#pragma unroll
          for (int t = 0; t < 27; ++t)
            if (t < a.T) nbr[t * kRows + slot] = pv[t];
        }
      }
      gather_bar<R>();
      }

      uint32_t row_mask = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (h0 + rbase + 4 * i < a.rows) row_mask |= 1u << i;
      int p[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) p[i] = h0 + rbase + 4 * i;      // (identity; masked rows are not copied)
      int t = 0, part = 0;
      for (int kb = 0; kb < a.nkb; ++kb, ++gk) {
        if (part == 0 && !a.identity) {
          const int4 lo = *reinterpret_cast<const int4*>(my_idx + t * kRows);
          const int4 hi = *reinterpret_cast<const int4*>(my_idx + t * kRows + 4);
          p[0] = lo.x; p[1] = lo.y; p[2] = lo.z; p[3] = lo.w;
          p[4] = hi.x; p[5] = hi.y; p[6] = hi.z; p[7] = hi.w;
        }
        if (alive && gk >= a.stages)
          alive = mbar_wait(smem_u32(&empty[s]), pe, abort_flag, a.status, kErrEmptyWait);
        bool paired = false;
        if constexpr (CPT == 0) paired = a.x2 != nullptr;
        if (alive && paired) {
          // two-input 1x1x1 layer: chunk g of a node's K row is chunk g of its row of x while
          // g < cpt_a, chunk g - cpt_a of its row of x2 after that, zeros beyond Cin
          const uint32_t stage_base = smem_u32(sA + s * (R * kStageA));
          const uint32_t g = (uint32_t)kb * 8u + (uint32_t)chunk;
          const uint32_t cpt_all = (uint32_t)a.cin >> 3, cpt_a = (uint32_t)a.cpt_a;
          const bool from_a = g < cpt_a, live = g < cpt_all;
          const char* base = from_a ? xb : reinterpret_cast<const char*>(a.x2);
          const uint32_t rb = (from_a ? cpt_a : cpt_all - cpt_a) * 16u;
          const uint32_t off = (from_a ? g : g - cpt_a) * 16u;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = rbase + 4 * i;
            const uint32_t dst = stage_base + (uint32_t)row * 128u +
                                 (((uint32_t)chunk ^ (uint32_t)(row & 7)) << 4);
            const char* src = live ? base + (size_t)p[i] * rb + off : xb;
            if ((row_mask >> i) & 1u) cp_async16(dst, src, live ? 16u : 0u);
          }
        } else if (alive) {
          const uint32_t stage_base = smem_u32(sA + s * (R * kStageA));
          const uint32_t off = (uint32_t)part * 128u + (uint32_t)chunk * 16u;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = rbase + 4 * i;
            const uint32_t dst = stage_base + (uint32_t)row * 128u +
                                 (((uint32_t)chunk ^ (uint32_t)(row & 7)) << 4);
            const int pi = p[i];
            const char* src = pi >= 0 ? xb + (size_t)((uint32_t)pi * row_bytes) + off : xb;
            if ((row_mask >> i) & 1u) cp_async16(dst, src, pi >= 0 ? 16u : 0u);
          }
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[s]))
                     : "memory");
        if (++s == a.stages) { s = 0; pe ^= 1u; }
        if (++part == kBlocksPerTap) { part = 0; ++t; }
      }
      // a thread that gave up keeps walking the tiles (without waiting or copying): the named
      // barrier above needs every gather thread every time
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == kGatherWarps) {
    // ---------------- MMA issue: one thread ----------------
    if (lane == 0) {
      const uint32_t ab = HALF ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (ab << 7) | (ab << 10) | ((uint32_t)(a.npad >> 3) << 17) |
                             ((uint32_t)(kTileM >> 4) << 24);
      bool alive = true;
      int s = 0;
      uint32_t pf = 0;
      int it = 0;
      if (b_resident) alive = mbar_wait(smem_u32(wfull), 0, abort_flag, a.status, kErrWeightWait);
      for (int tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++it) {
        const int b = it % acc_bufs;
        const uint32_t use = (uint32_t)(it / acc_bufs);
        // the epilogue must have drained accumulator set b (first use: passes at once)
        alive = mbar_wait(smem_u32(&tempty[b]), (use & 1u) ^ 1u, abort_flag, a.status, kErrAccumWait);
        if (!alive) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(b * acc_cols);
        for (int kb = 0; kb < a.nkb && alive; ++kb) {
          alive = mbar_wait(smem_u32(&full[s]), pf, abort_flag, a.status, kErrFullWait);
          if (!alive) break;
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(sA + s * (R * kStageA));
          const uint32_t b_addr = smem_u32(sB + (b_resident ? 0 : s * stage_b));
#pragma unroll
          for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int k4 = 0; k4 < kBlockK / 16; ++k4) {
              umma_bf16(tmem_d + (uint32_t)(r * a.tmem_cols), smem_desc_sw128(a_addr + r * kStageA + k4 * 32),
                        smem_desc_sw128(b_addr + k4 * 32), idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&empty[s]));
          if (++s == a.stages) { s = 0; pf ^= 1u; }
        }
        umma_commit(smem_u32(&tfull[b]));
      }
      if (!alive) {
        // gave up: wait (bounded) until the MMAs already issued have retired before TMEM is freed
        umma_commit(smem_u32(&tfull[0]));
        for (int w = 0; w < 64; ++w) __nanosleep(1000);
      }
    }
  } else if (warp == kGatherWarps + 1) {
    // ---------------- weight tiles ----------------
    {
      const int wave = gridDim.x < kSMs ? (int)gridDim.x : kSMs;
      if ((int)blockIdx.x < wave) {
        for (int kb = blockIdx.x + lane * wave; kb < a.nkb; kb += 32 * wave)
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(wpacked + (size_t)kb * stage_b),
                       "r"((uint32_t)stage_b)
                       : "memory");
      }
    }
    if (lane == 0 && b_resident) {
      const uint32_t bar = smem_u32(wfull);
      mbar_arrive_expect_tx(bar, (uint32_t)stage_b);
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
          ::"r"(smem_u32(sB)), "l"(wpacked), "r"((uint32_t)stage_b), "r"(bar)
          : "memory");
      // stay until it has landed (bounded): the CTA must not retire under the copy
      mbar_wait(bar, 0, abort_flag, a.status, kErrWeightWait);
    } else if (lane == 0) {
      bool alive = true;
      int s = 0;
      uint32_t pe = 1;
      long long gk = 0;
      for (int tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
        for (int kb = 0; kb < a.nkb && alive; ++kb, ++gk) {
          if (gk >= a.stages)
            alive = mbar_wait(smem_u32(&empty[s]), pe, abort_flag, a.status, kErrWeightWait);
          if (!alive) break;
          const uint32_t bar = smem_u32(&full[s]);
          mbar_arrive_expect_tx(bar, (uint32_t)stage_b);
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
              ::"r"(smem_u32(sB + s * stage_b)), "l"(wpacked + (size_t)kb * stage_b),
                "r"((uint32_t)stage_b), "r"(bar)
              : "memory");
          if (++s == a.stages) { s = 0; pe ^= 1u; }
        }
      }
      if (!alive) {
        for (int w = 0; w < 64; ++w) __nanosleep(1000);
      }
    }
  } else {
    // ---------------- epilogue warps: TMEM -> registers -> global, tile after tile ----------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    constexpr bool f16 = HALF;
    bool alive = true;
    const bool has_sb = a.scale != nullptr || a.bias != nullptr;
    int it = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int b = it % acc_bufs;
      const uint32_t use = (uint32_t)(it / acc_bufs);
      alive = mbar_wait(smem_u32(&tfull[b]), use & 1u, abort_flag, a.status, kErrAccumWait);
      alive = __all_sync(0xffffffffu, alive);
      if (!alive) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int r = 0; r < R; ++r) {
        const int h = tile * kRows + r * kTileM + q * 32 + lane;
        const bool row_ok = h < a.rows;
        const __nv_bfloat16* res_row =
            (a.residual && row_ok) ? a.residual + (long long)h * a.y_stride + co_base : nullptr;
        uint4 res_nxt[4];
        auto load_line = [&](int c0) {
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) res_nxt[qq] = make_uint4(0, 0, 0, 0);
          if (res_row == nullptr) return;
          if (a.wide) {
#pragma unroll
            for (int qq = 0; qq < 4; qq += 2)
              if (c0 + 8 * qq < a.row_elems) ld_global_32B(res_row + c0 + 8 * qq, res_nxt[qq], res_nxt[qq + 1]);
          } else {
#pragma unroll
            for (int qq = 0; qq < 4; ++qq)
              if (c0 + 8 * qq < a.row_elems)
                res_nxt[qq] = *reinterpret_cast<const uint4*>(res_row + c0 + 8 * qq);
          }
        };
        load_line(0);
        const uint32_t lane_base = tmem_base + (uint32_t)(b * acc_cols + r * a.tmem_cols) + ((uint32_t)(q * 32) << 16);
        __nv_bfloat16* y_row = a.y + (long long)h * a.y_stride + co_base;
        for (int c0 = 0; c0 < a.npad; c0 += 32) {
          uint4 res_cur[4];
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) res_cur[qq] = res_nxt[qq];
          if (c0 + 32 < a.npad) load_line(c0 + 32);
#pragma unroll
          for (int step = 0; step < 2; ++step) {
            const int n0 = c0 + 16 * step;
            if (n0 >= a.npad) break;
            uint32_t v[16];
            tmem_ld16(lane_base + (uint32_t)n0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            uint4 ov[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int n = n0 + 8 * half;
              if (!row_ok || n >= a.row_elems) continue;
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[8 * half + j]);
              if (has_sb) {
                const float4 sc0 = *reinterpret_cast<const float4*>(s_scale + n);
                const float4 sc1 = *reinterpret_cast<const float4*>(s_scale + n + 4);
                const float4 bi0 = *reinterpret_cast<const float4*>(s_bias + n);
                const float4 bi1 = *reinterpret_cast<const float4*>(s_bias + n + 4);
                const float sc[8] = {sc0.x, sc0.y, sc0.z, sc0.w, sc1.x, sc1.y, sc1.z, sc1.w};
                const float bi[8] = {bi0.x, bi0.y, bi0.z, bi0.w, bi1.x, bi1.y, bi1.z, bi1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], sc[j], bi[j]);
              }
              if (res_row != nullptr) {
                const uint32_t* rp = reinterpret_cast<const uint32_t*>(&res_cur[2 * step + half]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 rf = unpack2(rp[j], f16);
                  f[2 * j] += rf.x;
                  f[2 * j + 1] += rf.y;
                }
              }
              if (a.relu) {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
              }
              uint32_t* op = reinterpret_cast<uint32_t*>(&ov[half]);
#pragma unroll
              for (int j = 0; j < 4; ++j) op[j] = pack2(f[2 * j], f[2 * j + 1], f16);
              if (!a.wide) *reinterpret_cast<uint4*>(y_row + n) = ov[half];
            }
            if (a.wide && row_ok && n0 < a.row_elems) st_global_32B(y_row + n0, ov[0], ov[1]);
          }
        }
      }
      // accumulator set b has been read out: hand it back to the MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(smem_u32(&tempty[b]));
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kGatherWarps) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)(acc_cols * acc_bufs))
                 : "memory");
  }
}

// ---- self-test of the bounded waits -------------------------------------------------------------
// One CTA, two waiting threads, a barrier that nobody ever arrives on: the first waiter must run
// out of polls, write its code to status[0] and raise the abort flag; the second must come back
// from its own wait with "stop" (status[1] = 1).  Exactly the mbar_wait the convolution kernels use.
__global__ void wait_selftest_kernel(int* status) {
  __shared__ uint64_t never;
  __shared__ int abort_flag_s;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&never), 1);
    abort_flag_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  volatile int* abort_flag = &abort_flag_s;
  if (threadIdx.x == 0) {
    mbar_wait(smem_u32(&never), 0, abort_flag, status, kErrFullWait);
  } else if (threadIdx.x == 32) {
    const bool ok = mbar_wait(smem_u32(&never), 0, abort_flag, status, kErrEmptyWait);
    status[1] = ok ? 0 : 1;
  }
}

// ---- weight packing -------------------------------------------------------------------------
// packed: per K-block a [npad x 64] tile of 16-bit floats in the swizzled K-major image: element
// (n, kk) at (n/8)*1024 + (n%8)*128 + (((kk/8) ^ (n%8)) * 16) + (kk%8)*2, k = kb*64 + kk.
// WeightView says where the value of (output column n, input channel ci, tap t) sits in the
// reference's fp32 weight tensor:
//   convolution    w[co, ci*T + t]             (pytorch/ocnn/octree_conv.py:51-58, [Cout, Cin*K])
//   deconvolution  w[ci, co*T + t]             ([Cin, Cout*K])
// and how the kernel-2 stride-2 layers are folded into dense products:
//   fold_in   (convolution):   K index k = o*Cin + ci over the 8 children of a sibling group, tap = o
//   expand_out (deconvolution): column n = o*Cout + co over the 8 children of a parent, tap = o
struct WeightView {
  int cin, cout, T;      // of the layer as the reference sees it
  int transposed;
  int fold_in, expand_out;
  int fold_nodes;        // > 1: 1x1x1 layer on rows of fold_nodes nodes: block-diagonal weights,
                         // K index k = node*Cin + ci, column n = node*Cout + co
  int co_base;           // first output column of this 256-column slice
};

__device__ __forceinline__ float weight_at(const float* __restrict__ w, const WeightView& v, int n,
                                           int ci, int t) {
  return v.transposed ? w[((long long)ci * v.cout + n) * v.T + t]
                      : w[((long long)n * v.cin + ci) * v.T + t];
}

__device__ __forceinline__ void store_packed(uint16_t* __restrict__ packed, long long off, float v,
                                             bool half) {
  if (half) {
    const __half h = __float2half(v);
    packed[off] = *reinterpret_cast<const uint16_t*>(&h);
  } else {
    const __nv_bfloat16 b = __float2bfloat16(v);
    packed[off] = *reinterpret_cast<const uint16_t*>(&b);
  }
}

__global__ void pack_weights_kernel(const float* __restrict__ w, uint16_t* __restrict__ packed,
                                    WeightView v, int ncols, int kdim, int npad, int nkb, bool half) {
  // ncols = output columns of this slice, kdim = K extent (taps * Cin, or 8*Cin when folded)
  const long long total = (long long)nkb * npad * kBlockK;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int kk = (int)(i % kBlockK);
    const int n = (int)((i / kBlockK) % npad);
    const int kb = (int)(i / ((long long)kBlockK * npad));
    const int k = kb * kBlockK + kk;
    float val = 0.f;
    if (n < ncols && k < kdim) {
      const int col = v.co_base + n;
      if (v.fold_nodes > 1) {
        val = (col / v.cout == k / v.cin) ? weight_at(w, v, col % v.cout, k % v.cin, 0) : 0.f;
      } else if (v.expand_out) {
        // column = octant * Cout + channel; the only tap that reaches octant o is tap o
        val = weight_at(w, v, col % v.cout, k, col / v.cout);
      } else {
        // K walks tap-major: k = t*Cin + ci (folded: the "tap" is the child's octant)
        val = weight_at(w, v, col, k % v.cin, k / v.cin);
      }
    }
    const long long off = (long long)kb * npad * 64 + (n >> 3) * 512 + (n & 7) * 64 +
                          (((kk >> 3) ^ (n & 7)) << 3) + (kk & 7);
    store_packed(packed, off, val, half);
  }
}

// Group mode: B[k][n], k = j*cin + ci over the 64 block positions j, n = o*cout + co over the
// 8 octants: W[co, ci*T + t] where tap t of the kernel sits at block position j for octant o
// (j = ((tx+ox)<<4)|((ty+oy)<<2)|(tz+oz)), zero elsewhere.  Same swizzled tile image as above.
struct TapsArg { int count; signed char tap[27]; };

__global__ void pack_weights_group_kernel(const float* __restrict__ w, uint16_t* __restrict__ packed,
                                          int cin, int cout, int T, TapsArg taps, int npad, int nkb,
                                          bool half) {
  const long long total = (long long)nkb * npad * kBlockK;
  const int KD = cin * T;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int kk = (int)(i % kBlockK);
    const int n = (int)((i / kBlockK) % npad);
    const int kb = (int)(i / ((long long)kBlockK * npad));
    const int k = kb * kBlockK + kk;
    const int j = k / cin, ci = k % cin;
    const int o = n / cout, co = n % cout;
    float v = 0.f;
    if (j < 64 && o < 8) {
      const int tx = (j >> 4) - (o >> 2), ty = ((j >> 2) & 3) - ((o >> 1) & 1), tz = (j & 3) - (o & 1);
      if (tx >= 0 && tx < 3 && ty >= 0 && ty < 3 && tz >= 0 && tz < 3) {
        const int tap27 = tx * 9 + ty * 3 + tz;
        for (int t = 0; t < T; ++t)
          if (taps.tap[t] == tap27) v = w[(long long)co * KD + ci * T + t];
      }
    }
    const long long off = (long long)kb * npad * 64 + (n >> 3) * 512 + (n & 7) * 64 +
                          (((kk >> 3) ^ (n & 7)) << 3) + (kk & 7);
    store_packed(packed, off, v, half);
  }
}

// The last h % fold nodes of a folded 1x1x1 layer (a node count that does not fill its last row;
// only data on non-empty nodes can have one): one thread per (node, output channel), weights read
// back from the first diagonal block of the packed image.
template <bool HALF>
__global__ void fold_tail_kernel(const __nv_bfloat16* __restrict__ x, const uint16_t* __restrict__ packed,
                                 __nv_bfloat16* __restrict__ y, long long first, int count, int cin,
                                 int cout, const float* __restrict__ scale, const float* __restrict__ bias,
                                 const __nv_bfloat16* __restrict__ residual, int relu) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count * cout) return;
  const int node = i / cout, co = i % cout;
  const uint16_t* xr = reinterpret_cast<const uint16_t*>(x) + (first + node) * cin;
  float acc = 0.f;
  for (int ci = 0; ci < cin; ++ci) {
    const uint16_t wv = packed[(co >> 3) * 512 + (co & 7) * 64 + (((ci >> 3) ^ (co & 7)) << 3) + (ci & 7)];
    const float2 xf = unpack2((uint32_t)xr[ci], HALF), wf = unpack2((uint32_t)wv, HALF);
    acc = fmaf(xf.x, wf.x, acc);
  }
  if (scale) acc *= scale[co];
  if (bias) acc += bias[co];
  const long long at = (first + node) * cout + co;
  if (residual) acc += unpack2((uint32_t)reinterpret_cast<const uint16_t*>(residual)[at], HALF).x;
  if (relu) acc = fmaxf(acc, 0.f);
  reinterpret_cast<uint16_t*>(y)[at] = (uint16_t)(pack2(acc, 0.f, HALF) & 0xffffu);
}

// What kind of layer a launch serves (the reference's OctreeConv / OctreeDeconv flags).
struct LayerKind {
  int stride;
  bool transposed, nempty;
};

// 0: never fold nodes of 1x1x1 layers into 128-byte rows; 1: fold where it applies (default).
// Read once: the packed weight image depends on it.
int fold_mode() {
  static const int mode = [] {
    const char* e = getenv("OCNN_CONV_FOLD");
    return e ? atoi(e) : 1;
  }();
  return mode;
}

struct TcShape {
  int T, npad, nkb, tmem_cols, stages, group, slices, tile_rows, gtable, ntable_stride;
  int fold_in, expand_out;   // kernel 2, stride 2 as a dense product (see WeightView)
  int fold_nodes;            // 1x1x1 with Cin < 64: 64/Cin nodes per tile row (1 = not folded)
  int cin_eff, cout_eff;     // channel counts the kernel sees: 8*Cin when folded, 8*Cout when expanded
  size_t smem;
  size_t fixed_bytes, stage_bytes;   // shared memory outside the ring / per ring stage
  bool small_grid;                   // the tiles do not fill the SMs once
};

int tc_shape(int cin, int cout, const int ks[3], const LayerKind& kind, TcShape* s,
             long long rows_hint = -1) {
  const TapList tl = taps_for_kernel(ks);
  const int stride = kind.stride;
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "tensor-core convolution: unsupported kernel size %dx%dx%d",
                ks[0], ks[1], ks[2]);
  if (stride != 1 && stride != 2)
    return fail(OCNN_ERR_INVALID, "tensor-core convolution: stride must be 1 or 2 (got %d)", stride);
  if (cin <= 0 || cin % 8 != 0)
    return fail(OCNN_ERR_UNSUPPORTED, "tensor-core convolution: Cin (%d) must be a multiple of 8", cin);
  const bool k222s2 = ks[0] == 2 && ks[1] == 2 && ks[2] == 2 && stride == 2;
  // kernel 2, stride 2: a sibling group's eight children are the whole neighbourhood.  On all nodes
  // the convolution reads them as one contiguous row of 8*Cin channels; the deconvolution writes a
  // parent's eight children as one row of 8*Cout channels (scattered through child on non-empty
  // nodes).  Both are then plain dense products with no gather.
  s->fold_in = (k222s2 && !kind.transposed && !kind.nempty) ? 1 : 0;
  s->expand_out = (k222s2 && kind.transposed && (cout * 8 <= 256 || cout % 32 == 0) && cout * 8 <= 4096) ? 1 : 0;
  // 1x1x1, stride 1, fewer than 64 channels in: a K-block of one node would be mostly padding and
  // a tile of 128 nodes only 128*Cin*2 bytes.  64/Cin consecutive nodes are one 128-byte line, so
  // the layer runs on rows of 64/Cin nodes with block-diagonal weights (K = 64 exactly, N =
  // 64/Cin * Cout): a plain stream of full lines through one K-block per tile.
  s->fold_nodes = 1;
  if (tl.count == 1 && stride == 1 && !kind.transposed && !kind.nempty && cin < 64 && 64 % cin == 0 &&
      cout % 8 == 0 && (64 / cin) * cout <= 256 && fold_mode() != 0)
    s->fold_nodes = 64 / cin;
  s->cin_eff = s->fold_in ? 8 * cin : (s->fold_nodes > 1 ? 64 : cin);
  s->cout_eff = s->expand_out ? 8 * cout : (s->fold_nodes > 1 ? s->fold_nodes * cout : cout);
  cout = s->cout_eff;
  if (cout <= 0 || cout % 8 != 0 || (cout > 256 && cout % 256 != 0) || cout > 4096)
    return fail(OCNN_ERR_UNSUPPORTED,
                "tensor-core convolution: Cout (%d) must be a multiple of 8 up to 256, or a multiple "
                "of 256 up to 4096", cout);
  // more than 256 output channels: produced 256 at a time (one TMEM accumulator is 256 columns)
  s->slices = cout > 256 ? cout / 256 : 1;
  if (s->slices > 1) cout = 256;
  // sibling-group mode: stride 1, a real neighbourhood, few channels (power-of-two Cout so that
  // column -> channel is a mask)
  // (not on non-empty nodes only, nor for the deconvolution: their tile rows are single nodes)
  const bool node_only = kind.nempty || kind.transposed;
  s->group = (!node_only && stride == 1 && tl.count > 1 && cin <= 32 && cout <= 32 && (cout & (cout - 1)) == 0) ? 1 : 0;
  s->T = s->group ? 64 : ((s->fold_in || s->expand_out) ? 1 : tl.count);
  s->npad = s->group ? 8 * cout : (cout + 15) / 16 * 16;
  s->nkb = (s->cin_eff * s->T + kBlockK - 1) / kBlockK;
  s->tmem_cols = 32;
  while (s->tmem_cols < s->npad) s->tmem_cols *= 2;
  // Ring depth.  Prefer a footprint that lets two CTAs share an SM (their set-up and epilogue
  // phases then overlap each other's main loop); otherwise take what one CTA can hold.
  const size_t stage_bytes = (size_t)kStageA + (size_t)s->npad * 128;
  // group mode with more than 16 channels gathers through a shared index table (fewer index reads
  // in the loop); with 8 or 16 channels filling the table costs more than it saves
  s->gtable = (s->group && cin > 16) ? 1 : 0;
  // node mode keeps a [taps][128] index table; Cin not a multiple of 64 reads it per K-block with
  // lanes on different taps, which wants the padded stride
  s->ntable_stride = (!s->group && s->cin_eff % 64 != 0 && s->T > 1) ? kGroupTableStride : kTileM;
  const size_t fixed = 1024 + (s->group ? (s->gtable ? 64 * kGroupTableStride * 4 : 0) : (size_t)s->T * s->ntable_stride * 4) +
                       (size_t)s->npad * 8 + 256;
  const size_t two_cta = 112 * 1024, one_cta = 200 * 1024;
  // every stage of the ring can be in flight at once, so prefer two CTAs per SM (set-up and
  // epilogue of one overlap the main loop of the other) whenever each still gets 2 stages
  int st = two_cta > fixed ? (int)((two_cta - fixed) / stage_bytes) : 0;
  // a grid that does not even fill the SMs once gains nothing from co-residency: give the lone CTA
  // of each SM the deepest ring instead (its K loop is a pure latency chain)
  const long long rows = rows_hint < 0 ? -1 : (s->group ? rows_hint / 8 : rows_hint / s->fold_nodes);
  // A level too small to give even half of the SMs a 128-row tile is cut into 64- or 32-row
  // tiles: the gather is then spread over more SMs.  Every CTA still streams the whole weight
  // image, so halving stops where a K-block's gather (about 8 cycles per row of 16-byte copies)
  // is no longer above its weight tile (about 3.2 cycles per 128-byte row).
  s->tile_rows = kTileM;
  const int sms = rows >= 0 ? sm_count() : kSMs;
  while (rows >= 0 && s->tile_rows > 32 && 2 * ((rows + s->tile_rows - 1) / s->tile_rows) <= sms &&
         8.0 * s->tile_rows > 3.2 * s->npad)
    s->tile_rows >>= 1;
  const bool small_grid = rows >= 0 && (rows + s->tile_rows - 1) / s->tile_rows <= sms;
  if (st < 2 || 2 * s->tmem_cols > 512 || small_grid) {
    st = (int)((one_cta - fixed) / stage_bytes);
    if (st > 7) st = 7;
  } else if (st > 6) {
    st = 6;
  }
  // Where two stages fit three times into an SM (and the accumulators into TMEM), three CTAs with
  // a two-stage ring each beat two CTAs with deeper rings: more set-up and epilogue phases overlap
  // the others' main loops (8->8: 0.050 -> 0.042 ms, 64->64: 0.417 -> 0.351 ms at 931 k nodes).
  const size_t three_cta = 74 * 1024;
  // (a level with at most two tiles per SM never has three CTAs on an SM: it keeps the deeper ring)
  // (depth-5 3x3x3 16 -> 16 of the benchmark: 0.026 -> 0.024 ms in the step's trace)
  const bool two_per_sm = rows >= 0 && (rows + s->tile_rows - 1) / s->tile_rows <= 2 * sms;
  if (!small_grid && !two_per_sm && st > 2 && fixed + 2 * stage_bytes <= three_cta && 3 * s->tmem_cols <= 512)
    st = 2;
  if (st > s->nkb) st = s->nkb < 2 ? 2 : s->nkb;
  s->stages = st;
  s->smem = fixed + (size_t)s->stages * stage_bytes;
  s->fixed_bytes = fixed;
  s->stage_bytes = stage_bytes;
  s->small_grid = small_grid;
  return OCNN_OK;
}

// 0: one tile per CTA always; 1: the persistent kernel where it pays (default).
int persist_mode() {
  static const int mode = [] {
    const char* e = getenv("OCNN_CONV_PERSIST");
    return e ? atoi(e) : 1;
  }();
  return mode;
}

// 0: few-channel sibling-group layers always on the one-tile kernel; 1: persistent on big levels.
int persist_group_mode() {
  static const int mode = [] {
    const char* e = getenv("OCNN_CONV_PERSIST_GROUP");
    return e ? atoi(e) : (persist_mode() != 0 ? 1 : 0);
  }();
  return mode;
}

// Launch shape of the persistent kernel: 128-row tiles per weight tile, ring depth, accumulator
// sets in TMEM, dynamic shared memory.  stages == 0: it does not fit.
struct PersistShape {
  int R, stages, acc_bufs;
  size_t smem;
};

PersistShape persist_shape(const TcShape& s, int R) {
  PersistShape p;
  p.R = R;
  p.acc_bufs = 2 * R * s.tmem_cols <= 512 ? 2 : 1;
  const size_t budget = 226 * 1024;           // one CTA per SM
  const size_t fixed = 1024 + (s.group ? 0 : (size_t)s.T * 128 * R * 4) + (size_t)s.npad * 8 + 256;
  const size_t stage = (size_t)R * kStageA + (size_t)s.npad * 128;
  int st = budget > fixed ? (int)((budget - fixed) / stage) : 0;
  if (st > 8) st = 8;
  if (st < 3 || R * s.tmem_cols > 512) st = 0;
  p.stages = st;
  p.smem = fixed + (size_t)st * stage;
  return p;
}

size_t packed_bytes_impl(int cin, int cout, const int kernel_size[3], const LayerKind& kind) {
  TcShape s;
  if (kernel_size == nullptr || tc_shape(cin, cout, kernel_size, kind, &s, -1) != OCNN_OK) return 0;
  return (size_t)s.slices * s.nkb * s.npad * 128;
}

int pack_weights_impl(const float* w, void* packed, int cin, int cout, const int kernel_size[3],
                      const LayerKind& kind, int dtype, void* stream) {
  OCNN_REQUIRE(w && packed && kernel_size, "ocnn_conv_pack_weights: null pointer");
  OCNN_REQUIRE(dtype == OCNN_BF16 || dtype == OCNN_F16,
               "ocnn_conv_pack_weights: the tensor-core kernel takes bf16 or fp16 (dtype %d given)", dtype);
  TcShape s;
  if (int st = tc_shape(cin, cout, kernel_size, kind, &s, -1)) return st;
  const long long total = (long long)s.nkb * s.npad * kBlockK;
  const bool half = dtype == OCNN_F16;
  const TapList tl = taps_for_kernel(kernel_size);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (s.group) {
    TapsArg ta;
    ta.count = tl.count;
    for (int i = 0; i < 27; ++i) ta.tap[i] = i < tl.count ? tl.tap[i] : -1;
    pack_weights_group_kernel<<<grid_for(total, 256), 256, 0, st>>>(
        w, static_cast<uint16_t*>(packed), cin, cout, tl.count, ta, s.npad, s.nkb, half);
  } else {
    // one packed image per slice of (at most) 256 output columns
    WeightView v;
    v.cin = cin; v.cout = cout; v.T = tl.count; v.transposed = kind.transposed ? 1 : 0;
    v.fold_in = s.fold_in; v.expand_out = s.expand_out; v.fold_nodes = s.fold_nodes;
    const int cslice = s.slices > 1 ? 256 : s.cout_eff;
    const int kdim = s.cin_eff * s.T;
    for (int sl = 0; sl < s.slices; ++sl) {
      v.co_base = sl * cslice;
      pack_weights_kernel<<<grid_for(total, 256), 256, 0, st>>>(
          w, static_cast<uint16_t*>(packed) + (size_t)sl * total, v, cslice, kdim, s.npad, s.nkb, half);
      if (sl > 0) note_launches(1);
    }
  }
  OCNN_LAUNCH_OK("pack_weights_kernel");
  return OCNN_OK;
}

int conv_tc_impl(const void* x, const void* packed, void* y, const ocnn_conv_geometry* g, int cin,
                 int cout, const int kernel_size[3], int dtype, const ocnn_conv_epilogue* ep,
                 int32_t* status, void* stream, const char* who, const void* x2 = nullptr,
                 int cin_a = 0) {
  OCNN_REQUIRE(kernel_size != nullptr, "%s: null kernel size", who);
  OCNN_REQUIRE(dtype == OCNN_BF16 || dtype == OCNN_F16, "%s: bf16 or fp16 data only (dtype %d)", who, dtype);
  const TapList tl = taps_for_kernel(kernel_size);
  if (tl.count < 0)
    return fail(OCNN_ERR_UNSUPPORTED, "%s: unsupported kernel size %dx%dx%d", who, kernel_size[0],
                kernel_size[1], kernel_size[2]);
  if (int rc = check_conv_geometry(g, tl, who)) return rc;
  const int stride = g->stride;
  const LayerKind kind{stride, g->transposed != 0, g->nempty != 0};
  const int h_in = g->h_in, h_out = g->h_out;
  TcShape s;
  // tile rows: output rows, except parents for the expanded kernel-2 deconvolution
  {
    TcShape probe;
    if (int st = tc_shape(cin, cout, kernel_size, kind, &probe, -1)) return st;
    if (int st = tc_shape(cin, cout, kernel_size, kind, &s, probe.expand_out ? h_in : h_out)) return st;
  }
  if (h_out == 0 || (s.expand_out && h_in == 0)) return OCNN_OK;
  const bool identity = s.T == 1 && (stride == 1 || s.fold_in || s.expand_out);
  OCNN_REQUIRE(x && packed && y && status, "%s: null pointer", who);
  OCNN_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) && ((uintptr_t)packed % 16 == 0),
               "%s: data and weight pointers must be 16-byte aligned", who);
  if (ep && ep->residual_dev)
    OCNN_REQUIRE((uintptr_t)ep->residual_dev % 16 == 0, "%s: residual must be 16-byte aligned", who);
  const bool scatter = s.expand_out && g->nempty;
  if (scatter) {
    OCNN_REQUIRE(g->child_dev != nullptr, "%s: child array of the finer level required", who);
    OCNN_REQUIRE(!(ep && ep->residual_dev), "%s: no residual on a scattered deconvolution", who);
  }
  if (x2 != nullptr && identity && !g->nempty && !g->transposed && s.fold_nodes == 1 && s.slices == 1 &&
      cin_a > 0 && cin_a < cin) {
    // few channels on a big level: the streaming kernel, on the same packed weights
    const int rc = conv_pointwise_pair_packed(x, cin_a, x2, cin - cin_a, packed, s.npad, y, h_out, cout, ep,
                                              static_cast<cudaStream_t>(stream), dtype == OCNN_F16);
    if (rc != -1) return rc;
  }
  TcArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.x2 = static_cast<const __nv_bfloat16*>(x2);
  a.cpt_a = x2 != nullptr ? cin_a / 8 : 0;
  if (x2 != nullptr) {
    OCNN_REQUIRE(identity && !g->nempty && !g->transposed && s.fold_nodes == 1 && !s.fold_in && !s.expand_out,
                 "%s: two inputs only for a plain 1x1x1 stride-1 layer", who);
    OCNN_REQUIRE(cin_a > 0 && cin_a < cin && cin_a % 8 == 0 && (uintptr_t)x2 % 16 == 0,
                 "%s: input channel split %d + %d must be multiples of 8, pointers 16-byte aligned", who,
                 cin_a, cin - cin_a);
  }
  a.wpacked = static_cast<const uint8_t*>(packed);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.neigh = identity ? nullptr : g->neigh_dev;
  const bool plain_gather = !identity && !s.fold_in && !s.expand_out;
  a.child = (plain_gather && g->nempty && !(kind.transposed && stride == 2)) ? g->child_dev : nullptr;
  a.ichild = (plain_gather && g->nempty && !(stride == 2 && !kind.transposed)) ? g->ichild_dev : nullptr;
  a.up = (plain_gather && kind.transposed && stride == 2) ? 1 : 0;
  a.f16 = dtype == OCNN_F16 ? 1 : 0;
  a.expand_cout = s.expand_out ? cout : 0;
  a.fold_cout = s.fold_nodes > 1 ? cout : 0;
  const int fold_tail = s.fold_nodes > 1 ? h_out % s.fold_nodes : 0;
  if (fold_tail > 0) {
    // the nodes that do not fill a row
    const long long first = h_out - fold_tail;
    const int threads = fold_tail * cout;
    if (dtype == OCNN_F16)
      fold_tail_kernel<true><<<ceil_div(threads, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<const uint16_t*>(packed),
          static_cast<__nv_bfloat16*>(y), first, fold_tail, cin, cout, ep ? ep->scale_dev : nullptr,
          ep ? ep->bias_dev : nullptr, ep ? static_cast<const __nv_bfloat16*>(ep->residual_dev) : nullptr,
          ep ? ep->relu : 0);
    else
      fold_tail_kernel<false><<<ceil_div(threads, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<const uint16_t*>(packed),
          static_cast<__nv_bfloat16*>(y), first, fold_tail, cin, cout, ep ? ep->scale_dev : nullptr,
          ep ? ep->bias_dev : nullptr, ep ? static_cast<const __nv_bfloat16*>(ep->residual_dev) : nullptr,
          ep ? ep->relu : 0);
    OCNN_LAUNCH_OK("fold_tail_kernel");
    note_launches(1);
    if (h_out < s.fold_nodes) return OCNN_OK;
  }
  a.scatter_child = scatter ? g->child_dev : nullptr;
  a.h_in = h_in; a.h_out = h_out; a.cin = s.cin_eff; a.npad = s.npad; a.T = s.T;
  a.stride = (s.fold_in || s.expand_out) ? 1 : stride;
  a.identity = identity ? 1 : 0; a.nkb = s.nkb; a.stages = s.stages;
  a.tmem_cols = s.tmem_cols;
  a.group = s.group;
  a.rows = s.group ? h_out / 8 : (s.expand_out ? h_in : h_out / s.fold_nodes);
  const int cslice = s.slices > 1 ? 256 : s.cout_eff;
  a.cout = cslice;
  a.row_elems = s.group ? 8 * cout : cslice;
  a.y_stride = s.group ? 8 * cout : s.cout_eff;
  a.rowsplit = (s.group && cin <= 16) ? 1 : 0;
  if (s.gtable) a.rowsplit = 3;
  if (!s.group && s.cin_eff % 64 == 0) a.rowsplit = 2;
  if (!s.group && s.ntable_stride == kGroupTableStride) a.rowsplit = 4;
  if (x2 != nullptr) a.rowsplit = 0;       // the two-input gather is written for one row per thread
  a.tile_rows = s.tile_rows;
  // 32-byte epilogue accesses: rows and channel slices on 32-byte boundaries
  a.wide = (a.row_elems % 16 == 0 && a.y_stride % 16 == 0 && (uintptr_t)y % 32 == 0 &&
            (!(ep && ep->residual_dev) || (uintptr_t)ep->residual_dev % 32 == 0)) ? 1 : 0;
  if (s.group)
    OCNN_REQUIRE(h_out % 8 == 0, "%s: an octree level holds whole sibling groups (got %d nodes)", who, h_out);
  a.scale = ep ? ep->scale_dev : nullptr;
  a.bias = ep ? ep->bias_dev : nullptr;
  a.residual = ep ? static_cast<const __nv_bfloat16*>(ep->residual_dev) : nullptr;
  a.relu = ep ? ep->relu : 0;
  a.status = status;
  for (int i = 0; i < 27; ++i) {
    int tap = i < tl.count ? tl.tap[i] : 0;
    // a stride-1 deconvolution gathers from the mirrored offsets
    if (kind.transposed && stride == 1) tap = 26 - tap;
    a.tap[i] = (signed char)(((tap / 9) << 4) | (((tap / 3) % 3) << 2) | (tap % 3));
  }
  // raising the dynamic shared memory limit is per function and per device
  static PerDeviceOnce attr_once;
  int device = 0;
  OCNN_CUDA_OK(cudaGetDevice(&device));
  typedef void (*KernelFn)(const TcArgs);
  static const KernelFn table[2][8] = {
      {conv_tc_kernel<0, false, false>, conv_tc_kernel<1, false, false>, conv_tc_kernel<2, false, false>,
       conv_tc_kernel<4, false, false>, conv_tc_kernel<8, false, false>, conv_tc_kernel<16, false, false>,
       conv_tc_kernel<32, false, false>, conv_tc_kernel<64, false, false>},
      {conv_tc_kernel<0, true, false>, conv_tc_kernel<1, true, false>, conv_tc_kernel<2, true, false>,
       conv_tc_kernel<4, true, false>, conv_tc_kernel<8, true, false>, conv_tc_kernel<16, true, false>,
       conv_tc_kernel<32, true, false>, conv_tc_kernel<64, true, false>}};
  static const KernelFn general[2] = {conv_tc_kernel<0, false, true>, conv_tc_kernel<0, true, true>};
  // persistent variant (two 128-row tiles per weight tile): Cin = any multiple of 64, 64, 128, 256, 512
  typedef void (*PersistFn)(const TcArgs, const int, const int);
  static const PersistFn persist[2][5] = {
      {conv_tc_persist_kernel<0, false, 2>, conv_tc_persist_kernel<8, false, 2>,
       conv_tc_persist_kernel<16, false, 2>, conv_tc_persist_kernel<32, false, 2>,
       conv_tc_persist_kernel<64, false, 2>},
      {conv_tc_persist_kernel<0, true, 2>, conv_tc_persist_kernel<8, true, 2>,
       conv_tc_persist_kernel<16, true, 2>, conv_tc_persist_kernel<32, true, 2>,
       conv_tc_persist_kernel<64, true, 2>}};
  // ... and for the few-channel sibling-group layers of big levels (one 128-row tile at a time)
  static const PersistFn persist_group[2][2] = {
      {conv_tc_persist_kernel<1, false, 1>, conv_tc_persist_kernel<2, false, 1>},
      {conv_tc_persist_kernel<1, true, 1>, conv_tc_persist_kernel<2, true, 1>}};
  int slot = 0;
  switch (a.cin >> 3) {
    case 1: slot = 1; break;
    case 2: slot = 2; break;
    case 4: slot = 3; break;
    case 8: slot = 4; break;
    case 16: slot = 5; break;
    case 32: slot = 6; break;
    case 64: slot = 7; break;
    default: break;
  }
  const bool needs_general = a.up || a.expand_cout > 0;
  if (x2 != nullptr) slot = 0;             // the variant with run-time channel counts
  KernelFn kernel = needs_general ? general[a.f16] : table[a.f16][slot];
  {
    std::lock_guard<std::mutex> lock(attr_once.mutex);
    const bool known = device >= 0 && device < 64;
    if (!known || !attr_once.done[device]) {
      for (int h = 0; h < 2; ++h) {
        for (int k = 0; k < 8; ++k)
          OCNN_CUDA_OK(cudaFuncSetAttribute(table[h][k], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            220 * 1024));
        for (int k = 0; k < 5; ++k)
          OCNN_CUDA_OK(cudaFuncSetAttribute(persist[h][k], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            227 * 1024));
        OCNN_CUDA_OK(cudaFuncSetAttribute(general[h], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          220 * 1024));
        for (int k = 0; k < 2; ++k)
          OCNN_CUDA_OK(cudaFuncSetAttribute(persist_group[h][k],
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      }
      if (known) attr_once.done[device] = true;
    }
  }
  OCNN_REQUIRE(x2 != nullptr || (long long)h_in * cin * 2 < (1LL << 32),
               "%s: input tensor of %lld bytes exceeds the 4 GiB this kernel addresses", who,
               (long long)h_in * cin * 2);
  const int ntiles = ceil_div(a.rows, a.tile_rows);
  // The persistent kernel pays where the weight tile is the larger part of a stage (256 output
  // columns: 1.1 -> 1.5 PFLOP/s at 256 -> 256 channels); with 128 columns or fewer the gather of A
  // from L2 bounds both kernels alike and the lighter one-tile kernel is as fast or faster.
  // ... and for single-K-block layers (1x1x1 on 64 channels, folded or not), which are plain
  // streams: its weight tile stays resident and nothing is set up per 128 rows.
  if (!needs_general && (a.rowsplit == 2 || x2 != nullptr) && (s.npad >= 256 || (s.nkb == 1 && identity)) &&
      persist_mode() != 0) {
    const PersistShape ps = persist_shape(s, 2);
    const int sms = sm_count();
    const int big_tiles = ceil_div(a.rows, kTileM * ps.R);
    // from a few tiles per CTA on: a CTA's first tile pays the set-up alone
    if (ps.stages > 0 && big_tiles >= 3 * sms) {
      a.stages = ps.stages;
      // the same number of tiles (within one) for every CTA
      const int waves = ceil_div(big_tiles, sms);
      const int ctas = ceil_div(big_tiles, waves);
      const int pslot = (slot >= 4 && x2 == nullptr) ? slot - 3 : 0;      // Cin = 64, 128, 256, 512 -> 1..4
      OCNN_CUDA_OK(launch_chained(persist[a.f16][pslot], dim3(ctas, s.slices), dim3(32 * (4 * ps.R + 6)),
                                  ps.smem, static_cast<cudaStream_t>(stream), a, big_tiles, ps.acc_bufs));
      OCNN_LAUNCH_OK("conv_tc_persist_kernel");
      return OCNN_OK;
    }
  }
  // Sibling-group layers with 8 or 16 channels on a level of many tiles: a one-tile CTA spends
  // most of its life in set-up, the latency of its first gathers and weight tiles, and its
  // epilogue (an empty skeleton of the one-tile kernel -- no gathers, MMAs, weight bytes or stores
  // -- runs 8 -> 8 at 972 k nodes in 0.026 ms of the full kernel's 0.044).  The persistent kernel
  // pays these once per CTA and keeps gathers, MMAs and the epilogue of different tiles in flight
  // together.
  if (!needs_general && s.group && a.rowsplit == 1 && x2 == nullptr && persist_group_mode() != 0) {
    const PersistShape ps = persist_shape(s, 1);
    const int sms = sm_count();
    const int tiles = ceil_div(a.rows, kTileM);
    if (ps.stages > 0 && tiles >= 3 * sms && s.nkb % 4 == 0) {
      a.stages = ps.stages;
      const int waves = ceil_div(tiles, sms);
      const int ctas = ceil_div(tiles, waves);
      OCNN_CUDA_OK(launch_chained(persist_group[a.f16][a.cin == 8 ? 0 : 1], dim3(ctas, 1), dim3(32 * 10),
                                  ps.smem, static_cast<cudaStream_t>(stream), a, tiles, ps.acc_bufs));
      OCNN_LAUNCH_OK("conv_tc_persist_kernel");
      return OCNN_OK;
    }
  }
  OCNN_CUDA_OK(launch_chained(kernel, dim3(ntiles, s.slices), dim3(kThreads), s.smem,
                              static_cast<cudaStream_t>(stream), a));
  OCNN_LAUNCH_OK("conv_tc_kernel");
  return OCNN_OK;
}

}  // namespace
}  // namespace ocnn

extern "C" {

size_t ocnn_conv_packed_weight_bytes(int cin, int cout, const int kernel_size[3], int stride) {
  return ocnn::packed_bytes_impl(cin, cout, kernel_size, ocnn::LayerKind{stride, false, false});
}

size_t ocnn_conv_packed_weight_bytes_nempty(int cin, int cout, const int kernel_size[3]) {
  return ocnn::packed_bytes_impl(cin, cout, kernel_size, ocnn::LayerKind{1, false, true});
}

size_t ocnn_conv_packed_weight_bytes_general(int cin, int cout, const int kernel_size[3], int stride,
                                             int transposed, int nempty) {
  return ocnn::packed_bytes_impl(cin, cout, kernel_size,
                                 ocnn::LayerKind{stride, transposed != 0, nempty != 0});
}

int ocnn_conv_pack_weights(const float* w, void* packed, int cin, int cout, const int kernel_size[3],
                           int stride, void* stream) {
  return ocnn::pack_weights_impl(w, packed, cin, cout, kernel_size, ocnn::LayerKind{stride, false, false},
                                 OCNN_BF16, stream);
}

int ocnn_conv_pack_weights_nempty(const float* w, void* packed, int cin, int cout,
                                  const int kernel_size[3], void* stream) {
  return ocnn::pack_weights_impl(w, packed, cin, cout, kernel_size, ocnn::LayerKind{1, false, true},
                                 OCNN_BF16, stream);
}

int ocnn_conv_pack_weights_general(const float* w, void* packed, int cin, int cout,
                                   const int kernel_size[3], int stride, int transposed, int nempty,
                                   int dtype, void* stream) {
  return ocnn::pack_weights_impl(w, packed, cin, cout, kernel_size,
                                 ocnn::LayerKind{stride, transposed != 0, nempty != 0}, dtype, stream);
}

int ocnn_octree_conv_tc(const void* x, const void* packed, void* y, const int32_t* neigh, int h_in,
                        int h_out, int cin, int cout, const int kernel_size[3], int stride,
                        const ocnn_conv_epilogue* ep, int32_t* status, void* stream) {
  ocnn_conv_geometry g = {};
  g.stride = stride; g.h_in = h_in; g.h_out = h_out; g.neigh_dev = neigh;
  return ocnn::conv_tc_impl(x, packed, y, &g, cin, cout, kernel_size, OCNN_BF16, ep, status, stream,
                            "ocnn_octree_conv_tc");
}

int ocnn_octree_conv_tc_pair(const void* xa, int cin_a, const void* xb, int cin_b, const void* packed,
                             void* y, int h, int cout, int dtype, const ocnn_conv_epilogue* ep,
                             int32_t* status, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(xa != nullptr && xb != nullptr, "ocnn_octree_conv_tc_pair: null input");
  OCNN_REQUIRE(cin_a > 0 && cin_b > 0, "ocnn_octree_conv_tc_pair: channel counts must be positive");
  const int ks[3] = {1, 1, 1};
  ocnn_conv_geometry g = {};
  g.stride = 1; g.h_in = h; g.h_out = h;
  return conv_tc_impl(xa, packed, y, &g, cin_a + cin_b, cout, ks, dtype, ep, status, stream,
                      "ocnn_octree_conv_tc_pair", xb, cin_a);
}

int ocnn_conv_tc_wait_selftest(int32_t* status, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(status != nullptr, "ocnn_conv_tc_wait_selftest: null status");
  wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status);
  OCNN_LAUNCH_OK("wait_selftest_kernel");
  return OCNN_OK;
}

int ocnn_octree_conv_tc_nempty(const void* x, const void* packed, void* y, const int32_t* neigh,
                               const int32_t* child, const int32_t* ichild, int nne, int cin,
                               int cout, const int kernel_size[3], const ocnn_conv_epilogue* ep,
                               int32_t* status, void* stream) {
  using namespace ocnn;
  OCNN_REQUIRE(child != nullptr && ichild != nullptr,
               "ocnn_octree_conv_tc_nempty: child and ichild required");
  ocnn_conv_geometry g = {};
  g.stride = 1; g.nempty = 1; g.h_in = nne; g.h_out = nne;
  g.neigh_dev = neigh; g.child_dev = child; g.ichild_dev = ichild;
  return conv_tc_impl(x, packed, y, &g, cin, cout, kernel_size, OCNN_BF16, ep, status, stream,
                      "ocnn_octree_conv_tc_nempty");
}

int ocnn_octree_conv_tc_general(const void* x, const void* packed, void* y,
                                const ocnn_conv_geometry* geometry, int cin, int cout,
                                const int kernel_size[3], int dtype, const ocnn_conv_epilogue* ep,
                                int32_t* status, void* stream) {
  return ocnn::conv_tc_impl(x, packed, y, geometry, cin, cout, kernel_size, dtype, ep, status, stream,
                            "ocnn_octree_conv_tc_general");
}

}  // extern "C"
