/* ocnn_b200 — C ABI of the B200 (sm_100a) implementation of O-CNN's octree hot path.
 *
 * This is the drop-in boundary: a framework binding (the reference's pytorch/cpp extension, its
 * TensorFlow op library, ...) links libocnn_b200.so and calls these entry points where it used to
 * call the `*_gpu` functions of the reference's octree library.  Each declaration cites the
 * reference interface it replaces (paths relative to the microsoft/O-CNN checkout).
 *
 * Conventions
 *  - Plain pointers and sizes only.  Pointers named *_dev are device pointers, *_host host pointers.
 *  - `stream` is a cudaStream_t passed as void*; every kernel is enqueued on it and, unless a
 *    function says otherwise, nothing synchronises.  The library never allocates device memory:
 *    scratch is passed in by the caller (sizes from the *_workspace_bytes functions).
 *  - Every function returns an ocnn_status; ocnn_last_error() gives the message of the last
 *    failure on the calling thread.  Nothing aborts the process (the reference's CHECK macros do,
 *    octree/octree/logs.h:46-49).
 *  - There is no CPU implementation behind these entry points: without a CUDA device they fail
 *    with OCNN_ERR_CUDA.
 */
#ifndef OCNN_B200_H_
#define OCNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ocnn_status {
  OCNN_OK = 0,
  OCNN_ERR_INVALID = 1,      /* bad argument / malformed header / size mismatch            */
  OCNN_ERR_UNSUPPORTED = 2,  /* valid request the library does not implement                */
  OCNN_ERR_CUDA = 3,         /* a CUDA runtime call failed                                  */
  OCNN_ERR_CAPACITY = 4,     /* caller-provided buffer or workspace too small               */
  OCNN_ERR_DEVICE = 5        /* a kernel reported an internal error through its status word */
} ocnn_status;

/* Element type of a data tensor.  The 16-bit types are accumulated in fp32 by every kernel. */
typedef enum ocnn_dtype { OCNN_F32 = 0, OCNN_BF16 = 1, OCNN_F16 = 2 } ocnn_dtype;

/* Memory layout of a data tensor of C channels over H octree nodes.
 * OCNN_CHANNEL_MAJOR is the reference's [1,C,H,1] contiguous tensor (data[c*H + h],
 * octree/octree/octree_nn.cu:125).  OCNN_NODE_MAJOR is data[h*C + c] — the same logical tensor
 * in torch's channels_last memory format. */
typedef enum ocnn_layout { OCNN_CHANNEL_MAJOR = 0, OCNN_NODE_MAJOR = 1 } ocnn_layout;

const char* ocnn_last_error(void);
/* Library version and the compute capability it was compiled for (100 = sm_100a). */
int ocnn_version(void);
int ocnn_compiled_arch(void);
/* Number of CUDA kernels this library has launched so far in this process (all threads). */
long long ocnn_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Octree wire format (host side).  Replaces OctreeInfo / OctreeParser,
 * octree/octree/octree_info.h:12-116, octree_info.cpp:157-167,254-268, octree_parser.h:13-83.
 * The reference copies the 716-byte header device->host inside every operator call
 * (octree_parser.cu:4-15); here the binding parses it once and passes pointers.
 * ------------------------------------------------------------------------------------------ */
#define OCNN_HEADER_BYTES 720   /* sizeof(OctreeInfo)=716 rounded up to the first block offset */
#define OCNN_MAX_DEPTH 16

enum { OCNN_PROP_KEY = 0, OCNN_PROP_CHILD = 1, OCNN_PROP_NEIGH = 2, OCNN_PROP_FEATURE = 3,
       OCNN_PROP_LABEL = 4, OCNN_PROP_SPLIT = 5, OCNN_PROP_COUNT = 6 };

typedef struct ocnn_octree_meta {
  int32_t key_bits;            /* 32 ("_OCTREE_1.0_") or 64 ("_OCTREE_2.0_")                  */
  int32_t batch_size, depth, full_depth;
  int32_t is_adaptive, key2xyz, has_node_dis, save_pts;
  int32_t nnum[OCNN_MAX_DEPTH];          /* nodes per level over the whole batch              */
  int32_t nnum_cum[OCNN_MAX_DEPTH + 2];  /* prefix sums; [depth+1] = total, [depth+2] = cap.   */
  int32_t nnum_nempty[OCNN_MAX_DEPTH];   /* non-empty nodes per level                         */
  int32_t channels[OCNN_PROP_COUNT];     /* 0 = property absent                               */
  int32_t locations[OCNN_PROP_COUNT];    /* -1 = every level, d = only level d                */
  int64_t ptr_dis[OCNN_PROP_COUNT + 1];  /* byte offset of each property block; [6] = size    */
} ocnn_octree_meta;

/* Parse and validate the first OCNN_HEADER_BYTES of an octree buffer held in host memory
 * (OctreeInfo::check_format, octree_info.cpp:80-116). */
int ocnn_parse_header(const void* header_host, size_t nbytes, ocnn_octree_meta* meta);
/* Byte offset of property `prop` at level `depth`, or -1 when absent
 * (OctreeInfo::ptr_dis, octree_info.cpp:157-167). */
int64_t ocnn_prop_offset(const ocnn_octree_meta* meta, int prop, int depth);

/* ------------------------------------------------------------------------------------------
 * octree_pad / octree_depad.  Replace pad_forward_gpu / pad_backward_gpu,
 * octree/octree/octree_nn.cu:65-106 (bindings: pytorch/cpp/octree_pad.cpp:6-60).
 *   pad  : y[.,h] = child[h] < 0 ? val : x[., child[h]]      x: [C,Hx] -> y: [C,Hy]
 *   depad: x[., child[h]] = y[.,h] for child[h] >= 0         y: [C,Hy] -> x: [C,Hx]
 * child_dev = the child array of the level (Hy ints).  depad writes every row of x when child is
 * an octree child array (its non-negative entries enumerate 0..Hx-1).
 * ------------------------------------------------------------------------------------------ */
int ocnn_octree_pad(const void* x_dev, void* y_dev, const int32_t* child_dev, int channels,
                    int hx, int hy, float val, int dtype, int layout, void* stream);
int ocnn_octree_depad(const void* y_dev, void* x_dev, const int32_t* child_dev, int channels,
                      int hx, int hy, int dtype, int layout, void* stream);

/* octree_max_pool.  Replaces octree_max_pool_gpu, octree/octree/octree_nn.cu:258-290
 * (binding: pytorch/cpp/octree_pool.cpp:6-34).  Per channel and sibling group: the maximum
 * (first one wins, NaN never wins) and the absolute bottom row of it.  btm: [C, 8*top_h],
 * top and mask: [C, top_h] in the same layout as the data. */
int ocnn_octree_max_pool(const void* btm_dev, void* top_dev, int32_t* mask_dev, int channels,
                         int top_h, int dtype, int layout, void* stream);

/* OctreeTile: nearest-neighbour upsampling to the next finer level, the octree_depad followed by
 * an eightfold repeat that the reference's module runs (pytorch/ocnn/modules.py:193-207).
 * y: [C, hy] rows of level `depth`; out: [C, hout] rows of level depth + 1 (hout = 8 * number of
 * non-empty nodes of level `depth`); child_dev: the Child block of level `depth`.
 * out[., 8*child[h] + j] = y[., h] for child[h] >= 0, j = 0..7. */
int ocnn_octree_tile(const void* y_dev, void* out_dev, const int32_t* child_dev, int channels,
                     int hy, int hout, int dtype, int layout, void* stream);

/* OctreeMaxPool in one pass: octree_max_pool followed by octree_pad with 0, the pair the
 * reference's module runs (pytorch/ocnn/octree_pool.py, OctreeMaxPool.forward: octree_max_pool
 * then octree_pad at depth - 1).  btm: [btm_h, C] rows of level `depth`; top: [top_h, C] rows of
 * level depth - 1; child_dev: the Child block of level depth - 1 (child[p] = sibling group of
 * node p, < 0 for a leaf, whose row becomes 0).  bf16 node-major data, C % 8 == 0; no argmax
 * (inference). */
int ocnn_octree_max_pool_pad(const void* btm_dev, void* top_dev, const int32_t* child_dev,
                             int channels, int btm_h, int top_h, int dtype, int layout,
                             void* stream);

/* ------------------------------------------------------------------------------------------
 * Neighbour table.  Replace calc_neigh_gpu (both overloads), octree/octree/octree_nn.cu:331-413,
 * and the CPU loop of merge_octrees that the PyTorch path actually runs
 * (octree/octree/merge_octrees.cpp:184-197 -> octree_nn.cpp:357-424).
 * ------------------------------------------------------------------------------------------ */
/* Full level `depth` of `batch` octrees: batch * 8^depth * 8 ints. */
int ocnn_calc_neigh_full(int32_t* neigh_dev, int depth, int batch, void* stream);
/* Level d from level d-1: neigh_dev / child_dev describe the nnum_parent nodes of level d-1;
 * neigh_child_dev receives one 64-int block per non-empty parent. */
int ocnn_calc_neigh_split(int32_t* neigh_child_dev, const int32_t* neigh_dev,
                          const int32_t* child_dev, int nnum_parent, void* stream);
/* All levels 1..depth of a merged octree buffer in device memory (its Child blocks must be
 * filled in); `meta` is the parsed header of that buffer. */
int ocnn_calc_neigh(void* octree_dev, const ocnn_octree_meta* meta, void* stream);

/* ------------------------------------------------------------------------------------------
 * octree2col (compatibility/test operator; the convolution below never materialises it).
 * Replaces octree2col_gpu, octree/octree/octree_nn.cu:110-159 (binding:
 * pytorch/cpp/octree2col.cpp:47-83).  data: [C, octree_h] fp32 channel-major;
 * col: [C, K, h_out]; stride 1: h_out = octree_h; stride 2: h_out = octree_h / 8.
 * ------------------------------------------------------------------------------------------ */
int ocnn_octree2col(const float* data_dev, float* col_dev, const int32_t* neigh_dev,
                    int channels, int h_out, const int kernel_size[3], int stride, void* stream);

/* octree2col on all nodes (child_dev == NULL) or on the non-empty nodes only, and its transpose.
 * Replace octree2colP_gpu and col2octree_gpu / col2octreeP_gpu, octree/octree/octree_nn.cu:130-253
 * (bindings pytorch/cpp/octree2col.cpp:47-226).  data: [C, octree_h] fp32 channel-major; col:
 * [C, K, h_col] with h_col = nodes (stride 1; the non-empty ones when child is given) or sibling
 * groups (stride 2).  ocnn_col2octree clears `data` and then adds every column entry to the node
 * it was gathered from (atomic additions: the summation order is not fixed). */
int ocnn_octree2col_general(const float* data_dev, float* col_dev, const int32_t* neigh_dev,
                            const int32_t* child_dev, const int32_t* ichild_dev, int channels,
                            int h_col, int octree_h, const int kernel_size[3], int stride,
                            void* stream);
int ocnn_col2octree(const float* col_dev, float* data_dev, const int32_t* neigh_dev,
                    const int32_t* child_dev, const int32_t* ichild_dev, int channels, int h_col,
                    int octree_h, const int kernel_size[3], int stride, void* stream);

/* ------------------------------------------------------------------------------------------
 * Octree convolution, forward.  Replaces OctreeBaseConv::forward_gpu_gemm
 * (octree/octree/octree_conv.cpp:276-298: octree2col_gpu + cublasSgemm through
 * pytorch/cpp/octree_conv.cpp:30-45) with one implicit-GEMM kernel: no im2col workspace.
 *
 *   y[co, h] = sum_{ci, t} w[co, ci*K + t] * x[ci, nbr(h, t)]        (taps with no neighbour = 0)
 *   stride 1: h over the h_out = nnum[d] nodes, nbr(h,t) = neigh[(h>>3)*64 + ni[(h&7)*K + t]]
 *   stride 2: h over the h_out = nnum[d]/8 sibling groups, nbr(h,t) = neigh[h*64 + ni[t]]
 *   kernel 1x1x1 stride 1: nbr(h) = h and neigh_dev may be NULL.
 *
 * x: h_in rows (nnum[d]); weights: fp32 [Cout, Cin*K] exactly as the reference module holds them
 * (pytorch/ocnn/octree_conv.py:90).  dtype/layout describe x and y.  OCNN_F32 computes in fp32 FMA
 * (parity path, rel 1e-5); OCNN_BF16 data uses the tensor-core path where the shape allows
 * (node-major, Cin % 8 == 0, packed weights) and an fp32-accumulating SIMT kernel otherwise.
 *
 * Optional fused epilogue (all NULL/0 for the plain reference operator):
 *   y = act( scale[co] * acc + bias[co] + residual[co,h] ),  act = ReLU when relu != 0.
 * This is how an inference BatchNorm / ReLU / skip connection that follows the convolution in the
 * reference's modules (pytorch/ocnn/modules.py:23-36,110-139) is applied without another pass.
 * ------------------------------------------------------------------------------------------ */
typedef struct ocnn_conv_epilogue {
  const float* scale_dev;     /* [Cout] or NULL (= 1)  */
  const float* bias_dev;      /* [Cout] or NULL (= 0)  */
  const void* residual_dev;   /* same dtype/layout/shape as y, or NULL */
  int32_t relu;
} ocnn_conv_epilogue;

int ocnn_octree_conv(const void* x_dev, const float* weights_dev, void* y_dev,
                     const int32_t* neigh_dev, int h_in, int h_out, int cin, int cout,
                     const int kernel_size[3], int stride, int dtype, int layout,
                     const ocnn_conv_epilogue* epilogue, void* stream);

/* The convolution on the non-empty nodes only: OctreeConv(nempty = True), stride 1.  Replaces
 * octree2colP_gpu + GEMM (octree/octree/octree_nn.cu:179-253, octree_conv.cpp:48-140 with nempty_,
 * binding pytorch/cpp/octree_conv.cpp:109-116).  x, y: nne rows (the non-empty nodes of the level
 * in order); child_dev: the level's Child block (nnum ints); ichild_dev: its inverse (nne ints),
 * filled by ocnn_octree_ichild.  y[co, i] = sum w[co, ci*K + t] * x[ci, child[nbr(ichild[i], t)]],
 * neighbours that are missing or empty contribute 0.  fp32 / bf16 data in either layout on the
 * CUDA-core kernel; bf16 node-major data on the tensor-core kernel through the *_nempty entry
 * points below (weights packed with ocnn_conv_pack_weights_nempty: a tile row is a single node
 * here, never a sibling group). */
int ocnn_octree_ichild(const int32_t* child_dev, int nnum, int32_t* ichild_dev, void* stream);
int ocnn_octree_conv_nempty(const void* x_dev, const float* weights_dev, void* y_dev,
                            const int32_t* neigh_dev, const int32_t* child_dev,
                            const int32_t* ichild_dev, int nne, int cin, int cout,
                            const int kernel_size[3], int dtype, int layout,
                            const ocnn_conv_epilogue* epilogue, void* stream);

/* Every OctreeConv / OctreeDeconv forward the reference offers, in one entry point: stride 1 or 2,
 * on all nodes or on the non-empty nodes only, convolution or deconvolution.  Replaces
 * OctreeBaseConv::forward_gpu_gemm / backward_gpu_gemm with octree2col(P)_gpu / col2octree(P)_gpu
 * (octree/octree/octree_conv.cpp:48-122, 276-330; octree_nn.cu:110-253; bindings
 * pytorch/cpp/octree_conv.cpp:137-154 octree_conv, :191-217 octree_deconv).  The deconvolution is
 * computed in gather form (each output node sums over the nodes that would scatter into it), so
 * there is no column buffer and no atomic addition.
 *
 * Rows of x / y, with d = the layer's depth (nnum, nne = node / non-empty node counts):
 *   convolution    stride 1: x nnum[d]          -> y nnum[d]        (nempty: nne[d] -> nne[d])
 *                  stride 2: x nnum[d]          -> y nnum[d]/8      (nempty: nne[d] -> nnum[d]/8)
 *   deconvolution  stride 1: x nnum[d]          -> y nnum[d]        (nempty: nne[d] -> nne[d])
 *                  stride 2: x nne[d]           -> y nnum[d+1]      (nempty: nne[d] -> nne[d+1])
 * neigh_dev / child_dev / ichild_dev belong to the level the reference's column matrix lives at:
 * d, except d + 1 for the stride-2 deconvolution.  child / ichild are read only when nempty is set
 * (ichild not by the stride-2 convolution).  Weights: fp32 [Cout, Cin*K] for the convolution,
 * [Cin, Cout*K] for the deconvolution, as the reference modules hold them
 * (pytorch/ocnn/octree_conv.py:51-58). */
typedef struct ocnn_conv_geometry {
  int32_t transposed;          /* 0: OctreeConv, 1: OctreeDeconv                              */
  int32_t stride;              /* 1 or 2                                                      */
  int32_t nempty;              /* data lives on the non-empty nodes only                      */
  int32_t h_in, h_out;         /* rows of x and of y                                          */
  const int32_t* neigh_dev;    /* NULL allowed for 1x1x1 stride 1                             */
  const int32_t* child_dev;
  const int32_t* ichild_dev;
} ocnn_conv_geometry;

int ocnn_octree_conv_general(const void* x_dev, const float* weights_dev, void* y_dev,
                             const ocnn_conv_geometry* geometry, int cin, int cout,
                             const int kernel_size[3], int dtype, int layout,
                             const ocnn_conv_epilogue* epilogue, void* stream);

/* Training support.  The gradient with respect to the data of a convolution is the deconvolution
 * with the same weights and vice versa (ocnn_octree_conv_general with `transposed` flipped).  The
 * gradient with respect to the weights, replacing OctreeBaseConv::weight_gpu_gemm
 * (octree/octree/octree_conv.cpp:332-360: octree2col_gpu + GEMM), is
 *     dw[m, c*K + k] = sum_h a[m, h] * x[c, nbr(h, k)]
 * where `geometry` is the CONVOLUTION-type gather (transposed = 0) of the layer's column matrix:
 * x has geometry->h_in rows, a has geometry->h_out rows.  Convolution: a = output gradient
 * [Cout, h_out], x = layer input [Cin, h_in], dw = [Cout, Cin*K].  Deconvolution at depth d: a =
 * layer input [Cin, .], x = output gradient [Cout, .], geometry = that of the convolution from the
 * output level back to the input level, dw = [Cin, Cout*K].  fp32 data in either layout; dw is
 * cleared and then accumulated with atomic additions. */
int ocnn_octree_conv_weight_grad(const float* a_dev, const float* x_dev, float* dw_dev,
                                 const ocnn_conv_geometry* geometry, int m_channels, int x_channels,
                                 const int kernel_size[3], int layout, void* stream);
/* The transposes of the max-pool through its argmax mask.  Replace octree_max_unpool_gpu /
 * octree_mask_pool_gpu, octree/octree/octree_nn.cu:293-329 (bindings pytorch/cpp/octree_pool.cpp:
 * 36-95).  top, mask: [C, top_h]; btm: [C, 8*top_h]; fp32.  unpool: btm = 0, btm[., mask] = top;
 * mask_pool: top = btm[., mask]. */
int ocnn_octree_max_unpool(const float* top_dev, const int32_t* mask_dev, float* btm_dev, int channels,
                           int top_h, int layout, void* stream);
int ocnn_octree_mask_pool(const float* btm_dev, const int32_t* mask_dev, float* top_dev, int channels,
                          int top_h, int layout, void* stream);

/* Tensor-core path: weights packed once per layer into bf16 K-major tiles.  The packed image
 * depends on the kernel shape AND the stride the layer will run with (stride-1 neighbourhood
 * convolutions with few channels use a per-sibling-group formulation with expanded weights). */
size_t ocnn_conv_packed_weight_bytes_nempty(int cin, int cout, const int kernel_size[3]);
int ocnn_conv_pack_weights_nempty(const float* weights_dev, void* packed_dev, int cin, int cout,
                                  const int kernel_size[3], void* stream);
int ocnn_octree_conv_tc_nempty(const void* x_dev, const void* packed_dev, void* y_dev,
                               const int32_t* neigh_dev, const int32_t* child_dev,
                               const int32_t* ichild_dev, int nne, int cin, int cout,
                               const int kernel_size[3], const ocnn_conv_epilogue* epilogue,
                               int32_t* status_dev, void* stream);
size_t ocnn_conv_packed_weight_bytes(int cin, int cout, const int kernel_size[3], int stride);
int ocnn_conv_pack_weights(const float* weights_dev, void* packed_dev, int cin, int cout,
                           const int kernel_size[3], int stride, void* stream);
/* x, y: bf16 node-major ([h, C]); cin % 8 == 0; cout % 8 == 0 up to 256, or a multiple of 256 up
 * to 4096 (then produced in 256-channel slices of one launch).
 * status_dev: one int32 in device memory, zero before the call; a kernel that gives up on a
 * bounded wait writes a non-zero code there instead of hanging. */
int ocnn_octree_conv_tc(const void* x_dev, const void* packed_weights_dev, void* y_dev,
                        const int32_t* neigh_dev, int h_in, int h_out, int cin, int cout,
                        const int kernel_size[3], int stride,
                        const ocnn_conv_epilogue* epilogue, int32_t* status_dev, void* stream);

/* A 1x1x1 stride-1 convolution over the concatenated channels of two node-major tensors of the
 * same h rows: y[h] = epilogue(W * [xa[h] | xb[h]]).  With W = [Wb | Wc] it is the sum of a residual
 * block's last convolution and its shortcut convolution, conv1x1b(y) + conv1x1c(x) of
 * pytorch/ocnn/modules.py OctreeResBlock.forward, in one launch and without the shortcut tensor
 * (BatchNorm scales folded into the two halves of W by the caller, the biases added up).
 * packed_weights_dev: ocnn_conv_pack_weights_general(W as fp32 [cout, cin_a + cin_b], 1x1x1,
 * stride 1); cin_a, cin_b multiples of 8 with a sum that the packer does not fold (not 8, 16, 32). */
int ocnn_octree_conv_tc_pair(const void* xa_dev, int cin_a, const void* xb_dev, int cin_b,
                             const void* packed_weights_dev, void* y_dev, int h, int cout, int dtype,
                             const ocnn_conv_epilogue* epilogue, int32_t* status_dev, void* stream);

/* Self-test of the bounded waits of the tensor-core kernels (no reference counterpart: the
 * reference has no such kernels).  Launches one small CTA whose two waiting threads wait on a
 * barrier that nobody arrives on.  status_dev: two int32, zero before the call; afterwards
 * status_dev[0] = 1 or 2 (the code of the wait that ran out of polls first) and status_dev[1] = 1
 * (the second waiter came back with "stop").  The kernel returns by itself after about 2^20 polls (well under a
 * second); the context stays usable. */
int ocnn_conv_tc_wait_selftest(int32_t* status_dev, void* stream);

/* The tensor-core kernel for every layer kind ocnn_octree_conv_general takes, on bf16 or fp16
 * node-major data (dtype = OCNN_BF16 / OCNN_F16; fp32 accumulation in TMEM either way).  The packed
 * image depends on (cin, cout, kernel, stride, transposed, nempty, dtype): pack with the same
 * values the layer runs with.  Kernel 2 with stride 2 — the down- and up-sampling layers of the
 * reference's U-Net (pytorch/ocnn/unet.py:19-36) — runs as a dense product: the convolution on all
 * nodes reads a sibling group's eight children as one row of 8*Cin channels, the deconvolution
 * writes a parent's eight children as one row of 8*Cout channels (through child on non-empty
 * nodes); neither gathers.  status_dev as for ocnn_octree_conv_tc. */
size_t ocnn_conv_packed_weight_bytes_general(int cin, int cout, const int kernel_size[3], int stride,
                                             int transposed, int nempty);
int ocnn_conv_pack_weights_general(const float* weights_dev, void* packed_dev, int cin, int cout,
                                   const int kernel_size[3], int stride, int transposed, int nempty,
                                   int dtype, void* stream);
int ocnn_octree_conv_tc_general(const void* x_dev, const void* packed_dev, void* y_dev,
                                const ocnn_conv_geometry* geometry, int cin, int cout,
                                const int kernel_size[3], int dtype,
                                const ocnn_conv_epilogue* epilogue, int32_t* status_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * Octree editing for the generative networks.  Replace octree_new / octree_grow / octree_update
 * (pytorch/cpp/octree_grow.cpp:108-148, 8-104, 150-177).  Headers are passed and returned as the
 * OCNN_HEADER_BYTES the caller holds on the host; results are byte-identical to the reference's.
 *
 * ocnn_octree_new: `batch_size` root nodes (depth 0, xyz keys, Key / Child / Neigh(8) /
 *   Feature(channel) on every level, box [0,2]^3), written into HOST memory as the reference does;
 *   the caller uploads it.
 * ocnn_octree_grow: a copy of the octree with level target_depth (<= depth + 1) added: eight
 *   children under every non-empty node of the level above, with their xyz keys
 *   (generate_key, octree/octree/octree_nn.cpp:428-464), child = 0..n-1 and the neighbour table
 *   (calc_neigh); full_octree: the level is complete (every node above must be non-empty).  First
 *   ocnn_octree_grow_header (host only) gives the new header, whose total size
 *   (ocnn_parse_header -> ptr_dis[6]) the caller allocates; then ocnn_octree_grow fills it.
 * ocnn_octree_update: in place, child[depth][i] = rank of node i among the nodes whose label equals
 *   `split`, -1 for the others (generate_label, octree_nn.cpp:466-473), and their number becomes
 *   nnum_nempty[depth] (1 with child[0] = 0 when there is none).  Synchronises the stream once (the
 *   number goes into the header).  workspace_dev: ocnn_octree_update_workspace_bytes() bytes.
 * ------------------------------------------------------------------------------------------ */
size_t ocnn_octree_new_bytes(int batch_size, int channel, int key_bits);
int ocnn_octree_new(int batch_size, int channel, int node_dis, int adaptive_layer, int key_bits,
                    void* out_host, size_t capacity);
int ocnn_octree_grow_header(const void* header_host_in, int target_depth, int full_octree,
                            void* header_host_out);
int ocnn_octree_grow(const void* octree_in_dev, const void* header_host_in, void* octree_out_dev,
                     const void* header_host_out, int target_depth, int full_octree, void* stream);
size_t ocnn_octree_update_workspace_bytes(void);
int ocnn_octree_update(void* octree_dev, const void* header_host_in, const int32_t* label_dev, int depth,
                       int split, void* workspace_dev, void* header_host_out, void* stream);

/* ------------------------------------------------------------------------------------------
 * points -> octree, batched, on the device.  Replaces Octree::build
 * (octree/octree/octree.cpp:74-121, binding pytorch/cpp/point2octree.cpp:5-34) and, when
 * `merged` is set, the merge_octrees call that follows it in the reference pipeline
 * (octree/octree/merge_octrees.cpp:7-15, binding pytorch/cpp/octree_batch.cpp:5-22): the output
 * is bit-identical to building each cloud with the reference and merging the results.
 *
 * Two calls, because the output size depends on the data:
 *   1. ocnn_octree_build_plan: sorts and counts on `stream`, then SYNCHRONISES that stream once
 *      and fills `meta` (node counts, block offsets, total size in meta->ptr_dis[6]).
 *   2. ocnn_octree_build_emit: writes the header and every block into out_dev
 *      (>= meta->ptr_dis[6] bytes), including the neighbour table when merged; the header
 *      bytes are also returned in header_host_out so the caller need not read them back.
 * The workspace must stay untouched between the two calls.
 * ------------------------------------------------------------------------------------------ */
typedef struct ocnn_build_params {
  int32_t depth, full_depth;
  int32_t key_bits;        /* 32 (depth <= 8, batch <= 255) or 64                               */
  int32_t merged;          /* 0: single octree (batch must be 1, no Neigh); 1: merged batch     */
  int32_t node_dis, split_label, save_pts;   /* as Points2Octree, pytorch/ocnn/transforms.py:10-25 */
  int32_t adp_depth;       /* recorded in the header only                                       */
  float th_normal, th_distance;              /* recorded in the header only                     */
  float bbmin[3], bbmax[3];                  /* points2octree always uses [-1,1]^3               */
} ocnn_build_params;

typedef struct ocnn_points_batch {
  int32_t batch;                   /* number of clouds                                          */
  const int32_t* offsets_host;     /* [batch+1] running point counts: cloud b has             */
                                   /* offsets[b+1]-offsets[b] points                            */
  /* Host arrays of `batch` device pointers, one per cloud, point-major float32 as in the      */
  /* reference's Points buffer (octree/octree/points_info.h:8-40); every cloud of a batch has   */
  /* the same set of properties.                                                               */
  const float* const* xyz_dev;     /* each [n_b,3]                                              */
  const float* const* normal_dev;  /* each [n_b,3], or NULL for the whole batch                 */
  const float* const* feature_dev; /* each [n_b,feature_channels], or NULL                      */
  int32_t feature_channels;
  const float* const* label_dev;   /* each [n_b], or NULL                                       */
} ocnn_points_batch;

size_t ocnn_octree_build_workspace_bytes(int64_t total_points, int batch, int depth,
                                         int full_depth);
int ocnn_octree_build_plan(const ocnn_points_batch* points, const ocnn_build_params* params,
                           void* workspace_dev, size_t workspace_bytes, ocnn_octree_meta* meta,
                           void* stream);
int ocnn_octree_build_emit(const ocnn_points_batch* points, const ocnn_build_params* params,
                           const ocnn_octree_meta* meta, void* workspace_dev,
                           size_t workspace_bytes, void* out_dev, size_t out_bytes,
                           void* header_host_out /* OCNN_HEADER_BYTES or NULL */, void* stream);

/* ------------------------------------------------------------------------------------------
 * octree_batch: merge already-built octrees held in device memory.  Replaces merge_octrees
 * (octree/octree/merge_octrees.cpp:7-198, binding pytorch/cpp/octree_batch.cpp:5-22).
 * headers_host: `batch` parsed headers; octrees_dev: `batch` device pointers (host array).
 * ocnn_octree_batch_meta computes the merged header; ocnn_octree_batch fills out_dev
 * (merged->ptr_dis[6] bytes) including the neighbour table.
 * ------------------------------------------------------------------------------------------ */
int ocnn_octree_batch_meta(const ocnn_octree_meta* headers_host, int batch,
                           ocnn_octree_meta* merged);
size_t ocnn_octree_batch_workspace_bytes(int batch, int depth);
int ocnn_octree_batch(const void* const* octrees_dev, const ocnn_octree_meta* headers_host,
                      const void* first_header_host, int batch, const ocnn_octree_meta* merged,
                      void* workspace_dev, size_t workspace_bytes, void* out_dev,
                      void* header_host_out /* OCNN_HEADER_BYTES or NULL */, void* stream);

/* octree_batch for callers that cannot provide device scratch (no counterpart in the reference:
 * its merge runs on the CPU).  Same arguments and result as ocnn_octree_batch, minus the
 * workspace: the small (octree, level) table the merge kernel reads is kept in a fixed array built
 * into the library's device image, so the call performs no device (or host heap) allocation.
 * Use it from code that must not allocate at that point — e.g. while a framework allocator owns
 * all device memory and a fresh cudaMalloc would fail.
 *  - Limit: batch * (depth + 1) <= 2048; larger requests fail with OCNN_ERR_CAPACITY.  The array
 *    (144 KiB) is held on every GPU that loads the library until the process exits.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call before starting any stream capture.
 *  - All calls share the one array.  Each call rewrites every table entry it uses, so stale
 *    contents are harmless, but two calls whose kernels overlap on the GPU (different streams)
 *    race on it: issue them on one stream or order them with events. */
int ocnn_octree_batch_noalloc(const void* const* octrees_dev, const ocnn_octree_meta* headers_host,
                              const void* first_header_host, int batch,
                              const ocnn_octree_meta* merged, void* out_dev,
                              void* header_host_out /* OCNN_HEADER_BYTES or NULL */, void* stream);

/* ------------------------------------------------------------------------------------------
 * Keys: conversion, search, and the operators built on the search.  A key packs four lanes
 * (x, y, z, batch id): bytes for 32-bit keys, 16-bit words for 64-bit keys
 * (octree/octree/types.h:16-24).
 * ------------------------------------------------------------------------------------------ */
/* xyz lanes -> Morton key (to_key != 0) or back.  Replaces xyz2key_gpu / key2xyz_gpu,
 * octree/octree/octree_nn.cu:594-660 (bindings pytorch/cpp/octree_key.cpp:47-77). */
int ocnn_convert_key(const void* in_dev, void* out_dev, int64_t num, int depth, int key_bits,
                     int to_key, void* stream);
/* idx[i] = position of query[i] among the n_key ascending keys, or -1.  query_is_xyz != 0: the
 * queries are xyz lanes and are converted with `depth` first.  Replaces search_key_gpu,
 * octree/octree/octree_nn.cu:575-590 (binding pytorch/cpp/octree_key.cpp:79-126). */
int ocnn_search_key(const void* keys_dev, int n_key, const void* query_dev, int64_t n_query,
                    int32_t* idx_dev, int query_is_xyz, int depth, int key_bits, void* stream);
/* out[child[h]] = key[h] for child[h] >= 0: the keys of a level's non-empty nodes, in order (the
 * pad_backward_gpu call on the key array at pytorch/cpp/octree_key.cpp:100-108). */
int ocnn_key_depad(const void* key_dev, const int32_t* child_dev, int nnum, void* out_dev,
                   int key_bits, void* stream);
/* Node data sampled at points, in one kernel.  Replaces the reference's octree_nearest_pts /
 * octree_trilinear_pts (pytorch/ocnn/modules.py:209-275: key arithmetic, octree_search_key, a
 * sparse matrix and two sparse products).  data: [C, h] rows of the nodes whose ascending keys are
 * keys_dev[0..n_key) (a level's Key block, or ocnn_key_depad of it); pts_dev: [n_pts, 4] float32 =
 * (x, y, z) scaled to [0, 2^depth] and the batch id; out: [C, n_pts] in the data's dtype / layout.
 * linear == 0: the row of the cell holding the point (0 if absent); linear != 0: trilinear weights
 * over the 8 cells around the point, renormalised over those that exist. */
int ocnn_octree_interp(const void* data_dev, void* out_dev, const float* pts_dev, const void* keys_dev,
                       int n_key, int channels, int h, int64_t n_pts, int depth, int key_bits,
                       int linear, int dtype, int layout, void* stream);
/* dst[., idx[h]] = src[., h] for idx[h] >= 0, every other row of dst 0.  Replaces
 * align_forward_gpu, octree/octree/octree_nn.cu:711-732 (binding pytorch/cpp/octree_align.cpp:9-60;
 * idx comes from ocnn_search_key of the source keys among the destination keys). */
int ocnn_octree_align(const void* src_dev, void* dst_dev, const int32_t* idx_dev, int channels,
                      int src_h, int dst_h, int dtype, int layout, void* stream);
/* Its transpose: src_grad[., h] = idx[h] < 0 ? 0 : dst_grad[., idx[h]].  Replaces
 * align_backward_gpu, octree/octree/octree_nn.cu:734-752 (binding octree_align.cpp:62-82). */
int ocnn_octree_align_backward(const void* dst_grad_dev, void* src_grad_dev, const int32_t* idx_dev,
                               int channels, int src_h, int dst_h, int dtype, int layout,
                               void* stream);

/* ------------------------------------------------------------------------------------------
 * Point-cloud preparation on the device (the reference runs these on the CPU in its DataLoader
 * workers before points2octree).  Replace PointsParser::displace / rotate / translate / scale /
 * orient_normal / clip, octree/octree/points_parser.cpp:42-259, and bounding_box,
 * octree/octree/math_functions.cpp:113-128 (bindings pytorch/cpp/transform_points.cpp:7-125).
 * ------------------------------------------------------------------------------------------ */
/* In place, in the reference's order: p += normal * offset (when offset > 1e-10 and normals
 * exist); p, normal = R p, R normal (rot9: out[m] = sum_k rot9[k*3 + m] * in[k], or NULL);
 * p += shift3 (or NULL); p *= scale3 (or NULL; with unequal factors the normals are divided by
 * them and renormalised); normals flipped so that component orient-1 is >= 0 (orient 1..3), made
 * non-negative per component (4) or left alone (0). */
int ocnn_points_transform(float* xyz_dev, float* normal_dev, int64_t n, float offset,
                          const float* rot9, const float* shift3, const float* scale3, int orient,
                          void* stream);
/* Keep, in order, the points strictly inside (bbmin, bbmax).  src/dst/channels: the four property
 * blocks (xyz, normal, feature, label; channels[t] == 0 = absent) of the source and of the
 * destination buffer (distinct memory).  mask_dev[i] = 1 for kept points; *pt_num_out_dev = their
 * number — it may point at the pt_num field of the destination's header.  If no point is inside,
 * one point at bbmin is kept (points_parser.cpp:169-175). */
size_t ocnn_points_clip_workspace_bytes(int64_t n);
int ocnn_points_clip(const float* const src_dev[4], float* const dst_dev[4], const int channels[4],
                     int64_t n, const float bbmin[3], const float bbmax[3], int32_t* mask_dev,
                     int32_t* pt_num_out_dev, void* workspace_dev, size_t workspace_bytes,
                     void* stream);
/* out6_dev = (min x, y, z, max x, y, z) of the n points. */
size_t ocnn_points_bbox_workspace_bytes(void);
int ocnn_points_bbox(const float* xyz_dev, int64_t n, float* out6_dev, void* workspace_dev,
                     size_t workspace_bytes, void* stream);

/* Feature block of the finest level (fp32 [C, nnum] channel-major, as stored in the octree) to the
 * bf16 node-major tensor [nnum, c_pad] the tensor-core convolution reads (channels >= C are 0).
 * Replaces the octree_property('feature') copy, pytorch/cpp/octree_property.cpp:89-97. */
int ocnn_feature_to_node_major(const float* feature_dev, void* out_dev, int channels, int c_pad,
                               int nnum, int dtype, void* stream);

/* A 1x1x1 convolution with its epilogue followed by OctreeMaxPool (octree_max_pool, then octree_pad
 * with 0 at depth - 1: pytorch/ocnn/octree_pool.py, OctreeMaxPool.forward) in one pass: the
 * convolution's own output is never written.  x: [h, cin] rows of level `depth`, 16-bit node-major;
 * weights fp32 [cout, cin]; epilogue as in ocnn_octree_conv (a residual has h rows of cout
 * channels); top: [top_h, cout] rows of level depth - 1; child_parent_dev: the Child block of level
 * depth - 1; group_parent_dev: scratch of h / 8 ints.  cin, cout in {8, 16, 32, 64} (not 64 -> 64),
 * OCNN_ERR_UNSUPPORTED otherwise: the caller then runs the two operators. */
int ocnn_octree_conv1x1_max_pool_pad(const void* x_dev, const float* weights_dev, void* top_dev,
                                     const int32_t* child_parent_dev, int h, int top_h, int cin,
                                     int cout, int dtype, const ocnn_conv_epilogue* epilogue,
                                     int32_t* group_parent_dev, void* stream);

/* Two 1x1x1 layers in a row in one pass: y1 = epilogue1(w1 * x) is written as usual and
 * y2 = epilogue2(w2 * y1) is computed from the rows of y1 while they are in registers (a residual
 * block's conv1x1b + shortcut followed by the next block's conv1x1a: pytorch/ocnn/modules.py,
 * OctreeResBlock.forward of two consecutive blocks).  16-bit node-major data of h rows; w1 fp32
 * [cmid, cin], w2 fp32 [cout2, cmid]; epilogue2 without residual.  Built for the channel triples
 * 8-32-8, 16-64-16, 16-32-8 and 8-16-8; OCNN_ERR_UNSUPPORTED otherwise (run the two layers). */
int ocnn_octree_conv1x1_chain(const void* x_dev, const float* w1_dev, void* y1_dev,
                              const ocnn_conv_epilogue* epilogue1, const float* w2_dev, void* y2_dev,
                              const ocnn_conv_epilogue* epilogue2, int h, int cin, int cmid, int cout2,
                              int dtype, void* stream);

/* The classification header of the reference's networks in one launch: FullOctreeGlobalPool (the
 * mean over the 8^d cells of each shape's full level, pytorch/ocnn/octree_pool.py:106-115) followed
 * by the Linear layer (pytorch/ocnn/resnet.py:18-21, lenet.py).  x: 16-bit node-major
 * [batch * per, channels] (a full level: per = 8^d rows per shape, shapes back to back);
 * w: fp32 [nout, channels]; bias: fp32 [nout] or NULL; out: fp32 [batch, nout]. */
int ocnn_global_pool_fc(const void* x_dev, const float* w_dev, const float* bias_dev, float* out_dev,
                        int batch, int per, int channels, int nout, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* OCNN_B200_H_ */
