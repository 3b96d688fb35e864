// `ocnn.nn` — the PyTorch binding of the octree hot path, with the function names, argument
// order and tensor conventions of the reference's extension (pytorch/cpp/pybind.cpp:3-49,
// pytorch/cpp/ocnn.h:11-72), implemented on libocnn_b200.so through its C ABI.
//
// Differences from the reference binding, all on purpose:
//  * points2octree / octree_batch run on the GPU and return CUDA tensors (the reference builds on
//    the CPU and the caller moves the result, pytorch/projects/classification.py:24).  CPU inputs
//    are uploaded; there is no CPU compute path.
//  * The 716-byte octree header is copied device->host once per octree tensor and cached, not once
//    per operator call (octree/octree/octree_parser.cu:4-15).
//  * Data tensors may be fp32 or bf16, and [1,C,H,1] contiguous (the reference layout) or
//    channels_last (node-major).  Outputs keep the dtype and layout of the input.
//  * Errors raise Python exceptions; nothing aborts (pytorch/cpp uses CHECK -> abort()).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "ocnn_b200.h"

namespace {

using torch::Tensor;
using std::string;
using std::vector;

#define OCNN_CALL(expr)                                                      \
  do {                                                                       \
    int status__ = (expr);                                                   \
    TORCH_CHECK(status__ == OCNN_OK, "ocnn_b200: ", ocnn_last_error());      \
  } while (0)

int g_key_bits = 64;  // the reference's PyTorch extension is always built with -DKEY64

void* current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// ---- octree header cache ------------------------------------------------------------------------
// Keyed by the tensor's StorageImpl; the weak reference keeps that address from being reused for
// another storage while the entry lives, so a hit is always the same buffer.
struct CachedHeader {
  c10::weak_intrusive_ptr<c10::StorageImpl> storage;
  int64_t offset;
  uint32_t version;
  ocnn_octree_meta meta;
  uint8_t raw[OCNN_HEADER_BYTES];
};
std::mutex g_cache_mutex;
std::unordered_map<const void*, CachedHeader> g_cache;

struct OctreeRef {
  ocnn_octree_meta meta;
  uint8_t raw[OCNN_HEADER_BYTES];
  uint8_t* base;   // device (or host) pointer of byte 0
  bool cuda;
};

OctreeRef get_octree(const Tensor& octree) {
  TORCH_CHECK(octree.scalar_type() == torch::kUInt8 && octree.dim() == 1 && octree.is_contiguous(),
              "the octree must be a contiguous 1-D uint8 tensor");
  TORCH_CHECK(octree.numel() >= 716, "the octree tensor is shorter than an octree header");
  OctreeRef ref;
  ref.base = octree.data_ptr<uint8_t>();
  ref.cuda = octree.is_cuda();
  if (!ref.cuda) {
    memset(ref.raw, 0, sizeof(ref.raw));
    memcpy(ref.raw, ref.base, 716);
    OCNN_CALL(ocnn_parse_header(ref.raw, (size_t)octree.numel(), &ref.meta));
    return ref;
  }
  c10::StorageImpl* impl = octree.storage().unsafeGetStorageImpl();
  const uint32_t version = octree._version();
  {
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    auto it = g_cache.find(impl);
    if (it != g_cache.end()) {
      CachedHeader& c = it->second;
      if (!c.storage.expired() && c.offset == octree.storage_offset() && c.version == version) {
        ref.meta = c.meta;
        memcpy(ref.raw, c.raw, sizeof(ref.raw));
        return ref;
      }
      g_cache.erase(it);
    }
  }
  memset(ref.raw, 0, sizeof(ref.raw));
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  TORCH_CHECK(cudaMemcpyAsync(ref.raw, ref.base, 716, cudaMemcpyDeviceToHost, st) == cudaSuccess &&
                  cudaStreamSynchronize(st) == cudaSuccess,
              "reading the octree header from the device failed");
  OCNN_CALL(ocnn_parse_header(ref.raw, (size_t)octree.numel(), &ref.meta));
  TORCH_CHECK(ref.meta.ptr_dis[OCNN_PROP_COUNT] <= octree.numel(),
              "the octree tensor is shorter than its header says");
  std::lock_guard<std::mutex> lock(g_cache_mutex);
  if (g_cache.size() > 256) {
    for (auto it = g_cache.begin(); it != g_cache.end();)
      it = it->second.storage.expired() ? g_cache.erase(it) : std::next(it);
  }
  CachedHeader c{c10::weak_intrusive_ptr<c10::StorageImpl>(
                     c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(impl)),
                 octree.storage_offset(), version, ref.meta, {}};
  memcpy(c.raw, ref.raw, sizeof(c.raw));
  g_cache.emplace(impl, std::move(c));
  return ref;
}

void remember_header(const Tensor& octree, const ocnn_octree_meta& meta, const uint8_t* raw) {
  c10::StorageImpl* impl = octree.storage().unsafeGetStorageImpl();
  CachedHeader c{c10::weak_intrusive_ptr<c10::StorageImpl>(
                     c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(impl)),
                 octree.storage_offset(), (uint32_t)octree._version(), meta, {}};
  memcpy(c.raw, raw, sizeof(c.raw));
  std::lock_guard<std::mutex> lock(g_cache_mutex);
  g_cache.erase(impl);
  g_cache.emplace(impl, std::move(c));
}

// ---- data tensor conventions ----------------------------------------------------------------------
struct DataRef {
  Tensor t;      // a tensor whose memory is exactly [C,H] (channel-major) or [H,C] (node-major)
  int C, H, dtype, layout;
};

DataRef get_data(const Tensor& data, const char* what) {
  TORCH_CHECK(data.is_cuda(), what, ": the data tensor must be a CUDA tensor (there is no CPU path)");
  TORCH_CHECK(data.dim() == 4 && data.size(0) == 1 && data.size(3) == 1, what,
              ": data must have shape [1, C, H, 1]");
  DataRef d;
  d.C = (int)data.size(1);
  d.H = (int)data.size(2);
  if (data.scalar_type() == torch::kFloat32) d.dtype = OCNN_F32;
  else if (data.scalar_type() == torch::kBFloat16) d.dtype = OCNN_BF16;
  else if (data.scalar_type() == torch::kFloat16) d.dtype = OCNN_F16;
  else TORCH_CHECK(false, what, ": data must be float32, bfloat16 or float16");
  if (data.is_contiguous()) {
    d.layout = OCNN_CHANNEL_MAJOR;
    d.t = data;
  } else if (data.is_contiguous(at::MemoryFormat::ChannelsLast)) {
    d.layout = OCNN_NODE_MAJOR;
    d.t = data;
  } else {
    d.layout = OCNN_CHANNEL_MAJOR;
    d.t = data.contiguous();
  }
  return d;
}

void need_cuda(const Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda(), what, ": the data tensor must be a CUDA tensor (there is no CPU path)");
}

Tensor new_data(int C, int H, const DataRef& like, bool zero = false) {
  auto opts = like.t.options();
  if (like.layout == OCNN_NODE_MAJOR) opts = opts.memory_format(at::MemoryFormat::ChannelsLast);
  // torch::zeros drops the memory format of its options, so zero an empty tensor instead
  Tensor out = torch::empty({1, C, H, 1}, opts);
  if (zero) out.zero_();
  return out;
}

vector<int> kernel3(vector<int> ks) {
  TORCH_CHECK(!ks.empty() && ks.size() <= 3, "kernel_size must hold 1 to 3 values");
  while (ks.size() < 3) ks.push_back(ks.back());   // resize_with_last_val, octree_nn.cpp:128-140
  for (int k : ks) TORCH_CHECK(k > 0 && k < 4, "Invalide kernel size");
  return ks;
}

const int32_t* level_ptr(const OctreeRef& o, int prop, int depth, const char* what) {
  const int64_t off = ocnn_prop_offset(&o.meta, prop, depth);
  TORCH_CHECK(off >= 0, what, ": the octree lacks the needed property at depth ", depth);
  return reinterpret_cast<const int32_t*>(o.base + off);
}

// ---- pad / depad / pool -------------------------------------------------------------------------
Tensor octree_pad(Tensor data_in, Tensor octree, int depth, float val) {
  TORCH_CHECK(depth >= 1, "Depth should be larger than 1");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_pad: the octree must be a CUDA tensor");
  TORCH_CHECK(depth <= o.meta.depth, "octree_pad: depth ", depth, " exceeds the octree depth");
  need_cuda(data_in, "octree_pad");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "octree_pad");
  TORCH_CHECK(o.meta.nnum_nempty[depth] == x.H, "octree_pad: data height ", x.H,
              " != non-empty node number ", o.meta.nnum_nempty[depth], ", d = ", depth,
              ", channel = ", x.C);
  const int top_h = o.meta.nnum[depth];
  Tensor y = new_data(x.C, top_h, x);
  OCNN_CALL(ocnn_octree_pad(x.t.data_ptr(), y.data_ptr(),
                            level_ptr(o, OCNN_PROP_CHILD, depth, "octree_pad"), x.C, x.H, top_h, val,
                            x.dtype, x.layout, current_stream()));
  return y;
}

Tensor octree_depad(Tensor data_in, Tensor octree, int depth) {
  TORCH_CHECK(depth >= 1, "Depth should be larger than 1");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_depad: the octree must be a CUDA tensor");
  TORCH_CHECK(depth <= o.meta.depth, "octree_depad: depth ", depth, " exceeds the octree depth");
  need_cuda(data_in, "octree_depad");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef y = get_data(data_in, "octree_depad");
  TORCH_CHECK(o.meta.nnum[depth] == y.H, "octree_depad: data height ", y.H, " != node number ",
              o.meta.nnum[depth], ", d = ", depth, ", channel = ", y.C);
  const int btm_h = o.meta.nnum_nempty[depth];
  Tensor x = new_data(y.C, btm_h, y, /*zero=*/true);
  OCNN_CALL(ocnn_octree_depad(y.t.data_ptr(), x.data_ptr(),
                              level_ptr(o, OCNN_PROP_CHILD, depth, "octree_depad"), y.C, btm_h, y.H,
                              y.dtype, y.layout, current_stream()));
  return x;
}

// OctreeTile (pytorch/ocnn/modules.py:193-207): depad at `depth`, every row repeated for its 8
// children: [1,C,nnum[depth],1] -> [1,C,nnum[depth+1],1], in one kernel.
Tensor octree_tile(Tensor data_in, Tensor octree, int depth) {
  TORCH_CHECK(depth >= 1, "Depth should be larger than 1");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_tile: the octree must be a CUDA tensor");
  TORCH_CHECK(depth < o.meta.depth, "octree_tile: depth ", depth, " has no finer level in the octree");
  need_cuda(data_in, "octree_tile");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef y = get_data(data_in, "octree_tile");
  TORCH_CHECK(o.meta.nnum[depth] == y.H, "octree_tile: data height ", y.H, " != node number ",
              o.meta.nnum[depth], ", d = ", depth, ", channel = ", y.C);
  const int hout = o.meta.nnum_nempty[depth] * 8;
  TORCH_CHECK(hout == o.meta.nnum[depth + 1], "octree_tile: level ", depth + 1, " does not hold the "
              "children of level ", depth);
  Tensor out = new_data(y.C, hout, y);
  OCNN_CALL(ocnn_octree_tile(y.t.data_ptr(), out.data_ptr(),
                             level_ptr(o, OCNN_PROP_CHILD, depth, "octree_tile"), y.C, y.H, hout,
                             y.dtype, y.layout, current_stream()));
  return out;
}

vector<Tensor> octree_max_pool(Tensor data_in, Tensor octree, int depth) {
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(depth > 1, "Depth should be larger than 1");
  TORCH_CHECK(depth <= o.meta.depth, "octree_max_pool: depth ", depth, " exceeds the octree depth");
  need_cuda(data_in, "octree_max_pool");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef b = get_data(data_in, "octree_max_pool");
  TORCH_CHECK(o.meta.nnum[depth] == b.H, "octree_max_pool: data height ", b.H, " != node number ",
              o.meta.nnum[depth]);
  const int top_h = b.H >> 3;
  Tensor top = new_data(b.C, top_h, b);
  auto mopts = b.t.options().dtype(torch::kInt32);
  if (b.layout == OCNN_NODE_MAJOR) mopts = mopts.memory_format(at::MemoryFormat::ChannelsLast);
  Tensor mask = torch::empty({1, b.C, top_h, 1}, mopts);
  OCNN_CALL(ocnn_octree_max_pool(b.t.data_ptr(), top.data_ptr(), mask.data_ptr<int32_t>(), b.C,
                                 top_h, b.dtype, b.layout, current_stream()));
  return {top, mask};
}

// OctreeMaxPool in one pass (bf16 node-major data, C % 8 == 0): pool level `depth`, one row per
// node of level depth - 1, zeros for leaves.  No argmax.
Tensor octree_max_pool_pad(Tensor data_in, Tensor octree, int depth) {
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(depth > 1, "Depth should be larger than 1");
  TORCH_CHECK(depth <= o.meta.depth, "octree_max_pool_pad: depth ", depth, " exceeds the octree depth");
  need_cuda(data_in, "octree_max_pool_pad");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef b = get_data(data_in, "octree_max_pool_pad");
  TORCH_CHECK(o.meta.nnum[depth] == b.H, "octree_max_pool_pad: data height ", b.H, " != node number ",
              o.meta.nnum[depth]);
  const int top_h = o.meta.nnum[depth - 1];
  Tensor top = new_data(b.C, top_h, b);
  OCNN_CALL(ocnn_octree_max_pool_pad(b.t.data_ptr(), top.data_ptr(),
                                     level_ptr(o, OCNN_PROP_CHILD, depth - 1, "octree_max_pool_pad"),
                                     b.C, b.H, top_h, b.dtype, b.layout, current_stream()));
  return top;
}

ocnn_conv_epilogue make_epilogue(const c10::optional<Tensor>& scale, const c10::optional<Tensor>& bias,
                                 const c10::optional<Tensor>& residual, bool relu, int cout,
                                 const Tensor& y);

// A 1x1x1 convolution (with scale / bias / residual / ReLU) followed by OctreeMaxPool, one pass:
// data [1, Cin, nnum[depth], 1] 16-bit channels_last -> [1, Cout, nnum[depth - 1], 1].
Tensor conv1x1_max_pool_pad(Tensor data_in, Tensor weights, Tensor octree, int depth,
                            c10::optional<Tensor> scale, c10::optional<Tensor> bias,
                            c10::optional<Tensor> residual, bool relu) {
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(depth > 1 && depth <= o.meta.depth, "conv1x1_max_pool_pad: depth ", depth, " out of range");
  need_cuda(data_in, "conv1x1_max_pool_pad");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "conv1x1_max_pool_pad");
  TORCH_CHECK(x.dtype != OCNN_F32 && (x.layout == OCNN_NODE_MAJOR || x.C == 1 || x.H == 1),
              "conv1x1_max_pool_pad takes bfloat16 or float16 channels_last data");
  x.layout = OCNN_NODE_MAJOR;
  TORCH_CHECK(o.meta.nnum[depth] == x.H, "conv1x1_max_pool_pad: data height ", x.H, " != node number ",
              o.meta.nnum[depth]);
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32 && weights.dim() == 2 &&
                  weights.size(1) == x.C, "conv1x1_max_pool_pad: weights float32 [Cout, Cin]");
  Tensor w = weights.contiguous();
  const int cout = (int)w.size(0), top_h = o.meta.nnum[depth - 1];
  Tensor top = new_data(cout, top_h, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, c10::nullopt, relu, cout, top);
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_cuda() && residual->dim() == 4 && residual->size(0) == 1 &&
                    residual->size(1) == cout && residual->size(2) == x.H && residual->size(3) == 1 &&
                    residual->scalar_type() == data_in.scalar_type() &&
                    residual->is_contiguous(at::MemoryFormat::ChannelsLast),
                "residual must be [1, Cout, H, 1] channels_last of the data's dtype");
    ep.residual_dev = residual->data_ptr();
  }
  Tensor inv = torch::empty({std::max(x.H / 8, 1)}, data_in.options().dtype(torch::kInt32).memory_format(c10::MemoryFormat::Contiguous));
  OCNN_CALL(ocnn_octree_conv1x1_max_pool_pad(x.t.data_ptr(), w.data_ptr<float>(), top.data_ptr(),
                                             level_ptr(o, OCNN_PROP_CHILD, depth - 1, "conv1x1_max_pool_pad"),
                                             x.H, top_h, x.C, cout, x.dtype, &ep, inv.data_ptr<int32_t>(),
                                             current_stream()));
  return top;
}

// Two 1x1x1 layers in one pass: y1 = act1(scale1 * (w1 * x) + bias1 + residual1), y2 = act2(scale2 *
// (w2 * y1) + bias2), 16-bit channels_last data; returns (y1, y2).
std::tuple<Tensor, Tensor> conv1x1_chain(Tensor data_in, Tensor w1, c10::optional<Tensor> scale1,
                                         c10::optional<Tensor> bias1, c10::optional<Tensor> residual1,
                                         bool relu1, Tensor w2, c10::optional<Tensor> scale2,
                                         c10::optional<Tensor> bias2, bool relu2) {
  need_cuda(data_in, "conv1x1_chain");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "conv1x1_chain");
  TORCH_CHECK(x.dtype != OCNN_F32 && (x.layout == OCNN_NODE_MAJOR || x.C == 1 || x.H == 1),
              "conv1x1_chain takes bfloat16 or float16 channels_last data");
  x.layout = OCNN_NODE_MAJOR;
  TORCH_CHECK(w1.is_cuda() && w1.scalar_type() == torch::kFloat32 && w1.dim() == 2 && w1.size(1) == x.C,
              "conv1x1_chain: w1 float32 [Cmid, Cin]");
  const int cmid = (int)w1.size(0);
  TORCH_CHECK(w2.is_cuda() && w2.scalar_type() == torch::kFloat32 && w2.dim() == 2 && w2.size(1) == cmid,
              "conv1x1_chain: w2 float32 [Cout2, Cmid]");
  const int cout2 = (int)w2.size(0);
  Tensor a = w1.contiguous(), b = w2.contiguous();
  Tensor y1 = new_data(cmid, x.H, x), y2 = new_data(cout2, x.H, x);
  ocnn_conv_epilogue ep1 = make_epilogue(scale1, bias1, residual1, relu1, cmid, y1);
  ocnn_conv_epilogue ep2 = make_epilogue(scale2, bias2, c10::nullopt, relu2, cout2, y2);
  OCNN_CALL(ocnn_octree_conv1x1_chain(x.t.data_ptr(), a.data_ptr<float>(), y1.data_ptr(), &ep1,
                                      b.data_ptr<float>(), y2.data_ptr(), &ep2, x.H, x.C, cmid, cout2,
                                      x.dtype, current_stream()));
  return std::make_tuple(y1, y2);
}

// ---- octree2col / col2octree ---------------------------------------------------------------------
// ichild of a level (node of the i-th non-empty node), as pytorch/cpp/octree2col.cpp:8-18 builds it.
Tensor make_ichild(const OctreeRef& o, int depth, const torch::TensorOptions& like, const char* what) {
  const int nne = o.meta.nnum_nempty[depth], nnum = o.meta.nnum[depth];
  Tensor ichild = torch::zeros({std::max(nne, 1)}, like.dtype(torch::kInt32));
  OCNN_CALL(ocnn_octree_ichild(level_ptr(o, OCNN_PROP_CHILD, depth, what), nnum,
                               ichild.data_ptr<int32_t>(), current_stream()));
  return ichild;
}

Tensor octree2col(Tensor data_in, Tensor octree, int depth, vector<int> kernel_size, int stride,
                  bool nempty) {
  vector<int> ks = kernel3(kernel_size);
  TORCH_CHECK(stride == 1 || stride == 2, "Unsupport stride");
  TORCH_CHECK(depth > 0, "Depth should be larger than 0");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree2col: the octree must be a CUDA tensor");
  TORCH_CHECK(depth <= o.meta.depth, "octree2col: depth ", depth, " exceeds the octree depth");
  need_cuda(data_in, "octree2col");
  c10::cuda::CUDAGuard guard(data_in.device());
  TORCH_CHECK(data_in.scalar_type() == torch::kFloat32, "octree2col takes float32 data");
  DataRef x = get_data(data_in.contiguous(), "octree2col");
  const int nnum = o.meta.nnum[depth], nne = o.meta.nnum_nempty[depth];
  TORCH_CHECK((nempty ? nne : nnum) == x.H, "octree2col: data height ", x.H, " != ",
              nempty ? "non-empty " : "", "node number ", nempty ? nne : nnum);
  int top_h = x.H;
  if (stride == 2) {
    top_h = nnum / 8;
    TORCH_CHECK(top_h == o.meta.nnum_nempty[depth - 1], "octree2col: inconsistent octree");
  }
  const int kdim = ks[0] * ks[1] * ks[2];
  Tensor col = torch::empty({x.C, kdim, top_h}, x.t.options());
  const int32_t* neigh = level_ptr(o, OCNN_PROP_NEIGH, depth, "octree2col");
  if (!nempty) {
    OCNN_CALL(ocnn_octree2col(x.t.data_ptr<float>(), col.data_ptr<float>(), neigh, x.C, top_h,
                              ks.data(), stride, current_stream()));
  } else {
    Tensor ichild = make_ichild(o, depth, x.t.options(), "octree2col");
    OCNN_CALL(ocnn_octree2col_general(x.t.data_ptr<float>(), col.data_ptr<float>(), neigh,
                                      level_ptr(o, OCNN_PROP_CHILD, depth, "octree2col"),
                                      ichild.data_ptr<int32_t>(), x.C, top_h, x.H, ks.data(), stride,
                                      current_stream()));
  }
  return col;
}

// The transpose of octree2col (pytorch/cpp/octree2col.cpp:85-122, 170-216): [C, K, h] -> [1,C,H,1].
Tensor col2octree(Tensor grad_in, Tensor octree, int depth, vector<int> kernel_size, int stride,
                  bool nempty) {
  vector<int> ks = kernel3(kernel_size);
  TORCH_CHECK(stride == 1 || stride == 2, "Unsupport stride");
  TORCH_CHECK(depth > 0, "Depth should be larger than 0");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "col2octree: the octree must be a CUDA tensor");
  TORCH_CHECK(depth <= o.meta.depth, "col2octree: depth ", depth, " exceeds the octree depth");
  TORCH_CHECK(grad_in.is_cuda() && grad_in.scalar_type() == torch::kFloat32 && grad_in.dim() == 3,
              "col2octree takes a float32 CUDA tensor of shape [C, K, H]");
  c10::cuda::CUDAGuard guard(grad_in.device());
  Tensor col = grad_in.contiguous();
  const int kdim = ks[0] * ks[1] * ks[2];
  const int channel = (int)col.size(0), top_h = (int)col.size(2);
  TORCH_CHECK(col.size(1) == kdim, "col2octree: the column tensor has ", col.size(1),
              " kernel entries, the kernel size has ", kdim);
  const int nnum = o.meta.nnum[depth], nne = o.meta.nnum_nempty[depth];
  if (stride == 2) {
    TORCH_CHECK(top_h == o.meta.nnum_nempty[depth - 1], "col2octree: height mismatch");
  } else {
    TORCH_CHECK(top_h == (nempty ? nne : nnum), "col2octree: height mismatch");
  }
  const int btm_h = nempty ? nne : nnum;
  Tensor out = torch::empty({1, channel, btm_h, 1}, col.options());
  const int32_t* neigh = level_ptr(o, OCNN_PROP_NEIGH, depth, "col2octree");
  Tensor ichild;
  const int32_t* child = nullptr;
  const int32_t* ich = nullptr;
  if (nempty) {
    ichild = make_ichild(o, depth, col.options(), "col2octree");
    child = level_ptr(o, OCNN_PROP_CHILD, depth, "col2octree");
    ich = ichild.data_ptr<int32_t>();
  }
  OCNN_CALL(ocnn_col2octree(col.data_ptr<float>(), out.data_ptr<float>(), neigh, child, ich, channel,
                            top_h, btm_h, ks.data(), stride, current_stream()));
  return out;
}

// ---- convolution -----------------------------------------------------------------------------------
struct ConvShape { int h_in, h_out; const int32_t* neigh; };

ConvShape conv_shape(const OctreeRef& o, const DataRef& x, int depth, const vector<int>& ks,
                     int stride, const char* what) {
  TORCH_CHECK(depth > 0 && depth <= o.meta.depth, what, ": The depth should be in (0, octree depth]");
  TORCH_CHECK(stride == 1 || stride == 2, "Unsupport stride");
  TORCH_CHECK(x.H == o.meta.nnum[depth], what, ": data height ", x.H, " != node number ",
              o.meta.nnum[depth], ", d: ", depth, ", channel_in: ", x.C);
  ConvShape s;
  s.h_in = x.H;
  s.h_out = stride == 2 ? x.H / 8 : x.H;
  if (stride == 2)
    TORCH_CHECK(s.h_out == o.meta.nnum_nempty[depth - 1], what, ": inconsistent octree");
  const bool identity = ks[0] * ks[1] * ks[2] == 1 && stride == 1;
  s.neigh = identity ? nullptr : level_ptr(o, OCNN_PROP_NEIGH, depth, what);
  return s;
}

ocnn_conv_epilogue make_epilogue(const c10::optional<Tensor>& scale, const c10::optional<Tensor>& bias,
                                 const c10::optional<Tensor>& residual, bool relu, int cout,
                                 const Tensor& y) {
  ocnn_conv_epilogue ep;
  ep.scale_dev = nullptr; ep.bias_dev = nullptr; ep.residual_dev = nullptr; ep.relu = relu ? 1 : 0;
  if (scale.has_value() && scale->defined()) {
    TORCH_CHECK(scale->is_cuda() && scale->scalar_type() == torch::kFloat32 && scale->is_contiguous() &&
                    scale->numel() == cout, "scale must be a contiguous float32 CUDA tensor of Cout values");
    ep.scale_dev = scale->data_ptr<float>();
  }
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == torch::kFloat32 && bias->is_contiguous() &&
                    bias->numel() == cout, "bias must be a contiguous float32 CUDA tensor of Cout values");
    ep.bias_dev = bias->data_ptr<float>();
  }
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_cuda() && residual->sizes() == y.sizes() &&
                    residual->strides() == y.strides() && residual->scalar_type() == y.scalar_type(),
                "residual must match the output's shape, dtype and memory layout");
    ep.residual_dev = residual->data_ptr();
  }
  return ep;
}

Tensor octree_conv_fused(Tensor data_in, Tensor weights, Tensor octree, int depth, int num_output,
                         vector<int> kernel_size, int stride, c10::optional<Tensor> scale,
                         c10::optional<Tensor> bias, c10::optional<Tensor> residual, bool relu) {
  vector<int> ks = kernel3(kernel_size);
  TORCH_CHECK(num_output > 0, "The num_output should be larger than 0");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_conv: the octree must be a CUDA tensor");
  need_cuda(data_in, "octree_conv");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "octree_conv");
  ConvShape s = conv_shape(o, x, depth, ks, stride, "octree_conv");
  const int kdim = ks[0] * ks[1] * ks[2];
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32 &&
                  weights.numel() == (int64_t)num_output * x.C * kdim,
              "weights must be a float32 CUDA tensor of shape [Cout, Cin*K]");
  Tensor w = weights.contiguous();
  Tensor y = new_data(num_output, s.h_out, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, num_output, y);
  OCNN_CALL(ocnn_octree_conv(x.t.data_ptr(), w.data_ptr<float>(), y.data_ptr(), s.neigh, s.h_in,
                             s.h_out, x.C, num_output, ks.data(), stride, x.dtype, x.layout, &ep,
                             current_stream()));
  return y;
}

// OctreeConv(nempty=True), stride 1: data and result live on the non-empty nodes of `depth` only
// (pytorch/cpp/octree_conv.cpp:61-120 with non_empty_).
Tensor octree_conv_nempty(Tensor data_in, Tensor weights, Tensor octree, int depth, int num_output,
                          vector<int> kernel_size) {
  vector<int> ks = kernel3(kernel_size);
  TORCH_CHECK(num_output > 0, "The num_output should be larger than 0");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_conv: the octree must be a CUDA tensor");
  TORCH_CHECK(depth >= 1 && depth <= o.meta.depth, "octree_conv: depth ", depth, " outside the octree");
  need_cuda(data_in, "octree_conv");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "octree_conv");
  const int nne = o.meta.nnum_nempty[depth], nnum = o.meta.nnum[depth];
  TORCH_CHECK(x.H == nne, "octree_conv (nempty): data height ", x.H, " != non-empty node number ", nne);
  const int kdim = ks[0] * ks[1] * ks[2];
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32 &&
                  weights.numel() == (int64_t)num_output * x.C * kdim,
              "weights must be a float32 CUDA tensor of shape [Cout, Cin*K]");
  Tensor w = weights.contiguous();
  Tensor y = new_data(num_output, nne, x);
  const int32_t* child = level_ptr(o, OCNN_PROP_CHILD, depth, "octree_conv");
  Tensor ichild = torch::empty({std::max(nne, 1)}, x.t.options().dtype(torch::kInt32));
  OCNN_CALL(ocnn_octree_ichild(child, nnum, ichild.data_ptr<int32_t>(), current_stream()));
  const int32_t* neigh = kdim > 1 ? level_ptr(o, OCNN_PROP_NEIGH, depth, "octree_conv") : nullptr;
  OCNN_CALL(ocnn_octree_conv_nempty(x.t.data_ptr(), w.data_ptr<float>(), y.data_ptr(), neigh, child,
                                    ichild.data_ptr<int32_t>(), nne, x.C, num_output, ks.data(),
                                    x.dtype, x.layout, nullptr, current_stream()));
  return y;
}

Tensor octree_conv_general(Tensor data_in, Tensor weights, Tensor octree, int depth, int num_output,
                           vector<int> kernel_size, int stride, bool nempty, bool transposed,
                           c10::optional<Tensor> scale, c10::optional<Tensor> bias,
                           c10::optional<Tensor> residual, bool relu);

Tensor octree_conv(Tensor data_in, Tensor weights, Tensor octree, int depth, int num_output,
                   vector<int> kernel_size, int stride, bool nempty) {
  if (nempty && stride == 1)
    return octree_conv_nempty(data_in, weights, octree, depth, num_output, kernel_size);
  if (nempty)
    return octree_conv_general(data_in, weights, octree, depth, num_output, kernel_size, stride, true,
                               false, c10::nullopt, c10::nullopt, c10::nullopt, false);
  return octree_conv_fused(data_in, weights, octree, depth, num_output, kernel_size, stride,
                           c10::nullopt, c10::nullopt, c10::nullopt, false);
}

Tensor conv_pack_weights(Tensor weights, int cin, int cout, vector<int> kernel_size, int stride) {
  vector<int> ks = kernel3(kernel_size);
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32,
              "weights must be a float32 CUDA tensor");
  const int kdim = ks[0] * ks[1] * ks[2];
  TORCH_CHECK(weights.numel() == (int64_t)cout * cin * kdim, "weights must have Cout*Cin*K values");
  c10::cuda::CUDAGuard guard(weights.device());
  const size_t bytes = ocnn_conv_packed_weight_bytes(cin, cout, ks.data(), stride);
  TORCH_CHECK(bytes > 0, "this shape is not supported by the tensor-core convolution: ",
              ocnn_last_error());
  Tensor packed = torch::empty({(int64_t)bytes}, weights.options().dtype(torch::kUInt8));
  Tensor w = weights.contiguous();
  OCNN_CALL(ocnn_conv_pack_weights(w.data_ptr<float>(), packed.data_ptr(), cin, cout, ks.data(),
                                   stride, current_stream()));
  return packed;
}

Tensor octree_conv_tc(Tensor data_in, Tensor packed, Tensor octree, int depth, int num_output,
                      vector<int> kernel_size, int stride, c10::optional<Tensor> scale,
                      c10::optional<Tensor> bias, c10::optional<Tensor> residual, bool relu,
                      Tensor status) {
  vector<int> ks = kernel3(kernel_size);
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_conv_tc: the octree must be a CUDA tensor");
  need_cuda(data_in, "octree_conv_tc");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "octree_conv_tc");
  TORCH_CHECK(x.dtype == OCNN_BF16 && (x.layout == OCNN_NODE_MAJOR || x.C == 1 || x.H == 1),
              "octree_conv_tc takes bfloat16 channels_last data (float16: octree_conv_tc_general)");
  x.layout = OCNN_NODE_MAJOR;
  ConvShape s = conv_shape(o, x, depth, ks, stride, "octree_conv_tc");
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == torch::kUInt8 &&
                  (size_t)packed.numel() ==
                      ocnn_conv_packed_weight_bytes(x.C, num_output, ks.data(), stride),
              "packed weights do not match this convolution's shape");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32 && status.numel() >= 1,
              "status must be an int32 CUDA tensor");
  Tensor y = new_data(num_output, s.h_out, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, num_output, y);
  OCNN_CALL(ocnn_octree_conv_tc(x.t.data_ptr(), packed.data_ptr(), y.data_ptr(), s.neigh, s.h_in,
                                s.h_out, x.C, num_output, ks.data(), stride, &ep,
                                status.data_ptr<int32_t>(), current_stream()));
  return y;
}

// ocnn_conv_tc_wait_selftest: [code of the expired wait, second waiter stopped] on the current device.
Tensor conv_tc_wait_selftest() {
  Tensor status = torch::zeros({2}, torch::dtype(torch::kInt32).device(torch::kCUDA));
  OCNN_CALL(ocnn_conv_tc_wait_selftest(status.data_ptr<int32_t>(), current_stream()));
  return status;
}

// Tensor-core convolution on the non-empty nodes only (nempty = True, stride 1).
Tensor conv_pack_weights_nempty(Tensor weights, int cin, int cout, vector<int> kernel_size) {
  vector<int> ks = kernel3(kernel_size);
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32,
              "weights must be a float32 CUDA tensor");
  const int kdim = ks[0] * ks[1] * ks[2];
  TORCH_CHECK(weights.numel() == (int64_t)cout * cin * kdim, "weights must have Cout*Cin*K values");
  c10::cuda::CUDAGuard guard(weights.device());
  const size_t bytes = ocnn_conv_packed_weight_bytes_nempty(cin, cout, ks.data());
  TORCH_CHECK(bytes > 0, "this shape is not supported by the tensor-core convolution: ",
              ocnn_last_error());
  Tensor packed = torch::empty({(int64_t)bytes}, weights.options().dtype(torch::kUInt8));
  Tensor w = weights.contiguous();
  OCNN_CALL(ocnn_conv_pack_weights_nempty(w.data_ptr<float>(), packed.data_ptr(), cin, cout,
                                          ks.data(), current_stream()));
  return packed;
}

Tensor octree_conv_tc_nempty(Tensor data_in, Tensor packed, Tensor octree, int depth, int num_output,
                             vector<int> kernel_size, c10::optional<Tensor> scale,
                             c10::optional<Tensor> bias, c10::optional<Tensor> residual, bool relu,
                             Tensor status) {
  vector<int> ks = kernel3(kernel_size);
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_conv_tc_nempty: the octree must be a CUDA tensor");
  TORCH_CHECK(depth >= 1 && depth <= o.meta.depth, "octree_conv_tc_nempty: depth ", depth,
              " outside the octree");
  need_cuda(data_in, "octree_conv_tc_nempty");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "octree_conv_tc_nempty");
  TORCH_CHECK(x.dtype == OCNN_BF16 && (x.layout == OCNN_NODE_MAJOR || x.C == 1 || x.H == 1),
              "octree_conv_tc_nempty takes bfloat16 channels_last data");
  x.layout = OCNN_NODE_MAJOR;
  const int nne = o.meta.nnum_nempty[depth], nnum = o.meta.nnum[depth];
  TORCH_CHECK(x.H == nne, "octree_conv_tc_nempty: data height ", x.H, " != non-empty node number ", nne);
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == torch::kUInt8 &&
                  (size_t)packed.numel() == ocnn_conv_packed_weight_bytes_nempty(x.C, num_output, ks.data()),
              "packed weights do not match this convolution's shape");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32 && status.numel() >= 1,
              "status must be an int32 CUDA tensor");
  Tensor y = new_data(num_output, nne, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, num_output, y);
  const int32_t* child = level_ptr(o, OCNN_PROP_CHILD, depth, "octree_conv_tc_nempty");
  Tensor ichild = torch::empty({std::max(nne, 1)}, x.t.options().dtype(torch::kInt32));
  OCNN_CALL(ocnn_octree_ichild(child, nnum, ichild.data_ptr<int32_t>(), current_stream()));
  const int kdim = ks[0] * ks[1] * ks[2];
  const int32_t* neigh = kdim > 1 ? level_ptr(o, OCNN_PROP_NEIGH, depth, "octree_conv_tc_nempty") : nullptr;
  OCNN_CALL(ocnn_octree_conv_tc_nempty(x.t.data_ptr(), packed.data_ptr(), y.data_ptr(), neigh, child,
                                       ichild.data_ptr<int32_t>(), nne, x.C, num_output, ks.data(),
                                       &ep, status.data_ptr<int32_t>(), current_stream()));
  return y;
}

// ---- every OctreeConv / OctreeDeconv forward (stride 1 or 2, nempty or not) -----------------------
// Row counts and level pointers as OctreeConvTH::setup_op / OctreeBaseConv::reshape derive them
// (pytorch/cpp/octree_conv.cpp:61-120, octree/octree/octree_conv.cpp:48-122).
struct Geometry {
  ocnn_conv_geometry g;
  Tensor ichild;      // keeps the inverse child table alive for the launch
};

Geometry make_geometry(const OctreeRef& o, const DataRef& x, int depth, const vector<int>& ks,
                       int stride, bool nempty, bool transposed, const char* what) {
  TORCH_CHECK(depth > 0 && depth <= o.meta.depth, what, ": The depth should be in (0, octree depth]");
  TORCH_CHECK(stride == 1 || stride == 2, "Unsupport stride");
  const ocnn_octree_meta& m = o.meta;
  const bool on_nempty = nempty || (transposed && stride == 2);
  TORCH_CHECK(x.H == (on_nempty ? m.nnum_nempty[depth] : m.nnum[depth]), what, ": data height ", x.H,
              " != ", on_nempty ? "non-empty " : "", "node number ",
              on_nempty ? m.nnum_nempty[depth] : m.nnum[depth], ", d: ", depth, ", channel_in: ", x.C);
  int work_depth = depth, top_depth = depth;
  if (stride == 2) {
    if (transposed) work_depth = top_depth = depth + 1; else top_depth = depth - 1;
    TORCH_CHECK(top_depth >= 0 && top_depth <= m.depth, what, ": the output level ", top_depth,
                " is outside the octree");
  }
  Geometry out;
  memset(&out.g, 0, sizeof(out.g));
  out.g.transposed = transposed ? 1 : 0;
  out.g.stride = stride;
  out.g.nempty = nempty ? 1 : 0;
  out.g.h_in = x.H;
  if (stride == 2 && !transposed) out.g.h_out = m.nnum[depth] / 8;
  else out.g.h_out = nempty ? m.nnum_nempty[top_depth] : m.nnum[top_depth];
  if (stride == 2 && !transposed)
    TORCH_CHECK(out.g.h_out == m.nnum_nempty[depth - 1], what, ": inconsistent octree");
  const bool identity = ks[0] * ks[1] * ks[2] == 1 && stride == 1;
  if (!identity) {
    out.g.neigh_dev = level_ptr(o, OCNN_PROP_NEIGH, work_depth, what);
    if (nempty) {
      out.g.child_dev = level_ptr(o, OCNN_PROP_CHILD, work_depth, what);
      out.ichild = make_ichild(o, work_depth, x.t.options(), what);
      out.g.ichild_dev = out.ichild.data_ptr<int32_t>();
    }
  }
  return out;
}

void check_weights(const Tensor& weights, int cin, int cout, int kdim) {
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32 &&
                  weights.numel() == (int64_t)cout * cin * kdim,
              "weights must be a float32 CUDA tensor of Cout*Cin*K values");
}

Tensor octree_conv_general(Tensor data_in, Tensor weights, Tensor octree, int depth, int num_output,
                           vector<int> kernel_size, int stride, bool nempty, bool transposed,
                           c10::optional<Tensor> scale, c10::optional<Tensor> bias,
                           c10::optional<Tensor> residual, bool relu) {
  const char* what = transposed ? "octree_deconv" : "octree_conv";
  vector<int> ks = kernel3(kernel_size);
  TORCH_CHECK(num_output > 0, "The num_output should be larger than 0");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, what, ": the octree must be a CUDA tensor");
  need_cuda(data_in, what);
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, what);
  Geometry geo = make_geometry(o, x, depth, ks, stride, nempty, transposed, what);
  check_weights(weights, x.C, num_output, ks[0] * ks[1] * ks[2]);
  Tensor w = weights.contiguous();
  Tensor y = new_data(num_output, geo.g.h_out, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, num_output, y);
  OCNN_CALL(ocnn_octree_conv_general(x.t.data_ptr(), w.data_ptr<float>(), y.data_ptr(), &geo.g, x.C,
                                     num_output, ks.data(), x.dtype, x.layout, &ep, current_stream()));
  return y;
}

Tensor octree_deconv(Tensor data_in, Tensor weights, Tensor octree, int depth, int num_output,
                     vector<int> kernel_size, int stride, bool nempty) {
  return octree_conv_general(data_in, weights, octree, depth, num_output, kernel_size, stride, nempty,
                             true, c10::nullopt, c10::nullopt, c10::nullopt, false);
}

Tensor conv_pack_weights_general(Tensor weights, int cin, int cout, vector<int> kernel_size,
                                 int stride, bool transposed, bool nempty, bool half) {
  vector<int> ks = kernel3(kernel_size);
  check_weights(weights, cin, cout, ks[0] * ks[1] * ks[2]);
  c10::cuda::CUDAGuard guard(weights.device());
  const size_t bytes = ocnn_conv_packed_weight_bytes_general(cin, cout, ks.data(), stride, transposed,
                                                             nempty);
  TORCH_CHECK(bytes > 0, "this shape is not supported by the tensor-core convolution: ",
              ocnn_last_error());
  Tensor packed = torch::empty({(int64_t)bytes}, weights.options().dtype(torch::kUInt8));
  Tensor w = weights.contiguous();
  OCNN_CALL(ocnn_conv_pack_weights_general(w.data_ptr<float>(), packed.data_ptr(), cin, cout, ks.data(),
                                           stride, transposed, nempty, half ? OCNN_F16 : OCNN_BF16,
                                           current_stream()));
  return packed;
}

Tensor octree_conv_tc_general(Tensor data_in, Tensor packed, Tensor octree, int depth, int num_output,
                              vector<int> kernel_size, int stride, bool nempty, bool transposed,
                              c10::optional<Tensor> scale, c10::optional<Tensor> bias,
                              c10::optional<Tensor> residual, bool relu, Tensor status) {
  const char* what = transposed ? "octree_deconv_tc" : "octree_conv_tc";
  vector<int> ks = kernel3(kernel_size);
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, what, ": the octree must be a CUDA tensor");
  need_cuda(data_in, what);
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, what);
  TORCH_CHECK(x.dtype != OCNN_F32 && (x.layout == OCNN_NODE_MAJOR || x.C == 1 || x.H == 1), what,
              " takes bfloat16 or float16 channels_last data");
  x.layout = OCNN_NODE_MAJOR;
  Geometry geo = make_geometry(o, x, depth, ks, stride, nempty, transposed, what);
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == torch::kUInt8 &&
                  (size_t)packed.numel() == ocnn_conv_packed_weight_bytes_general(
                                                x.C, num_output, ks.data(), stride, transposed, nempty),
              "packed weights do not match this convolution's shape");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32 && status.numel() >= 1,
              "status must be an int32 CUDA tensor");
  Tensor y = new_data(num_output, geo.g.h_out, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, num_output, y);
  OCNN_CALL(ocnn_octree_conv_tc_general(x.t.data_ptr(), packed.data_ptr(), y.data_ptr(), &geo.g, x.C,
                                        num_output, ks.data(), x.dtype, &ep,
                                        status.data_ptr<int32_t>(), current_stream()));
  return y;
}

// ---- gradients (pytorch/cpp/octree_conv.cpp:159-189, 219-253, 262-298; octree_pool.cpp:36-95) ---------
// Returns {gradient of the data, gradient of the weights} of OctreeConv (deconv = false) or
// OctreeDeconv (deconv = true) given the gradient of its output.  fp32.
vector<Tensor> conv_grad_impl(Tensor data_in, Tensor weights, Tensor octree, Tensor grad_in, int depth,
                              int num_output, vector<int> kernel_size, int stride, bool nempty,
                              bool deconv) {
  const char* what = deconv ? "octree_deconv_grad" : "octree_conv_grad";
  vector<int> ks = kernel3(kernel_size);
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, what, ": the octree must be a CUDA tensor");
  need_cuda(data_in, what);
  need_cuda(grad_in, what);
  c10::cuda::CUDAGuard guard(data_in.device());
  TORCH_CHECK(data_in.scalar_type() == torch::kFloat32 && grad_in.scalar_type() == torch::kFloat32,
              what, ": float32 data only");
  DataRef x = get_data(data_in, what);
  DataRef gy = get_data(x.layout == OCNN_NODE_MAJOR ? grad_in.contiguous(at::MemoryFormat::ChannelsLast)
                                                    : grad_in.contiguous(), what);
  const int kdim = ks[0] * ks[1] * ks[2];
  check_weights(weights, x.C, num_output, kdim);
  TORCH_CHECK(gy.C == num_output, what, ": the gradient has ", gy.C, " channels, expected ", num_output);
  Tensor w = weights.contiguous();
  // forward geometry: checks the data height and gives the output height
  Geometry fwd = make_geometry(o, x, depth, ks, stride, nempty, deconv, what);
  TORCH_CHECK(gy.H == fwd.g.h_out, what, ": the gradient has ", gy.H, " rows, expected ", fwd.g.h_out);
  // data gradient: the transposed operator with the same weights, from the output level back
  const int back_depth = stride == 1 ? depth : (deconv ? depth + 1 : depth - 1);
  Geometry back = make_geometry(o, gy, back_depth, ks, stride, nempty, !deconv, what);
  TORCH_CHECK(back.g.h_out == x.H, what, ": inconsistent octree");
  Tensor gx = new_data(x.C, x.H, x);
  OCNN_CALL(ocnn_octree_conv_general(gy.t.data_ptr(), w.data_ptr<float>(), gx.data_ptr(), &back.g, gy.C,
                                     x.C, ks.data(), OCNN_F32, x.layout, nullptr, current_stream()));
  // weight gradient: reduction over the rows of the convolution-type column matrix
  Tensor gw = torch::empty_like(w);
  const Geometry& conv_geo = deconv ? back : fwd;
  const DataRef& a = deconv ? x : gy;      // the operand with one row per column-matrix row
  const DataRef& src = deconv ? gy : x;    // the operand that is gathered
  OCNN_CALL(ocnn_octree_conv_weight_grad(a.t.data_ptr<float>(), src.t.data_ptr<float>(),
                                         gw.data_ptr<float>(), &conv_geo.g, a.C, src.C, ks.data(),
                                         x.layout, current_stream()));
  return {gx, gw};
}

vector<Tensor> octree_conv_grad(Tensor data_in, Tensor weights, Tensor octree, Tensor grad_in, int depth,
                                int num_output, vector<int> kernel_size, int stride, bool nempty) {
  return conv_grad_impl(data_in, weights, octree, grad_in, depth, num_output, kernel_size, stride,
                        nempty, false);
}

vector<Tensor> octree_deconv_grad(Tensor data_in, Tensor weights, Tensor octree, Tensor grad_in,
                                  int depth, int num_output, vector<int> kernel_size, int stride,
                                  bool nempty) {
  return conv_grad_impl(data_in, weights, octree, grad_in, depth, num_output, kernel_size, stride,
                        nempty, true);
}

Tensor octree_max_unpool(Tensor top_data, Tensor mask, Tensor octree, int depth) {
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(depth > 1 && depth <= o.meta.depth, "octree_max_unpool: depth out of range");
  need_cuda(top_data, "octree_max_unpool");
  c10::cuda::CUDAGuard guard(top_data.device());
  TORCH_CHECK(top_data.scalar_type() == torch::kFloat32, "octree_max_unpool: float32 data only");
  DataRef t = get_data(top_data, "octree_max_unpool");
  TORCH_CHECK(t.H == o.meta.nnum_nempty[depth - 1], "octree_max_unpool: data height ", t.H,
              " != non-empty node number ", o.meta.nnum_nempty[depth - 1]);
  TORCH_CHECK(mask.is_cuda() && mask.scalar_type() == torch::kInt32 && mask.sizes() == top_data.sizes(),
              "octree_max_unpool: mask must be an int32 CUDA tensor shaped like the data");
  Tensor m = t.layout == OCNN_NODE_MAJOR ? mask.contiguous(at::MemoryFormat::ChannelsLast) : mask.contiguous();
  Tensor btm = new_data(t.C, t.H * 8, t);
  OCNN_CALL(ocnn_octree_max_unpool(t.t.data_ptr<float>(), m.data_ptr<int32_t>(), btm.data_ptr<float>(),
                                   t.C, t.H, t.layout, current_stream()));
  return btm;
}

Tensor octree_mask_pool(Tensor btm_data, Tensor mask, Tensor octree, int depth) {
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(depth > 1 && depth <= o.meta.depth, "octree_mask_pool: depth out of range");
  need_cuda(btm_data, "octree_mask_pool");
  c10::cuda::CUDAGuard guard(btm_data.device());
  TORCH_CHECK(btm_data.scalar_type() == torch::kFloat32, "octree_mask_pool: float32 data only");
  DataRef b = get_data(btm_data, "octree_mask_pool");
  TORCH_CHECK(b.H == o.meta.nnum[depth], "octree_mask_pool: data height ", b.H, " != node number ",
              o.meta.nnum[depth]);
  const int top_h = b.H >> 3;
  TORCH_CHECK(mask.is_cuda() && mask.scalar_type() == torch::kInt32 && mask.dim() == 4 &&
                  mask.size(1) == b.C && mask.size(2) == top_h,
              "octree_mask_pool: mask must be an int32 CUDA tensor [1, C, H/8, 1]");
  Tensor m = b.layout == OCNN_NODE_MAJOR ? mask.contiguous(at::MemoryFormat::ChannelsLast) : mask.contiguous();
  Tensor top = new_data(b.C, top_h, b);
  OCNN_CALL(ocnn_octree_mask_pool(b.t.data_ptr<float>(), m.data_ptr<int32_t>(), top.data_ptr<float>(),
                                  b.C, top_h, b.layout, current_stream()));
  return top;
}

// ---- 1x1x1 convolution without an octree -------------------------------------------------------------
// The reference's OctreeConv1x1 is a torch Conv1d over [1,C,H] (pytorch/ocnn/modules.py:71-83): a
// per-node matrix product that needs no octree.  weights: float32 [Cout, Cin].
Tensor pointwise_conv(Tensor data_in, Tensor weights, c10::optional<Tensor> scale,
                      c10::optional<Tensor> bias, c10::optional<Tensor> residual, bool relu) {
  need_cuda(data_in, "pointwise_conv");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "pointwise_conv");
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32 && weights.numel() > 0 &&
                  weights.numel() % x.C == 0, "weights must be a float32 CUDA tensor [Cout, Cin]");
  const int cout = (int)(weights.numel() / x.C);
  Tensor w = weights.contiguous();
  Tensor y = new_data(cout, x.H, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, cout, y);
  const int ks[3] = {1, 1, 1};
  OCNN_CALL(ocnn_octree_conv(x.t.data_ptr(), w.data_ptr<float>(), y.data_ptr(), nullptr, x.H, x.H, x.C,
                             cout, ks, 1, x.dtype, x.layout, &ep, current_stream()));
  return y;
}

Tensor pointwise_conv_tc(Tensor data_in, Tensor packed, int num_output, c10::optional<Tensor> scale,
                         c10::optional<Tensor> bias, c10::optional<Tensor> residual, bool relu,
                         Tensor status) {
  need_cuda(data_in, "pointwise_conv_tc");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "pointwise_conv_tc");
  TORCH_CHECK(x.dtype != OCNN_F32 && (x.layout == OCNN_NODE_MAJOR || x.C == 1 || x.H == 1),
              "pointwise_conv_tc takes bfloat16 or float16 channels_last data");
  x.layout = OCNN_NODE_MAJOR;
  const int ks[3] = {1, 1, 1};
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == torch::kUInt8 &&
                  (size_t)packed.numel() == ocnn_conv_packed_weight_bytes(x.C, num_output, ks, 1),
              "packed weights do not match this convolution's shape");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32 && status.numel() >= 1,
              "status must be an int32 CUDA tensor");
  Tensor y = new_data(num_output, x.H, x);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, num_output, y);
  ocnn_conv_geometry g;
  memset(&g, 0, sizeof(g));
  g.stride = 1; g.h_in = x.H; g.h_out = x.H;
  OCNN_CALL(ocnn_octree_conv_tc_general(x.t.data_ptr(), packed.data_ptr(), y.data_ptr(), &g, x.C,
                                        num_output, ks, x.dtype, &ep, status.data_ptr<int32_t>(),
                                        current_stream()));
  return y;
}

// 1x1x1 convolution over the concatenated channels of two tensors of the same rows: the sum of a
// residual block's conv1x1b and its shortcut conv1x1c (pytorch/ocnn/modules.py OctreeResBlock) in
// one launch; `packed` = conv_pack_weights of [Wb | Wc] with cin = Cb + Cc.
Tensor pointwise_conv_tc_pair(Tensor data_a, Tensor data_b, Tensor packed, int num_output,
                              c10::optional<Tensor> scale, c10::optional<Tensor> bias,
                              c10::optional<Tensor> residual, bool relu, Tensor status) {
  need_cuda(data_a, "pointwise_conv_tc_pair");
  need_cuda(data_b, "pointwise_conv_tc_pair");
  c10::cuda::CUDAGuard guard(data_a.device());
  DataRef xa = get_data(data_a, "pointwise_conv_tc_pair");
  DataRef xb = get_data(data_b, "pointwise_conv_tc_pair");
  TORCH_CHECK(xa.dtype != OCNN_F32 && xa.dtype == xb.dtype &&
                  (xa.layout == OCNN_NODE_MAJOR || xa.C == 1 || xa.H == 1) &&
                  (xb.layout == OCNN_NODE_MAJOR || xb.C == 1 || xb.H == 1),
              "pointwise_conv_tc_pair takes two bfloat16 or two float16 channels_last tensors");
  TORCH_CHECK(xa.H == xb.H, "pointwise_conv_tc_pair: the inputs have ", xa.H, " and ", xb.H, " rows");
  xa.layout = OCNN_NODE_MAJOR;
  const int ks[3] = {1, 1, 1};
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == torch::kUInt8 &&
                  (size_t)packed.numel() == ocnn_conv_packed_weight_bytes(xa.C + xb.C, num_output, ks, 1),
              "packed weights do not match this convolution's shape");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32 && status.numel() >= 1,
              "status must be an int32 CUDA tensor");
  Tensor y = new_data(num_output, xa.H, xa);
  ocnn_conv_epilogue ep = make_epilogue(scale, bias, residual, relu, num_output, y);
  OCNN_CALL(ocnn_octree_conv_tc_pair(xa.t.data_ptr(), xa.C, xb.t.data_ptr(), xb.C, packed.data_ptr(),
                                     y.data_ptr(), xa.H, num_output, xa.dtype, &ep,
                                     status.data_ptr<int32_t>(), current_stream()));
  return y;
}

// FullOctreeGlobalPool + Linear (pytorch/ocnn/octree_pool.py:106-115, resnet.py:18-21) in one
// launch: data [1, C, batch * per, 1] 16-bit channels_last over a full level -> [batch, nout] fp32.
Tensor global_pool_fc(Tensor data_in, Tensor weights, c10::optional<Tensor> bias, int batch) {
  need_cuda(data_in, "global_pool_fc");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "global_pool_fc");
  TORCH_CHECK(x.dtype != OCNN_F32 && (x.layout == OCNN_NODE_MAJOR || x.C == 1 || x.H == 1),
              "global_pool_fc takes bfloat16 or float16 channels_last data");
  TORCH_CHECK(batch > 0 && x.H % batch == 0, "global_pool_fc: ", x.H, " rows for a batch of ", batch);
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32 && weights.dim() == 2 &&
                  weights.size(1) == x.C, "global_pool_fc: weights float32 [nout, C]");
  Tensor w = weights.contiguous();
  const int nout = (int)w.size(0);
  Tensor b;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == torch::kFloat32 && bias->numel() == nout,
                "global_pool_fc: bias float32 [nout]");
    b = bias->contiguous();
  }
  Tensor out = torch::empty({batch, nout}, data_in.options().dtype(torch::kFloat32).memory_format(c10::MemoryFormat::Contiguous));
  OCNN_CALL(ocnn_global_pool_fc(x.t.data_ptr(), w.data_ptr<float>(), b.defined() ? b.data_ptr<float>() : nullptr,
                                out.data_ptr<float>(), batch, x.H / batch, x.C, nout, x.dtype,
                                current_stream()));
  return out;
}

// ---- keys, search, interpolation, alignment (pytorch/cpp/octree_key.cpp, octree_align.cpp) ------------
// The reference's binding is compiled with 64-bit keys only (pytorch/cpp/octree_key.cpp:1-3), so
// key tensors are int64; a 32-bit-key octree is rejected here with a message.
void need_key64(const OctreeRef& o, const char* what) {
  TORCH_CHECK(o.meta.key_bits == 64, what, ": int64 key tensors need an octree with 64-bit keys "
              "(this one has 32-bit keys)");
}

Tensor octree_encode_key(Tensor xyz) {
  TORCH_CHECK(xyz.dim() == 2, "The dim of input tensor must be 2.");
  TORCH_CHECK(xyz.size(1) == 4, "The channel of input tensor must be 4.");
  TORCH_CHECK(xyz.scalar_type() == torch::kInt16, "octree_encode_key takes an int16 tensor");
  return xyz.contiguous().view(torch::kInt64).reshape({xyz.size(0)}).clone();
}

Tensor octree_decode_key(Tensor key) {
  TORCH_CHECK(key.dim() == 1, "The dim of input tensor must be 1.");
  TORCH_CHECK(key.scalar_type() == torch::kInt64, "octree_decode_key takes an int64 tensor");
  return key.contiguous().view(torch::kInt16).reshape({key.size(0), 4}).clone();
}

Tensor convert_key(Tensor in, int depth, bool to_key, const char* what) {
  TORCH_CHECK(in.scalar_type() == torch::kInt64 && in.numel() >= 1, what,
              ": The numel of the input int64 tensor must be larger than 1.");
  TORCH_CHECK(in.is_cuda(), what, ": the tensor must be a CUDA tensor (there is no CPU path)");
  c10::cuda::CUDAGuard guard(in.device());
  Tensor src = in.contiguous();
  Tensor out = torch::empty_like(src);
  OCNN_CALL(ocnn_convert_key(src.data_ptr(), out.data_ptr(), src.numel(), depth, 64, to_key ? 1 : 0,
                             current_stream()));
  return out;
}
Tensor octree_xyz2key(Tensor xyz, int depth) { return convert_key(xyz, depth, true, "octree_xyz2key"); }
Tensor octree_key2xyz(Tensor key, int depth) { return convert_key(key, depth, false, "octree_key2xyz"); }

// The ascending Morton keys of a level: its Key block (converted when the octree stores xyz), or the
// keys of its non-empty nodes only.  `hold` keeps temporaries alive.
const void* level_keys(const OctreeRef& o, const Tensor& octree, int depth, bool nempty, int* n_key,
                       vector<Tensor>& hold, const char* what) {
  TORCH_CHECK(depth >= 1 && depth <= o.meta.depth, what, ": depth ", depth, " outside the octree");
  const int64_t off = ocnn_prop_offset(&o.meta, OCNN_PROP_KEY, depth);
  TORCH_CHECK(off >= 0, what, ": the octree has no keys at depth ", depth);
  const void* keys = o.base + off;
  *n_key = o.meta.nnum[depth];
  const int kb = o.meta.key_bits / 8;
  auto opts = octree.options().dtype(torch::kUInt8);
  if (nempty) {
    const int nne = o.meta.nnum_nempty[depth];
    Tensor t = torch::zeros({(int64_t)std::max(nne, 1) * kb}, opts);
    OCNN_CALL(ocnn_key_depad(keys, level_ptr(o, OCNN_PROP_CHILD, depth, what), *n_key, t.data_ptr(),
                             o.meta.key_bits, current_stream()));
    hold.push_back(t);
    keys = t.data_ptr();
    *n_key = nne;
  }
  if (o.meta.key2xyz) {
    Tensor t = torch::empty({(int64_t)std::max(*n_key, 1) * kb}, opts);
    OCNN_CALL(ocnn_convert_key(keys, t.data_ptr(), *n_key, depth, o.meta.key_bits, 1, current_stream()));
    hold.push_back(t);
    keys = t.data_ptr();
  }
  return keys;
}

Tensor octree_search_key(Tensor key, Tensor octree, int depth, bool key_is_xyz, bool nempty) {
  TORCH_CHECK(key.scalar_type() == torch::kInt64 && key.numel() >= 1,
              "The numel of the input tensor must be larger than 1.");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda && key.is_cuda(), "octree_search_key: key and octree must be CUDA tensors");
  need_key64(o, "octree_search_key");
  c10::cuda::CUDAGuard guard(key.device());
  Tensor q = key.contiguous();
  vector<Tensor> hold;
  int n_key = 0;
  const void* keys = level_keys(o, octree, depth, nempty, &n_key, hold, "octree_search_key");
  Tensor idx = torch::empty({q.numel()}, q.options().dtype(torch::kInt32));
  OCNN_CALL(ocnn_search_key(keys, n_key, q.data_ptr(), q.numel(), idx.data_ptr<int32_t>(),
                            key_is_xyz ? 1 : 0, depth, 64, current_stream()));
  return idx;
}

// OctreeInterp in one kernel: data [1,C,H,1] at `depth` sampled at pts [N,4] = (x,y,z in
// [0, 2^depth], batch id).  method: "nearest" or "linear".  Returns [1,C,N,1].
Tensor octree_interp(Tensor data_in, Tensor octree, int depth, Tensor pts, string method, bool nempty) {
  TORCH_CHECK(method == "nearest" || method == "linear", "octree_interp: unknown method ", method);
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "octree_interp: the octree must be a CUDA tensor");
  need_cuda(data_in, "octree_interp");
  c10::cuda::CUDAGuard guard(data_in.device());
  DataRef x = get_data(data_in, "octree_interp");
  TORCH_CHECK(pts.is_cuda() && pts.dim() == 2 && pts.size(1) == 4, "octree_interp: pts must be a CUDA "
              "tensor of shape [N, 4]");
  Tensor p = pts.to(torch::kFloat32).contiguous();
  vector<Tensor> hold;
  int n_key = 0;
  const void* keys = level_keys(o, octree, depth, nempty, &n_key, hold, "octree_interp");
  TORCH_CHECK(x.H == n_key, "octree_interp: data height ", x.H, " != ", nempty ? "non-empty " : "",
              "node number ", n_key);
  const int64_t n = p.size(0);
  Tensor out = new_data(x.C, (int)n, x);
  OCNN_CALL(ocnn_octree_interp(x.t.data_ptr(), out.data_ptr(), p.data_ptr<float>(), keys, n_key, x.C,
                               x.H, n, depth, o.meta.key_bits, method == "linear" ? 1 : 0, x.dtype,
                               x.layout, current_stream()));
  return out;
}

vector<Tensor> octree_align(Tensor src_data, Tensor src_octree, Tensor des_octree, int depth) {
  OctreeRef so = get_octree(src_octree), dso = get_octree(des_octree);
  TORCH_CHECK(so.cuda && dso.cuda, "octree_align: the octrees must be CUDA tensors");
  TORCH_CHECK(so.meta.key_bits == dso.meta.key_bits, "octree_align: the octrees differ in key width");
  need_cuda(src_data, "octree_align");
  c10::cuda::CUDAGuard guard(src_data.device());
  DataRef x = get_data(src_data, "octree_align");
  TORCH_CHECK(depth >= 1 && depth <= so.meta.depth && depth <= dso.meta.depth,
              "octree_align: depth outside the octrees");
  TORCH_CHECK(so.meta.nnum[depth] == x.H, "octree_align: data height ", x.H, " != node number ",
              so.meta.nnum[depth]);
  vector<Tensor> hold;
  int n_src = 0, n_des = 0;
  const void* skeys = level_keys(so, src_octree, depth, false, &n_src, hold, "octree_align");
  const void* dkeys = level_keys(dso, des_octree, depth, false, &n_des, hold, "octree_align");
  Tensor idx = torch::empty({x.H}, x.t.options().dtype(torch::kInt32));
  OCNN_CALL(ocnn_search_key(dkeys, n_des, skeys, n_src, idx.data_ptr<int32_t>(), 0, depth,
                            so.meta.key_bits, current_stream()));
  Tensor des = new_data(x.C, n_des, x);
  OCNN_CALL(ocnn_octree_align(x.t.data_ptr(), des.data_ptr(), idx.data_ptr<int32_t>(), x.C, x.H, n_des,
                              x.dtype, x.layout, current_stream()));
  return {des, idx};
}

// Backward of octree_align: src_grad[., h] = idx[h] < 0 ? 0 : des_grad[., idx[h]]
// (align_backward_gpu, octree/octree/octree_nn.cu:734-752).
Tensor octree_align_grad(Tensor des_grad, Tensor idx_tensor) {
  need_cuda(des_grad, "octree_align_grad");
  c10::cuda::CUDAGuard guard(des_grad.device());
  DataRef g = get_data(des_grad, "octree_align_grad");
  TORCH_CHECK(idx_tensor.is_cuda() && idx_tensor.scalar_type() == torch::kInt32 && idx_tensor.dim() == 1,
              "octree_align_grad: idx must be a 1-D int32 CUDA tensor");
  Tensor idx = idx_tensor.contiguous();
  const int src_h = (int)idx.numel();
  Tensor out = new_data(g.C, src_h, g);
  OCNN_CALL(ocnn_octree_align_backward(g.t.data_ptr(), out.data_ptr(), idx.data_ptr<int32_t>(), g.C,
                                       src_h, g.H, g.dtype, g.layout, current_stream()));
  return out;
}

// ---- points ------------------------------------------------------------------------------------------
// Points buffer: 88-byte PointsInfo header (magic[16], pt_num, content_flags, channels[8],
// ptr_dis[8]) then xyz / normal / feature / label float arrays
// (octree/octree/points_info.h:8-40, points.cpp:96-150).
struct PointsHeader {
  char magic[16];
  int32_t pt_num, content_flags, channels[8], ptr_dis[8];
};
static_assert(sizeof(PointsHeader) == 88, "PointsInfo is 88 bytes");

Tensor points_new(Tensor pts, Tensor normals, Tensor features, Tensor labels) {
  auto flat = [](const Tensor& t) { return t.to(torch::kCPU, torch::kFloat32).contiguous().view({-1}); };
  Tensor p = flat(pts);
  const int64_t n = p.numel() / 3;
  TORCH_CHECK(n > 0 && p.numel() % 3 == 0, "points_new: pts must hold 3*N values, N > 0");
  Tensor blocks[4] = {p, flat(normals), flat(features), flat(labels)};
  PointsHeader h;
  memset(&h, 0, sizeof(h));
  strcpy(h.magic, "_POINTS_1.0_");
  h.pt_num = (int32_t)n;
  h.content_flags = 1;
  h.channels[0] = 3;
  if (blocks[1].numel() > 0) {
    TORCH_CHECK(blocks[1].numel() == 3 * n, "points_new: the channel of normal has to be 3");
    h.channels[1] = 3; h.content_flags |= 2;
  }
  if (blocks[2].numel() > 0) {
    TORCH_CHECK(blocks[2].numel() % n == 0, "points_new: features must hold C*N values");
    h.channels[2] = (int32_t)(blocks[2].numel() / n); h.content_flags |= 4;
  }
  if (blocks[3].numel() > 0) {
    TORCH_CHECK(blocks[3].numel() == n, "points_new: the channel of label has to be 1");
    h.channels[3] = 1; h.content_flags |= 8;
  }
  h.ptr_dis[0] = 88;
  for (int i = 1; i <= 4; ++i) h.ptr_dis[i] = h.ptr_dis[i - 1] + 4 * (int32_t)n * h.channels[i - 1];
  Tensor out = torch::empty({(int64_t)h.ptr_dis[4]}, torch::dtype(torch::kUInt8));
  uint8_t* o = out.data_ptr<uint8_t>();
  memcpy(o, &h, 88);
  for (int i = 0; i < 4; ++i)
    if (h.channels[i] > 0) memcpy(o + h.ptr_dis[i], blocks[i].data_ptr<float>(), 4 * n * h.channels[i]);
  return out;
}

// ---- transform_points / normalize_points / clip_points / bounding_sphere / points_property ----------
// (pytorch/cpp/transform_points.cpp:7-125, points_property.cpp:90-190).  CPU point buffers are
// uploaded; the results are CUDA tensors that points2octree takes as they are.
PointsHeader read_points_header(const Tensor& points) {
  TORCH_CHECK(points.scalar_type() == torch::kUInt8 && points.dim() == 1 && points.numel() >= 88,
              "a points tensor must be a 1-D uint8 tensor with an 88-byte header");
  Tensor head = points.slice(0, 0, 88).to(torch::kCPU).contiguous();
  PointsHeader h;
  memcpy(&h, head.data_ptr<uint8_t>(), 88);
  TORCH_CHECK(strncmp(h.magic, "_POINTS_1.0_", 13) == 0, "The version of points format is not _POINTS_1.0_.");
  TORCH_CHECK(h.pt_num > 0, "The pt_num_ should be larger than 0.");
  TORCH_CHECK((h.content_flags & 1) && h.channels[0] == 3, "points need xyz coordinates");
  TORCH_CHECK(h.ptr_dis[4] <= points.numel(), "the points tensor is shorter than its header says");
  return h;
}

float* points_block(Tensor& buf, const PointsHeader& h, int t) {
  return h.channels[t] > 0 ? reinterpret_cast<float*>(buf.data_ptr<uint8_t>() + h.ptr_dis[t]) : nullptr;
}

vector<float> three(vector<float> v, const char* what) {
  TORCH_CHECK(!v.empty() && v.size() <= 3, what, " must hold 1 to 3 values");
  while (v.size() < 3) v.push_back(v.back());
  return v;
}

// rotation_matrix(rot, angles), octree/octree/math_functions.cpp:148-158: Rx * Ry * Rz in the
// reference's column-major 3x3 product
void euler_rotation(const float* angle, float* rot) {
  // (the reference evaluates cos / sin in double and rounds the result)
  const float cx = (float)cos((double)angle[0]), sx = (float)sin((double)angle[0]);
  const float cy = (float)cos((double)angle[1]), sy = (float)sin((double)angle[1]);
  const float cz = (float)cos((double)angle[2]), sz = (float)sin((double)angle[2]);
  const float rx[9] = {1.f, 0, 0, 0, cx, sx, 0, -sx, cx};
  const float ry[9] = {cy, 0, -sy, 0, 1.f, 0, sy, 0, cy};
  const float rz[9] = {cz, sz, 0, -sz, cz, 0, 0, 0, 1.f};
  auto prod = [](float* C, const float* A, const float* B) {
    for (int n = 0; n < 3; ++n)
      for (int m = 0; m < 3; ++m) {
        C[n * 3 + m] = 0;
        for (int k = 0; k < 3; ++k) C[n * 3 + m] += A[k * 3 + m] * B[n * 3 + k];
      }
  };
  float tmp[9];
  prod(tmp, rx, ry);
  prod(rot, tmp, rz);
}

Tensor transform_points(Tensor data_in, vector<float> angle, vector<float> scale, vector<float> jitter,
                        float offset, string normal_axis) {
  PointsHeader h = read_points_header(data_in);
  Tensor out = data_in.to(torch::kCUDA).contiguous().clone();
  c10::cuda::CUDAGuard guard(out.device());
  angle = three(angle, "angle"); scale = three(scale, "scale"); jitter = three(jitter, "jitter");
  const float eps = 1.0e-10f;
  float rot[9];
  const bool do_rot = fabsf(angle[0]) > eps || fabsf(angle[1]) > eps || fabsf(angle[2]) > eps;
  if (do_rot) euler_rotation(angle.data(), rot);
  const bool do_jit = fabsf(jitter[0]) > eps || fabsf(jitter[1]) > eps || fabsf(jitter[2]) > eps;
  const bool do_scale = scale[0] != 1.0f || scale[1] != 1.0f || scale[2] != 1.0f;
  int orient = 0;
  if (normal_axis == "x") orient = 1;
  else if (normal_axis == "y") orient = 2;
  else if (normal_axis == "z") orient = 3;
  else if (normal_axis == "xyz") orient = 4;
  OCNN_CALL(ocnn_points_transform(points_block(out, h, 0), points_block(out, h, 1), h.pt_num, offset,
                                  do_rot ? rot : nullptr, do_jit ? jitter.data() : nullptr,
                                  do_scale ? scale.data() : nullptr, orient, current_stream()));
  return out;
}

Tensor normalize_points(Tensor data_in, float radius, vector<float> center) {
  TORCH_CHECK(radius >= 0.0f, "normalize_points: the radius must not be negative");
  TORCH_CHECK(center.size() == 3, "normalize_points: center must hold 3 values");
  PointsHeader h = read_points_header(data_in);
  Tensor out = data_in.to(torch::kCUDA).contiguous().clone();
  c10::cuda::CUDAGuard guard(out.device());
  const float dis[3] = {-center[0], -center[1], -center[2]};
  const bool do_shift = dis[0] != 0.0f || dis[1] != 0.0f || dis[2] != 0.0f;
  const float inv = 1.0f / radius;
  const float sc[3] = {inv, inv, inv};
  OCNN_CALL(ocnn_points_transform(points_block(out, h, 0), points_block(out, h, 1), h.pt_num, 0.f, nullptr,
                                  do_shift ? dis : nullptr, inv != 1.0f ? sc : nullptr, 0, current_stream()));
  return out;
}

vector<Tensor> clip_points(Tensor data_in, vector<float> bbmin, vector<float> bbmax) {
  TORCH_CHECK(bbmin.size() == 3 && bbmax.size() == 3, "clip_points: bbmin / bbmax must hold 3 values");
  PointsHeader h = read_points_header(data_in);
  Tensor src = data_in.to(torch::kCUDA).contiguous();
  c10::cuda::CUDAGuard guard(src.device());
  Tensor out = src.clone();      // header and (for an all-inside cloud) every block already in place
  const float* sp[4]; float* dp[4]; int ch[4];
  for (int t = 0; t < 4; ++t) {
    ch[t] = h.channels[t];
    sp[t] = points_block(src, h, t);
    dp[t] = points_block(out, h, t);
  }
  Tensor mask = torch::empty({(int64_t)h.pt_num}, src.options().dtype(torch::kInt32));
  const size_t ws_bytes = ocnn_points_clip_workspace_bytes(h.pt_num);
  Tensor ws = torch::empty({(int64_t)ws_bytes}, src.options());
  int32_t* pt_num_dev = reinterpret_cast<int32_t*>(out.data_ptr<uint8_t>() + 16);   // PointsInfo::pt_num_
  OCNN_CALL(ocnn_points_clip(sp, dp, ch, h.pt_num, bbmin.data(), bbmax.data(), mask.data_ptr<int32_t>(),
                             pt_num_dev, ws.data_ptr(), ws_bytes, current_stream()));
  return {out, mask};
}

vector<float> bounding_sphere(Tensor data_in, string method) {
  TORCH_CHECK(method != "sphere", "bounding_sphere(method='sphere') needs the reference's external "
              "Miniball code and is not implemented; use method='box'");
  PointsHeader h = read_points_header(data_in);
  Tensor src = data_in.to(torch::kCUDA).contiguous();
  c10::cuda::CUDAGuard guard(src.device());
  const size_t ws_bytes = ocnn_points_bbox_workspace_bytes();
  Tensor ws = torch::empty({(int64_t)ws_bytes}, src.options());
  Tensor box = torch::empty({6}, src.options().dtype(torch::kFloat32));
  OCNN_CALL(ocnn_points_bbox(points_block(src, h, 0), h.pt_num, box.data_ptr<float>(), ws.data_ptr(),
                             ws_bytes, current_stream()));
  Tensor b = box.cpu();
  const float* p = b.data_ptr<float>();
  float radius = 0.f, center[3];
  for (int j = 0; j < 3; ++j) {
    center[j] = (p[3 + j] + p[j]) / 2.0f;
    const float width = (p[3 + j] - p[j]) / 2.0f;
    radius += width * width;
  }
  radius = sqrtf(radius + 1.0e-20f);
  return {radius, center[0], center[1], center[2]};
}

int points_prop_index(const string& property) {
  if (property == "xyz" || property == "xyzi") return 0;
  if (property == "normal") return 1;
  if (property == "feature") return 2;
  if (property == "label") return 3;
  TORCH_CHECK(false, "Unsupported Property: ", property);
  return -1;
}

Tensor points_property(Tensor points, string property) {
  PointsHeader h = read_points_header(points);
  const int t = points_prop_index(property);
  if (h.channels[t] == 0) return Tensor();
  Tensor buf = points.contiguous();
  return buf.slice(0, h.ptr_dis[t], h.ptr_dis[t] + (int64_t)4 * h.pt_num * h.channels[t])
      .clone().view(torch::kFloat32).view({h.pt_num, h.channels[t]});
}

Tensor points_batch_property(vector<Tensor> tensors, string property) {
  TORCH_CHECK(!tensors.empty(), "points_batch_property: empty input");
  vector<Tensor> parts;
  for (size_t i = 0; i < tensors.size(); ++i) {
    Tensor p = points_property(tensors[i], property);
    TORCH_CHECK(p.defined(), "The specified property does not exist.");
    if (property == "xyzi")
      p = torch::cat({p, torch::full({p.size(0), 1}, (double)i, p.options())}, 1);
    parts.push_back(p);
  }
  return torch::cat(parts, 0);
}

Tensor points_set_property(Tensor points_in, Tensor data, string property) {
  TORCH_CHECK(data.dim() == 2, "points_set_property: data must be [N, C]");
  PointsHeader h = read_points_header(points_in);
  const int t = points_prop_index(property);
  TORCH_CHECK(h.channels[t] > 0, "The property does not exist.");
  TORCH_CHECK(data.size(1) == h.channels[t], "The channel is wrong.");
  TORCH_CHECK(data.size(0) == h.pt_num, "The point number is wrong.");
  Tensor out = points_in.contiguous().clone();
  Tensor bytes = data.to(out.device(), torch::kFloat32).contiguous().view({-1}).view(torch::kUInt8);
  out.slice(0, h.ptr_dis[t], h.ptr_dis[t] + bytes.numel()).copy_(bytes);
  return out;
}

struct CloudInfo { int64_t byte_offset; PointsHeader h; };

void check_points_header(const PointsHeader& h, int64_t nbytes) {
  TORCH_CHECK(strncmp(h.magic, "_POINTS_1.0_", 13) == 0, "The version of points format is not _POINTS_1.0_.");
  TORCH_CHECK(h.pt_num > 0, "The pt_num_ should be larger than 0.");
  TORCH_CHECK((h.content_flags & 1) && h.channels[0] == 3, "points need xyz coordinates");
  TORCH_CHECK(h.ptr_dis[4] <= nbytes, "the points tensor is shorter than its header says");
}

struct BuildFlags {
  int depth, full_depth;
  bool node_dis, node_feature, split_label, adaptive;
  int adp_depth;
  float th_normal, th_distance;
  bool extrapolate, save_pts, key2xyz;
};

// Build the (merged or single) octree of clouds stored back to back in one CUDA uint8 buffer.
Tensor build_from_device(const Tensor& packed_dev, const vector<CloudInfo>& clouds,
                         const BuildFlags& f, bool merged) {
  TORCH_CHECK(!f.adaptive, "points2octree: adaptive octrees are not implemented");
  TORCH_CHECK(!f.node_feature, "points2octree: node_feature=True is not implemented");
  TORCH_CHECK(!f.extrapolate, "points2octree: extrapolate=True is not implemented");
  TORCH_CHECK(!f.key2xyz, "points2octree: key2xyz=True is not implemented");
  const int B = (int)clouds.size();
  const PointsHeader& h0 = clouds[0].h;
  vector<int32_t> offsets(B + 1, 0);
  vector<const float*> xyz(B), nrm(B), feat(B), lab(B);
  const uint8_t* base = packed_dev.data_ptr<uint8_t>();
  for (int b = 0; b < B; ++b) {
    const PointsHeader& h = clouds[b].h;
    TORCH_CHECK(h.content_flags == h0.content_flags && h.channels[1] == h0.channels[1] &&
                    h.channels[2] == h0.channels[2] && h.channels[3] == h0.channels[3],
                "all point clouds of a batch must carry the same properties");
    const uint8_t* p = base + clouds[b].byte_offset;
    TORCH_CHECK(((uintptr_t)p & 3) == 0, "point buffers must be 4-byte aligned");
    offsets[b + 1] = offsets[b] + h.pt_num;
    xyz[b] = reinterpret_cast<const float*>(p + h.ptr_dis[0]);
    nrm[b] = reinterpret_cast<const float*>(p + h.ptr_dis[1]);
    feat[b] = reinterpret_cast<const float*>(p + h.ptr_dis[2]);
    lab[b] = reinterpret_cast<const float*>(p + h.ptr_dis[3]);
  }
  ocnn_points_batch pb;
  pb.batch = B;
  pb.offsets_host = offsets.data();
  pb.xyz_dev = xyz.data();
  pb.normal_dev = (h0.content_flags & 2) ? nrm.data() : nullptr;
  pb.feature_dev = (h0.content_flags & 4) ? feat.data() : nullptr;
  pb.feature_channels = (h0.content_flags & 4) ? h0.channels[2] : 0;
  pb.label_dev = (h0.content_flags & 8) ? lab.data() : nullptr;
  ocnn_build_params prm;
  memset(&prm, 0, sizeof(prm));
  prm.depth = f.depth;
  prm.full_depth = f.full_depth < 1 ? 1 : f.full_depth;   // OctreeInfo::set_full_layer
  prm.key_bits = g_key_bits;
  prm.merged = merged ? 1 : 0;
  prm.node_dis = f.node_dis; prm.split_label = f.split_label; prm.save_pts = f.save_pts;
  prm.adp_depth = f.adp_depth; prm.th_normal = f.th_normal; prm.th_distance = f.th_distance;
  for (int j = 0; j < 3; ++j) { prm.bbmin[j] = -1.f; prm.bbmax[j] = 1.f; }

  const size_t ws_bytes = ocnn_octree_build_workspace_bytes(offsets[B], B, prm.depth, prm.full_depth);
  TORCH_CHECK(ws_bytes > 0, "points2octree: invalid depth / full_depth");
  auto opts = packed_dev.options();
  Tensor ws = torch::empty({(int64_t)ws_bytes}, opts);
  ocnn_octree_meta meta;
  OCNN_CALL(ocnn_octree_build_plan(&pb, &prm, ws.data_ptr(), ws_bytes, &meta, current_stream()));
  Tensor out = torch::empty({(int64_t)meta.ptr_dis[OCNN_PROP_COUNT]}, opts);
  uint8_t raw[OCNN_HEADER_BYTES];
  OCNN_CALL(ocnn_octree_build_emit(&pb, &prm, &meta, ws.data_ptr(), ws_bytes, out.data_ptr(),
                                   (size_t)out.numel(), raw, current_stream()));
  remember_header(out, meta, raw);   // later operators need no device->host copy of the header
  return out;
}

BuildFlags make_flags(int depth, int full_depth, bool node_dis, bool node_feature, bool split_label,
                      bool adaptive, int adp_depth, float th_normal, float th_distance,
                      bool extrapolate, bool save_pts, bool key2xyz) {
  return BuildFlags{depth, full_depth, node_dis, node_feature, split_label, adaptive, adp_depth,
                    th_normal, th_distance, extrapolate, save_pts, key2xyz};
}

// Pack CPU point buffers back to back (4-byte sizes keep every cloud aligned) and describe them.
// meta: int64 [B, 2] = (byte offset, byte size).  pin=True returns pinned memory for async H2D.
vector<Tensor> points_pack(vector<Tensor> points, bool pin) {
  TORCH_CHECK(!points.empty(), "points_pack: empty list");
  int64_t total = 0;
  for (auto& p : points) {
    TORCH_CHECK(!p.is_cuda() && p.scalar_type() == torch::kUInt8 && p.dim() == 1 && p.is_contiguous(),
                "points_pack takes CPU uint8 point buffers");
    total += (p.numel() + 3) / 4 * 4;
  }
  Tensor packed = torch::empty({total}, torch::dtype(torch::kUInt8).pinned_memory(pin));
  Tensor meta = torch::empty({(int64_t)points.size(), 2}, torch::dtype(torch::kInt64));
  int64_t at = 0;
  for (size_t b = 0; b < points.size(); ++b) {
    memcpy(packed.data_ptr<uint8_t>() + at, points[b].data_ptr<uint8_t>(), points[b].numel());
    meta.data_ptr<int64_t>()[2 * b] = at;
    meta.data_ptr<int64_t>()[2 * b + 1] = points[b].numel();
    at += (points[b].numel() + 3) / 4 * 4;
  }
  return {packed, meta};
}

// packed: all clouds back to back (CPU or CUDA); packed_host: the same bytes on the host when
// `packed` is a CUDA tensor (only the 88-byte headers are read from it), or undefined.
Tensor points2octree_packed(Tensor packed, Tensor meta, Tensor headers_host, int depth, int full_depth,
                            bool node_dis, bool node_feature, bool split_label, bool adaptive,
                            int adp_depth, float th_normal, float th_distance, bool extrapolate,
                            bool save_pts, bool key2xyz, bool merged) {
  TORCH_CHECK(packed.scalar_type() == torch::kUInt8 && packed.dim() == 1 && packed.is_contiguous(),
              "packed points must be a contiguous 1-D uint8 tensor");
  TORCH_CHECK(!meta.is_cuda() && meta.scalar_type() == torch::kInt64 && meta.dim() == 2 &&
                  meta.size(1) == 2 && meta.is_contiguous(), "meta must be a CPU int64 [B,2] tensor");
  const int B = (int)meta.size(0);
  TORCH_CHECK(!headers_host.is_cuda() && headers_host.scalar_type() == torch::kUInt8 &&
                  headers_host.is_contiguous() && headers_host.numel() == 88 * (int64_t)B,
              "headers_host must be a CPU uint8 tensor of 88*B bytes");
  vector<CloudInfo> clouds(B);
  for (int b = 0; b < B; ++b) {
    clouds[b].byte_offset = meta.data_ptr<int64_t>()[2 * b];
    memcpy(&clouds[b].h, headers_host.data_ptr<uint8_t>() + 88 * b, 88);
    check_points_header(clouds[b].h, meta.data_ptr<int64_t>()[2 * b + 1]);
    TORCH_CHECK(clouds[b].byte_offset >= 0 &&
                    clouds[b].byte_offset + meta.data_ptr<int64_t>()[2 * b + 1] <= packed.numel(),
                "meta describes bytes outside the packed tensor");
  }
  Tensor dev = packed;
  if (!packed.is_cuda()) dev = packed.to(torch::kCUDA, /*non_blocking=*/true);
  c10::cuda::CUDAGuard guard(dev.device());
  return build_from_device(dev, clouds,
                           make_flags(depth, full_depth, node_dis, node_feature, split_label, adaptive,
                                      adp_depth, th_normal, th_distance, extrapolate, save_pts, key2xyz),
                           merged);
}

Tensor headers_of(const vector<Tensor>& points) {
  Tensor headers = torch::empty({88 * (int64_t)points.size()}, torch::dtype(torch::kUInt8));
  for (size_t b = 0; b < points.size(); ++b) {
    const Tensor& p = points[b];
    TORCH_CHECK(p.scalar_type() == torch::kUInt8 && p.dim() == 1 && p.numel() >= 88,
                "a points tensor must be a 1-D uint8 tensor with an 88-byte header");
    Tensor head = p.slice(0, 0, 88).to(torch::kCPU).contiguous();   // D2H of 88 bytes for CUDA input
    memcpy(headers.data_ptr<uint8_t>() + 88 * b, head.data_ptr<uint8_t>(), 88);
  }
  return headers;
}

Tensor points2octree_list(vector<Tensor> points, const BuildFlags& f, bool merged) {
  TORCH_CHECK(!points.empty(), "points2octree: empty input");
  bool all_cpu = true;
  for (auto& p : points) all_cpu = all_cpu && !p.is_cuda();
  Tensor packed, meta;
  if (all_cpu) {
    for (auto& p : points) p = p.contiguous();
    auto pm = points_pack(points, false);
    packed = pm[0]; meta = pm[1];
  } else {
    // device inputs: concatenate on the device (padded to 4 bytes each)
    meta = torch::empty({(int64_t)points.size(), 2}, torch::dtype(torch::kInt64));
    vector<Tensor> parts;
    int64_t at = 0;
    for (size_t b = 0; b < points.size(); ++b) {
      Tensor p = points[b].to(torch::kCUDA).contiguous();
      const int64_t padded = (p.numel() + 3) / 4 * 4;
      meta.data_ptr<int64_t>()[2 * b] = at;
      meta.data_ptr<int64_t>()[2 * b + 1] = p.numel();
      parts.push_back(p);
      if (padded != p.numel()) parts.push_back(torch::zeros({padded - p.numel()}, p.options()));
      at += padded;
    }
    packed = parts.size() == 1 ? parts[0] : torch::cat(parts);
  }
  Tensor headers = headers_of(points);
  return points2octree_packed(packed, meta, headers, f.depth, f.full_depth, f.node_dis, f.node_feature,
                              f.split_label, f.adaptive, f.adp_depth, f.th_normal, f.th_distance,
                              f.extrapolate, f.save_pts, f.key2xyz, merged);
}

Tensor points2octree(Tensor points, int depth, int full_depth, bool node_dis, bool node_feature,
                     bool split_label, bool adaptive, int adp_depth, float th_normal,
                     float th_distance, bool extrapolate, bool save_pts, bool key2xyz) {
  return points2octree_list({points},
                            make_flags(depth, full_depth, node_dis, node_feature, split_label, adaptive,
                                       adp_depth, th_normal, th_distance, extrapolate, save_pts, key2xyz),
                            false);
}

Tensor points2octree_batch(vector<Tensor> points, int depth, int full_depth, bool node_dis,
                           bool node_feature, bool split_label, bool adaptive, int adp_depth,
                           float th_normal, float th_distance, bool extrapolate, bool save_pts,
                           bool key2xyz) {
  return points2octree_list(points,
                            make_flags(depth, full_depth, node_dis, node_feature, split_label, adaptive,
                                       adp_depth, th_normal, th_distance, extrapolate, save_pts, key2xyz),
                            true);
}

// ---- octree_batch -------------------------------------------------------------------------------------
Tensor octree_batch(vector<Tensor> tensors_in) {
  const int B = (int)tensors_in.size();
  TORCH_CHECK(B >= 1, "octree_batch: empty input");
  vector<Tensor> dev(B);
  vector<ocnn_octree_meta> metas(B);
  vector<const void*> ptrs(B);
  uint8_t first[OCNN_HEADER_BYTES];
  for (int b = 0; b < B; ++b) {
    OctreeRef o = get_octree(tensors_in[b].contiguous());
    metas[b] = o.meta;
    if (b == 0) memcpy(first, o.raw, sizeof(first));
    dev[b] = tensors_in[b].is_cuda() ? tensors_in[b].contiguous()
                                     : tensors_in[b].contiguous().to(torch::kCUDA, /*non_blocking=*/false);
    ptrs[b] = dev[b].data_ptr();
  }
  c10::cuda::CUDAGuard guard(dev[0].device());
  ocnn_octree_meta merged;
  OCNN_CALL(ocnn_octree_batch_meta(metas.data(), B, &merged));
  const size_t ws_bytes = ocnn_octree_batch_workspace_bytes(B, merged.depth);
  Tensor ws = torch::empty({(int64_t)ws_bytes}, dev[0].options());
  Tensor out = torch::empty({(int64_t)merged.ptr_dis[OCNN_PROP_COUNT]}, dev[0].options());
  uint8_t raw[OCNN_HEADER_BYTES];
  OCNN_CALL(ocnn_octree_batch(ptrs.data(), metas.data(), first, B, &merged, ws.data_ptr(), ws_bytes,
                              out.data_ptr(), raw, current_stream()));
  remember_header(out, merged, raw);
  return out;
}

// ---- octree_property ------------------------------------------------------------------------------------
Tensor octree_property(Tensor octree, string property, int depth) {
  OctreeRef o = get_octree(octree);
  const ocnn_octree_meta& m = o.meta;
  TORCH_CHECK(depth >= 0 && depth <= m.depth, "octree_property: depth out of range");
  const int nnum = depth > 0 ? m.nnum[depth] : m.nnum_cum[m.depth + 1];
  auto block = [&](int prop, int elem_bytes, int channel) {
    const int64_t off = ocnn_prop_offset(&m, prop, depth);
    TORCH_CHECK(off >= 0, "The ", property, " do not exist: d = ", depth);
    return octree.slice(0, off, off + (int64_t)nnum * channel * elem_bytes);
  };
  auto small = [&](const int32_t* src, int n) {
    Tensor t = torch::empty({n}, torch::dtype(torch::kInt32));
    memcpy(t.data_ptr<int32_t>(), src, sizeof(int32_t) * n);
    return t.to(octree.device());
  };
  if (property == "key" || property == "xyz" || property == "index") {
    const int kb = m.key_bits / 8;
    Tensor raw = block(OCNN_PROP_KEY, kb, 1);
    Tensor key = kb == 8 ? raw.view(torch::kInt64).clone()
                         : raw.view(torch::kInt32).to(torch::kInt64).bitwise_and(0xffffffffLL);
    if (property == "index") {
      Tensor idx = kb == 8 ? key.bitwise_right_shift(48).bitwise_and(0xffff)
                           : key.bitwise_right_shift(24).bitwise_and(0xff);
      return idx.to(torch::kInt32);
    }
    if ((property == "key") != (m.key2xyz == 0)) {
      // the octree stores the other form: convert (octree_property.cpp:58-75 of the reference)
      TORCH_CHECK(octree.is_cuda() && kb == 8, "octree_property('", property, "'): converting between "
                  "Morton keys and packed xyz needs a CUDA octree with 64-bit keys");
      c10::cuda::CUDAGuard guard(octree.device());
      Tensor out = torch::empty_like(key);
      OCNN_CALL(ocnn_convert_key(key.data_ptr(), out.data_ptr(), key.numel(), depth, 64,
                                 property == "key" ? 1 : 0, current_stream()));
      return out;
    }
    return key;
  }
  if (property == "child") return block(OCNN_PROP_CHILD, 4, 1).view(torch::kInt32).clone();
  if (property == "neigh")
    return block(OCNN_PROP_NEIGH, 4, 8).view(torch::kInt32).clone().view({nnum, 8});
  if (property == "feature") {
    const int ch = m.channels[OCNN_PROP_FEATURE];
    return block(OCNN_PROP_FEATURE, 4, ch).view(torch::kFloat32).clone().view({1, ch, nnum, 1});
  }
  if (property == "label") return block(OCNN_PROP_LABEL, 4, 1).view(torch::kFloat32).clone();
  if (property == "split") return block(OCNN_PROP_SPLIT, 4, 1).view(torch::kFloat32).clone();
  if (property == "node_num") return small(m.nnum + depth, depth > 0 ? 1 : m.depth + 1);
  if (property == "node_num_ne" || property == "node_num_nempty")
    return small(m.nnum_nempty + depth, depth > 0 ? 1 : m.depth + 1);
  if (property == "node_num_cum") return small(m.nnum_cum + depth, depth > 0 ? 1 : m.depth + 2);
  if (property == "batch_size") return small(&m.batch_size, 1);
  if (property == "depth") return small(&m.depth, 1);
  if (property == "full_depth") return small(&m.full_depth, 1);
  TORCH_CHECK(false, "Unsupport octree property: ", property);
  return Tensor();
}

// Host-side view of the header: ints only, no device access after the first call on a tensor.
vector<int64_t> octree_info(Tensor octree) {
  OctreeRef o = get_octree(octree);
  const ocnn_octree_meta& m = o.meta;
  vector<int64_t> out = {m.key_bits, m.batch_size, m.depth, m.full_depth};
  for (int d = 0; d < OCNN_MAX_DEPTH; ++d) out.push_back(m.nnum[d]);
  for (int d = 0; d < OCNN_MAX_DEPTH; ++d) out.push_back(m.nnum_nempty[d]);
  for (int p = 0; p < OCNN_PROP_COUNT; ++p) out.push_back(m.channels[p]);
  return out;
}

Tensor feature_node_major(Tensor octree, int c_pad, bool bf16, bool half) {
  TORCH_CHECK(!(bf16 && half), "feature_node_major: choose one of bf16 / half");
  OctreeRef o = get_octree(octree);
  TORCH_CHECK(o.cuda, "feature_node_major: the octree must be a CUDA tensor");
  const ocnn_octree_meta& m = o.meta;
  const int d = m.depth, ch = m.channels[OCNN_PROP_FEATURE];
  const int64_t off = ocnn_prop_offset(&m, OCNN_PROP_FEATURE, d);
  TORCH_CHECK(off >= 0 && ch > 0, "the octree has no features at its finest level");
  TORCH_CHECK(c_pad >= ch, "c_pad must be at least the feature channel count ", ch);
  c10::cuda::CUDAGuard guard(octree.device());
  auto opts = octree.options().dtype(bf16 ? torch::kBFloat16 : (half ? torch::kFloat16 : torch::kFloat32))
                  .memory_format(at::MemoryFormat::ChannelsLast);
  Tensor out = torch::empty({1, c_pad, m.nnum[d], 1}, opts);
  OCNN_CALL(ocnn_feature_to_node_major(reinterpret_cast<const float*>(o.base + off), out.data_ptr(),
                                       ch, c_pad, m.nnum[d],
                                       bf16 ? OCNN_BF16 : (half ? OCNN_F16 : OCNN_F32), current_stream()));
  return out;
}


// ---- network executor ---------------------------------------------------------------------------
// A recorded sequence of hot-path operators over numbered activation slots, replayed on one octree
// per call.  It exists because at these problem sizes a Python-level operator call costs more host
// time than its kernel runs for on a B200: the executor issues the same C-ABI calls back to back
// from C++, with every activation carved out of one arena that is reused across calls.
// Activations are bf16 node-major ([H, C]); slot s at depth d holds nnum[d] rows.
struct ExecOp {
  enum Kind { kFeature, kConvTc, kConv, kPool, kHead, kConvPool } kind;
  // a second 1x1x1 layer chained onto this (1x1x1) one: see add_chain
  int out2 = -1, cout2 = 0, relu2 = 0;
  Tensor weights2, packed2, scale2, bias2;
  int64_t pointwise_above2 = -1, chain_above = -1;
  std::string name2;
  std::string name;
  int depth = 0, cin = 0, cout = 0, stride = 1, relu = 0;
  int in = -1, out = -1, res = -1;
  int in2 = -1, cin2 = 0;         // second input of a two-input 1x1x1 layer (cin = the first one's)
  int tmp = -1;                   // kConvPool: slot of the un-pooled output when the two run apart
  int64_t pointwise_above = -1;   // >= 0: prefer the streaming pointwise kernel from this many nodes
  std::vector<int> ks;
  Tensor weights, packed, scale, bias;     // kept alive here
};

class NetExecutor {
 public:
  NetExecutor() { status_ = Tensor(); }

  int add_feature(int depth, int c_pad, int out) {
    ExecOp op; op.kind = ExecOp::kFeature; op.name = "feature"; op.depth = depth; op.cout = c_pad;
    op.out = out;
    return push(op);
  }
  int add_conv(string name, int depth, int cin, int cout, vector<int> ks, int stride, Tensor weights,
               c10::optional<Tensor> packed, c10::optional<Tensor> scale, c10::optional<Tensor> bias,
               bool relu, int in, int out, int res, int64_t pointwise_above) {
    ExecOp op;
    op.pointwise_above = pointwise_above;
    op.kind = (packed.has_value() && packed->defined()) ? ExecOp::kConvTc : ExecOp::kConv;
    op.name = name; op.depth = depth; op.cin = cin; op.cout = cout; op.ks = kernel3(ks);
    op.stride = stride; op.relu = relu ? 1 : 0; op.in = in; op.out = out; op.res = res;
    TORCH_CHECK(stride == 1, "the executor records stride-1 convolutions only");
    TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32, "weights: float32 CUDA");
    op.weights = weights.contiguous();
    if (op.kind == ExecOp::kConvTc) op.packed = *packed;
    if (scale.has_value() && scale->defined()) op.scale = scale->contiguous();
    if (bias.has_value() && bias->defined()) op.bias = bias->contiguous();
    return push(op);
  }
  // conv1x1b(in) + conv1x1c(in2) of a residual block as one layer over [in | in2]
  int add_conv_pair(string name, int depth, int cin_a, int cin_b, int cout, Tensor packed,
                    c10::optional<Tensor> scale, c10::optional<Tensor> bias, bool relu, int in_a,
                    int in_b, int out) {
    ExecOp op;
    op.kind = ExecOp::kConvTc;
    op.name = name; op.depth = depth; op.cin = cin_a; op.cin2 = cin_b; op.cout = cout;
    op.ks = {1, 1, 1}; op.relu = relu ? 1 : 0; op.in = in_a; op.in2 = in_b; op.out = out;
    TORCH_CHECK(packed.defined() && packed.is_cuda(), "add_conv_pair: packed weights required");
    op.packed = packed;
    if (scale.has_value() && scale->defined()) op.scale = scale->contiguous();
    if (bias.has_value() && bias->defined()) op.bias = bias->contiguous();
    return push(op);
  }
  int add_pool(int depth, int channels, int in, int out) {
    ExecOp op; op.kind = ExecOp::kPool; op.name = "pool" + std::to_string(depth); op.depth = depth;
    op.cin = op.cout = channels; op.in = in; op.out = out;
    return push(op);
  }
  // Chains a second 1x1x1 layer (`name2`: cout -> cout2, no residual) onto the 1x1x1 layer recorded
  // last: from `fused_above` nodes on, and for the channel triples the streaming kernel is built
  // for, the two run as one pass; otherwise one after the other, exactly as recorded separately.
  void add_chain(string name2, int cout2, Tensor weights2, c10::optional<Tensor> packed2,
                 c10::optional<Tensor> scale2, c10::optional<Tensor> bias2, bool relu2, int out2,
                 int64_t fused_above, int64_t pointwise_above2) {
    TORCH_CHECK(!ops_.empty(), "add_chain: nothing recorded");
    ExecOp& op = ops_.back();
    TORCH_CHECK((op.kind == ExecOp::kConvTc || op.kind == ExecOp::kConv) && op.in2 < 0 &&
                    op.ks[0] * op.ks[1] * op.ks[2] == 1, "add_chain: the last op must be a plain 1x1x1 layer");
    TORCH_CHECK(out2 != op.out && out2 != op.in && out2 != op.res, "add_chain: out2 must be a slot of its own");
    TORCH_CHECK(weights2.is_cuda() && weights2.scalar_type() == torch::kFloat32, "weights2: float32 CUDA");
    op.name2 = name2; op.cout2 = cout2; op.relu2 = relu2 ? 1 : 0; op.out2 = out2;
    op.weights2 = weights2.contiguous();
    if (packed2.has_value() && packed2->defined()) op.packed2 = *packed2;
    if (scale2.has_value() && scale2->defined()) op.scale2 = scale2->contiguous();
    if (bias2.has_value() && bias2->defined()) op.bias2 = bias2->contiguous();
    op.chain_above = fused_above;
    op.pointwise_above2 = pointwise_above2;
  }
  // A 1x1x1 layer followed by OctreeMaxPool.  From `fused_above` nodes on (and for the channel
  // counts the streaming kernel takes) the two run as one pass that never writes the un-pooled
  // tensor; otherwise the layer writes slot `tmp` and the pool reads it.  `out` holds level
  // depth - 1 and must differ from `in`, `res` and `tmp`.
  int add_conv_pool(string name, int depth, int cin, int cout, Tensor weights,
                    c10::optional<Tensor> packed, c10::optional<Tensor> scale,
                    c10::optional<Tensor> bias, bool relu, int in, int tmp, int res, int out,
                    int64_t fused_above) {
    ExecOp op;
    op.kind = ExecOp::kConvPool;
    op.name = name; op.depth = depth; op.cin = cin; op.cout = cout; op.ks = {1, 1, 1};
    op.relu = relu ? 1 : 0; op.in = in; op.tmp = tmp; op.res = res; op.out = out;
    op.pointwise_above = fused_above;
    TORCH_CHECK(out != in && out != tmp && out != res && tmp != in && tmp != res,
                "add_conv_pool: the slots must be distinct");
    TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32, "weights: float32 CUDA");
    op.weights = weights.contiguous();
    if (packed.has_value() && packed->defined()) op.packed = *packed;
    if (scale.has_value() && scale->defined()) op.scale = scale->contiguous();
    if (bias.has_value() && bias->defined()) op.bias = bias->contiguous();
    return push(op);
  }
  // global average pool over the full level `depth` + Linear: the output is fp32 [batch, nout]
  int add_head(int depth, int channels, int nout, Tensor weights, c10::optional<Tensor> bias, int in,
               int out) {
    ExecOp op; op.kind = ExecOp::kHead; op.name = "head"; op.depth = depth; op.cin = channels;
    op.cout = nout; op.in = in; op.out = out;
    TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == torch::kFloat32 &&
                    weights.numel() == (int64_t)channels * nout, "add_head: weights float32 [nout, channels]");
    op.weights = weights.contiguous();
    if (bias.has_value() && bias->defined()) op.bias = bias->contiguous();
    return push(op);
  }
  void set_trace(int op_index) { trace_ = op_index; }   // -2 none, -1 every op, >= 0 one op

  // Runs the recorded ops; returns the last op's output as a [1,C,H,1] channels_last tensor
  // (a view into the arena: valid until the next forward).
  Tensor forward(Tensor octree) {
    OctreeRef o = get_octree(octree);
    TORCH_CHECK(o.cuda, "NetExecutor: the octree must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(octree.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
    if (!status_.defined())
      status_ = torch::zeros({1}, octree.options().dtype(torch::kInt32));
    // slot capacity = the largest tensor any op writes into it (slots are reused along the net)
    int nslots = 0;
    for (auto& op : ops_) nslots = std::max(nslots, std::max(std::max(op.out, op.tmp), op.out2) + 1);
    vector<int64_t> rows(nslots, 0), chans(nslots, 0), offs(nslots, 0), cap(nslots, 0);
    for (auto& op : ops_) {
      const int d = (op.kind == ExecOp::kPool || op.kind == ExecOp::kConvPool) ? op.depth - 1 : op.depth;
      if (op.kind == ExecOp::kConvPool)
        cap[op.tmp] = std::max<int64_t>(cap[op.tmp], (int64_t)o.meta.nnum[op.depth] * op.cout * 2);
      if (op.out2 >= 0)
        cap[op.out2] = std::max<int64_t>(cap[op.out2], (int64_t)o.meta.nnum[op.depth] * op.cout2 * 2);
      TORCH_CHECK(d >= 1 && d <= o.meta.depth, "NetExecutor: op ", op.name, " outside the octree depth");
      cap[op.out] = std::max<int64_t>(cap[op.out], (int64_t)o.meta.nnum[d] * op.cout * (op.kind == ExecOp::kHead ? 4 : 2));
    }
    int64_t total = 0, pool_tmp = 0;
    for (int s = 0; s < nslots; ++s) { offs[s] = total; total += (cap[s] + 255) / 256 * 256; }
    for (auto& op : ops_)
      if (op.kind == ExecOp::kPool)
        pool_tmp = std::max<int64_t>(pool_tmp, (int64_t)o.meta.nnum[op.depth] / 8 * op.cin * 6);
      else if (op.kind == ExecOp::kConvPool)
        pool_tmp = std::max<int64_t>(pool_tmp, (int64_t)o.meta.nnum[op.depth] / 8 * 4);
    const int64_t tmp_off = total;
    total += (pool_tmp + 255) / 256 * 256;
    if (!arena_.defined() || arena_.numel() < total || arena_.device() != octree.device())
      arena_ = torch::empty({total + total / 4}, octree.options());
    uint8_t* base = arena_.data_ptr<uint8_t>();
    auto slot = [&](int s) { return s < 0 ? nullptr : base + offs[s]; };

    // a classification head's logits outlive the arena's next use: they get a tensor of their own
    Tensor head_out;
    if (ops_.back().kind == ExecOp::kHead)
      head_out = torch::empty({(int64_t)o.meta.batch_size, (int64_t)ops_.back().cout},
                              octree.options().dtype(torch::kFloat32));
    int index = 0;     // (events of earlier forwards stay queued until trace_ms() collects them)
    for (auto& op : ops_) {
      const bool traced = trace_ == -1 || trace_ == index;
      cudaEvent_t e0 = nullptr, e1 = nullptr;
      if (traced) {
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        cudaEventRecord(e0, st);
      }
      const ocnn_octree_meta& m = o.meta;
      switch (op.kind) {
        case ExecOp::kFeature: {
          const int ch = m.channels[OCNN_PROP_FEATURE];
          const int64_t off = ocnn_prop_offset(&m, OCNN_PROP_FEATURE, op.depth);
          TORCH_CHECK(off >= 0 && ch > 0 && op.cout >= ch, "NetExecutor: octree features missing");
          OCNN_CALL(ocnn_feature_to_node_major(reinterpret_cast<const float*>(o.base + off),
                                               slot(op.out), ch, op.cout, m.nnum[op.depth],
                                               OCNN_BF16, st));
          break;
        }
        case ExecOp::kConvTc:
        case ExecOp::kConv: {
          const int h = m.nnum[op.depth];
          TORCH_CHECK(op.in >= 0 && op.in != op.out && op.res != op.out && rows[op.in] == h &&
                          chans[op.in] == op.cin, "NetExecutor: ", op.name, " input slot does not match");
          TORCH_CHECK(op.res < 0 || (rows[op.res] == h && chans[op.res] == op.cout), "NetExecutor: ",
                      op.name, " residual slot does not match");
          ocnn_conv_epilogue ep;
          ep.scale_dev = op.scale.defined() ? op.scale.data_ptr<float>() : nullptr;
          ep.bias_dev = op.bias.defined() ? op.bias.data_ptr<float>() : nullptr;
          ep.residual_dev = slot(op.res);
          ep.relu = op.relu;
          const bool identity = op.ks[0] * op.ks[1] * op.ks[2] == 1;
          const int32_t* neigh = identity ? nullptr : level_ptr(o, OCNN_PROP_NEIGH, op.depth, "conv");
          const bool stream_pw = identity && op.pointwise_above >= 0 && h >= op.pointwise_above;
          bool chained = false;
          if (op.out2 >= 0) {
            ocnn_conv_epilogue ep2;
            ep2.scale_dev = op.scale2.defined() ? op.scale2.data_ptr<float>() : nullptr;
            ep2.bias_dev = op.bias2.defined() ? op.bias2.data_ptr<float>() : nullptr;
            ep2.residual_dev = nullptr;
            ep2.relu = op.relu2;
            if (op.chain_above >= 0 && h >= op.chain_above) {
              const int rc = ocnn_octree_conv1x1_chain(slot(op.in), op.weights.data_ptr<float>(), slot(op.out),
                                                       &ep, op.weights2.data_ptr<float>(), slot(op.out2), &ep2,
                                                       h, op.cin, op.cout, op.cout2, OCNN_BF16, st);
              if (rc == OCNN_OK) chained = true;
              else TORCH_CHECK(rc == OCNN_ERR_UNSUPPORTED, "ocnn_b200: ", ocnn_last_error());
            }
          }
          if (chained) {
            rows[op.out2] = h;
            chans[op.out2] = op.cout2;
          } else if (op.in2 >= 0) {
            TORCH_CHECK(op.in2 != op.out && rows[op.in2] == h && chans[op.in2] == op.cin2,
                        "NetExecutor: ", op.name, " second input slot does not match");
            OCNN_CALL(ocnn_octree_conv_tc_pair(slot(op.in), op.cin, slot(op.in2), op.cin2,
                                               op.packed.data_ptr(), slot(op.out), h, op.cout,
                                               OCNN_BF16, &ep, status_.data_ptr<int32_t>(), st));
          } else if (op.kind == ExecOp::kConvTc && !stream_pw) {
            OCNN_CALL(ocnn_octree_conv_tc(slot(op.in), op.packed.data_ptr(), slot(op.out), neigh, h, h,
                                          op.cin, op.cout, op.ks.data(), 1, &ep,
                                          status_.data_ptr<int32_t>(), st));
          } else {
            OCNN_CALL(ocnn_octree_conv(slot(op.in), op.weights.data_ptr<float>(), slot(op.out), neigh,
                                       h, h, op.cin, op.cout, op.ks.data(), 1, OCNN_BF16,
                                       OCNN_NODE_MAJOR, &ep, st));
          }
          if (op.out2 >= 0 && !chained) {
            ocnn_conv_epilogue ep2;
            ep2.scale_dev = op.scale2.defined() ? op.scale2.data_ptr<float>() : nullptr;
            ep2.bias_dev = op.bias2.defined() ? op.bias2.data_ptr<float>() : nullptr;
            ep2.residual_dev = nullptr;
            ep2.relu = op.relu2;
            const bool stream2 = op.pointwise_above2 >= 0 && h >= op.pointwise_above2;
            if (op.packed2.defined() && !stream2) {
              OCNN_CALL(ocnn_octree_conv_tc(slot(op.out), op.packed2.data_ptr(), slot(op.out2), nullptr, h, h,
                                            op.cout, op.cout2, op.ks.data(), 1, &ep2,
                                            status_.data_ptr<int32_t>(), st));
            } else {
              OCNN_CALL(ocnn_octree_conv(slot(op.out), op.weights2.data_ptr<float>(), slot(op.out2), nullptr,
                                         h, h, op.cout, op.cout2, op.ks.data(), 1, OCNN_BF16,
                                         OCNN_NODE_MAJOR, &ep2, st));
            }
            rows[op.out2] = h;
            chans[op.out2] = op.cout2;
          }
          break;
        }
        case ExecOp::kConvPool: {
          const int h = m.nnum[op.depth], top_h = m.nnum[op.depth - 1];
          TORCH_CHECK(op.in >= 0 && rows[op.in] == h && chans[op.in] == op.cin, "NetExecutor: ", op.name,
                      " input slot does not match");
          TORCH_CHECK(op.res < 0 || (rows[op.res] == h && chans[op.res] == op.cout), "NetExecutor: ",
                      op.name, " residual slot does not match");
          ocnn_conv_epilogue ep;
          ep.scale_dev = op.scale.defined() ? op.scale.data_ptr<float>() : nullptr;
          ep.bias_dev = op.bias.defined() ? op.bias.data_ptr<float>() : nullptr;
          ep.residual_dev = slot(op.res);
          ep.relu = op.relu;
          const int32_t* child_parent = level_ptr(o, OCNN_PROP_CHILD, op.depth - 1, "pool");
          int rc = OCNN_ERR_UNSUPPORTED;
          if (op.pointwise_above >= 0 && h >= op.pointwise_above)
            rc = ocnn_octree_conv1x1_max_pool_pad(slot(op.in), op.weights.data_ptr<float>(), slot(op.out),
                                                  child_parent, h, top_h, op.cin, op.cout, OCNN_BF16, &ep,
                                                  reinterpret_cast<int32_t*>(base + tmp_off), st);
          if (rc == OCNN_ERR_UNSUPPORTED) {
            if (op.packed.defined()) {
              OCNN_CALL(ocnn_octree_conv_tc(slot(op.in), op.packed.data_ptr(), slot(op.tmp), nullptr, h, h,
                                            op.cin, op.cout, op.ks.data(), 1, &ep,
                                            status_.data_ptr<int32_t>(), st));
            } else {
              OCNN_CALL(ocnn_octree_conv(slot(op.in), op.weights.data_ptr<float>(), slot(op.tmp), nullptr, h,
                                         h, op.cin, op.cout, op.ks.data(), 1, OCNN_BF16, OCNN_NODE_MAJOR,
                                         &ep, st));
            }
            OCNN_CALL(ocnn_octree_max_pool_pad(slot(op.tmp), slot(op.out), child_parent, op.cout, h, top_h,
                                               OCNN_BF16, OCNN_NODE_MAJOR, st));
          } else {
            OCNN_CALL(rc);
          }
          break;
        }
        case ExecOp::kHead: {
          const int h = m.nnum[op.depth], batch = m.batch_size;
          TORCH_CHECK(rows[op.in] == h && chans[op.in] == op.cin && batch > 0 &&
                          (int64_t)h == ((int64_t)batch << (3 * op.depth)),
                      "NetExecutor: the head needs a full level (depth ", op.depth, ": ", h,
                      " nodes for a batch of ", batch, ")");
          OCNN_CALL(ocnn_global_pool_fc(slot(op.in), op.weights.data_ptr<float>(),
                                        op.bias.defined() ? op.bias.data_ptr<float>() : nullptr,
                                        (&op == &ops_.back() && head_out.defined())
                                            ? head_out.data_ptr<float>()
                                            : reinterpret_cast<float*>(slot(op.out)),
                                        batch, h / batch, op.cin, op.cout, OCNN_BF16, st));
          break;
        }
        case ExecOp::kPool: {
          // OctreeMaxPool: max over sibling groups, then pad to every node of depth - 1
          const int h = m.nnum[op.depth], top = h / 8;
          TORCH_CHECK(rows[op.in] == h && chans[op.in] == op.cin, "NetExecutor: pool input mismatch");
          if (op.cin % 8 == 0) {
            OCNN_CALL(ocnn_octree_max_pool_pad(slot(op.in), slot(op.out),
                                               level_ptr(o, OCNN_PROP_CHILD, op.depth - 1, "pool"),
                                               op.cin, h, m.nnum[op.depth - 1], OCNN_BF16,
                                               OCNN_NODE_MAJOR, st));
          } else {
            uint8_t* tmp = base + tmp_off;
            int32_t* mask = reinterpret_cast<int32_t*>(tmp + (int64_t)top * op.cin * 2);
            OCNN_CALL(ocnn_octree_max_pool(slot(op.in), tmp, mask, op.cin, top, OCNN_BF16,
                                           OCNN_NODE_MAJOR, st));
            OCNN_CALL(ocnn_octree_pad(tmp, slot(op.out), level_ptr(o, OCNN_PROP_CHILD, op.depth - 1, "pool"),
                                      op.cin, top, m.nnum[op.depth - 1], 0.f, OCNN_BF16,
                                      OCNN_NODE_MAJOR, st));
          }
          break;
        }
      }
      rows[op.out] = m.nnum[(op.kind == ExecOp::kPool || op.kind == ExecOp::kConvPool) ? op.depth - 1 : op.depth];
      chans[op.out] = op.cout;
      if (traced) {
        cudaEventRecord(e1, st);
        events_.push_back({index, e0, e1});
      }
      ++index;
    }
    const ExecOp& last = ops_.back();
    if (last.kind == ExecOp::kHead) return head_out;
    auto opts = octree.options().dtype(torch::kBFloat16);
    return torch::from_blob(slot(last.out), {1, chans[last.out], rows[last.out], 1},
                            {chans[last.out] * rows[last.out], 1, chans[last.out], chans[last.out]},
                            opts);
  }

  // (op index, milliseconds) of the traced ops of the last forward; synchronises on their events.
  vector<std::pair<int, float>> trace_ms() {
    vector<std::pair<int, float>> out;
    for (auto& e : events_) {
      cudaEventSynchronize(e.e1);
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e.e0, e.e1);
      out.push_back({e.index, ms});
      cudaEventDestroy(e.e0);
      cudaEventDestroy(e.e1);
    }
    events_.clear();
    return out;
  }
  vector<string> op_names() const {
    vector<string> n;
    for (auto& op : ops_) n.push_back(op.name);
    return n;
  }
  int status() { return status_.defined() ? status_.item<int>() : 0; }

 private:
  int push(const ExecOp& op) { ops_.push_back(op); return (int)ops_.size() - 1; }
  struct Ev { int index; cudaEvent_t e0, e1; };
  vector<ExecOp> ops_;
  vector<Ev> events_;
  Tensor arena_, status_;
  int trace_ = -2;
};

void set_key_bits(int bits) {
  TORCH_CHECK(bits == 32 || bits == 64, "key bits must be 32 or 64");
  g_key_bits = bits;
}
int get_key_bits() { return g_key_bits; }

// ---- octree editing for the generative networks (pytorch/cpp/octree_grow.cpp) --------------------
// octree_new builds on the host and uploads, as the reference does; its keys follow the
// binding's key width (ocnn.nn.set_key_bits, 64 like the reference's build).
Tensor octree_new(int batch_size, int channel, bool node_dis, int adaptive_layer) {
  const size_t bytes = ocnn_octree_new_bytes(batch_size, channel, g_key_bits);
  TORCH_CHECK(bytes > 0, "octree_new: batch_size must be at least 1 and channel non-negative");
  Tensor host = torch::zeros({(int64_t)bytes}, torch::kUInt8);
  OCNN_CALL(ocnn_octree_new(batch_size, channel, node_dis ? 1 : 0, adaptive_layer, g_key_bits,
                            host.data_ptr<uint8_t>(), bytes));
  return host.cuda();
}

Tensor octree_grow(Tensor octree_in, int target_depth, bool full_octree) {
  OctreeRef o = get_octree(octree_in);
  TORCH_CHECK(o.cuda, "octree_grow: the octree must be a CUDA tensor");
  c10::cuda::CUDAGuard guard(octree_in.device());
  uint8_t header_out[OCNN_HEADER_BYTES];
  OCNN_CALL(ocnn_octree_grow_header(o.raw, target_depth, full_octree ? 1 : 0, header_out));
  ocnn_octree_meta mo;
  OCNN_CALL(ocnn_parse_header(header_out, OCNN_HEADER_BYTES, &mo));
  Tensor out = torch::empty({(int64_t)mo.ptr_dis[OCNN_PROP_COUNT]}, octree_in.options());
  OCNN_CALL(ocnn_octree_grow(octree_in.data_ptr<uint8_t>(), o.raw, out.data_ptr<uint8_t>(), header_out,
                             target_depth, full_octree ? 1 : 0, current_stream()));
  remember_header(out, mo, header_out);
  return out;
}

Tensor octree_update(Tensor octree_in, Tensor label_in, int depth, int split) {
  OctreeRef o = get_octree(octree_in);
  TORCH_CHECK(o.cuda, "octree_update: the octree must be a CUDA tensor");
  c10::cuda::CUDAGuard guard(octree_in.device());
  TORCH_CHECK(depth >= 0 && depth <= o.meta.depth, "octree_update: depth ", depth, " outside the octree");
  TORCH_CHECK(label_in.is_cuda() && label_in.scalar_type() == torch::kInt32,
              "octree_update: the label must be an int32 CUDA tensor");
  TORCH_CHECK(label_in.numel() == o.meta.nnum[depth], "octree_update: ", label_in.numel(),
              " labels for ", o.meta.nnum[depth], " nodes");
  Tensor label = label_in.contiguous();
  Tensor out = octree_in.clone();
  Tensor ws = torch::empty({(int64_t)ocnn_octree_update_workspace_bytes()}, octree_in.options());
  uint8_t header_out[OCNN_HEADER_BYTES];
  OCNN_CALL(ocnn_octree_update(out.data_ptr<uint8_t>(), o.raw, label.data_ptr<int32_t>(), depth, split,
                               ws.data_ptr<uint8_t>(), header_out, current_stream()));
  ocnn_octree_meta mo;
  OCNN_CALL(ocnn_parse_header(header_out, OCNN_HEADER_BYTES, &mo));
  remember_header(out, mo, header_out);
  return out;
}

template <typename... Args>
Tensor not_built(const char* name) {
  TORCH_CHECK(false, "ocnn.nn.", name, " is outside the inference hot path and is not implemented "
              "in ocnn_b200");
  return Tensor();
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.doc() = "ocnn.nn on libocnn_b200 (CUDA sm_100a)";
  // reference names and signatures (pytorch/cpp/pybind.cpp:3-49)
  m.def("octree_batch", &octree_batch, "merge a batch of octrees");
  m.def("octree_property", &octree_property, "get the octree property", py::arg("octree"),
        py::arg("property"), py::arg("depth") = 0);
  m.def("points2octree", &points2octree, "convert points to octree");
  m.def("octree2col", &octree2col, "octree2col");
  m.def("col2octree", &col2octree, "col2octree");
  m.def("octree_conv", &octree_conv, "octree based convolution");
  m.def("octree_deconv", &octree_deconv, "octree based deconvolution");
  m.def("octree_conv_grad", &octree_conv_grad, "octree based convolution");
  m.def("octree_deconv_grad", &octree_deconv_grad, "octree based deconvolution");
  m.def("octree_max_unpool", &octree_max_unpool, "octree max unpooling");
  m.def("octree_mask_pool", &octree_mask_pool, "octree mask pooling");
  m.def("octree_pad", &octree_pad, "octree pad", py::arg("data_in"), py::arg("octree"),
        py::arg("depth"), py::arg("val") = 0.0f);
  m.def("octree_depad", &octree_depad, "octree depad");
  m.def("octree_tile", &octree_tile, "nearest upsampling: depad + repeat each row for its 8 children");
  m.def("octree_max_pool", &octree_max_pool, "octree max pooling");
  m.def("octree_max_pool_pad", &octree_max_pool_pad, "octree max pooling + pad to depth - 1 (bf16 node-major)");
  m.def("points_new", &points_new, "create a point cloud");
  m.def("transform_points", &transform_points, "transform the point cloud");
  m.def("clip_points", &clip_points, "clip the points with unit boundingbox");
  m.def("normalize_points", &normalize_points, "normalize the point cloud");
  m.def("bounding_sphere", &bounding_sphere, "calc the bounding sphere");
  m.def("points_property", &points_property, "get the points' property");
  m.def("points_batch_property", &points_batch_property, "get batch of points' property");
  m.def("points_set_property", &points_set_property, "set the points' property");
  // additions of this implementation
  m.def("points2octree_batch", &points2octree_batch,
        "build the merged batch octree of a list of point clouds in one pass");
  m.def("points_pack", &points_pack, py::arg("points"), py::arg("pin") = false);
  // (the GIL is released: the build blocks once on its stream, and a second Python thread may be
  // enqueueing a forward pass meanwhile)
  m.def("points2octree_packed", &points2octree_packed, py::call_guard<py::gil_scoped_release>());
  m.def("octree_conv_fused", &octree_conv_fused, py::arg("data_in"), py::arg("weights"),
        py::arg("octree"), py::arg("depth"), py::arg("num_output"), py::arg("kernel_size"),
        py::arg("stride"), py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false);
  m.def("conv_pack_weights", &conv_pack_weights, py::arg("weights"), py::arg("cin"), py::arg("cout"),
        py::arg("kernel_size"), py::arg("stride") = 1);
  m.def("conv_tc_wait_selftest", &conv_tc_wait_selftest);
  m.def("octree_conv_tc", &octree_conv_tc, py::arg("data_in"), py::arg("packed"), py::arg("octree"),
        py::arg("depth"), py::arg("num_output"), py::arg("kernel_size"), py::arg("stride"),
        py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false, py::arg("status"));
  m.def("conv_pack_weights_nempty", &conv_pack_weights_nempty, py::arg("weights"), py::arg("cin"),
        py::arg("cout"), py::arg("kernel_size"));
  m.def("octree_conv_tc_nempty", &octree_conv_tc_nempty, py::arg("data_in"), py::arg("packed"),
        py::arg("octree"), py::arg("depth"), py::arg("num_output"), py::arg("kernel_size"),
        py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false, py::arg("status"));
  m.def("octree_conv_general", &octree_conv_general, py::arg("data_in"), py::arg("weights"),
        py::arg("octree"), py::arg("depth"), py::arg("num_output"), py::arg("kernel_size"),
        py::arg("stride") = 1, py::arg("nempty") = false, py::arg("transposed") = false,
        py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false);
  m.def("conv_pack_weights_general", &conv_pack_weights_general, py::arg("weights"), py::arg("cin"),
        py::arg("cout"), py::arg("kernel_size"), py::arg("stride") = 1,
        py::arg("transposed") = false, py::arg("nempty") = false, py::arg("half") = false);
  m.def("octree_conv_tc_general", &octree_conv_tc_general, py::arg("data_in"), py::arg("packed"),
        py::arg("octree"), py::arg("depth"), py::arg("num_output"), py::arg("kernel_size"),
        py::arg("stride") = 1, py::arg("nempty") = false, py::arg("transposed") = false,
        py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false, py::arg("status"));
  m.def("pointwise_conv", &pointwise_conv, py::arg("data_in"), py::arg("weights"),
        py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false);
  m.def("pointwise_conv_tc", &pointwise_conv_tc, py::arg("data_in"), py::arg("packed"),
        py::arg("num_output"), py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false, py::arg("status"));
  m.def("pointwise_conv_tc_pair", &pointwise_conv_tc_pair, py::arg("data_a"), py::arg("data_b"),
        py::arg("packed"), py::arg("num_output"), py::arg("scale") = py::none(),
        py::arg("bias") = py::none(), py::arg("residual") = py::none(), py::arg("relu") = false,
        py::arg("status"));
  m.def("conv1x1_max_pool_pad", &conv1x1_max_pool_pad, py::arg("data_in"), py::arg("weights"),
        py::arg("octree"), py::arg("depth"), py::arg("scale") = py::none(), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("relu") = false);
  m.def("conv1x1_chain", &conv1x1_chain, py::arg("data_in"), py::arg("w1"), py::arg("scale1") = py::none(),
        py::arg("bias1") = py::none(), py::arg("residual1") = py::none(), py::arg("relu1") = false,
        py::arg("w2"), py::arg("scale2") = py::none(), py::arg("bias2") = py::none(),
        py::arg("relu2") = false);
  m.def("global_pool_fc", &global_pool_fc, py::arg("data_in"), py::arg("weights"),
        py::arg("bias") = py::none(), py::arg("batch"));
  m.def("octree_encode_key", &octree_encode_key, "encode xyz-id to octree key");
  m.def("octree_decode_key", &octree_decode_key, "decode octree key to xyz-id");
  m.def("octree_xyz2key", &octree_xyz2key, "convert key from xyz order");
  m.def("octree_key2xyz", &octree_key2xyz, "convert key to xyz order");
  m.def("octree_search_key", &octree_search_key, "search key from octree", py::arg("key"),
        py::arg("octree"), py::arg("depth"), py::arg("key_is_xyz") = true, py::arg("nempty") = false);
  m.def("octree_interp", &octree_interp, py::arg("data_in"), py::arg("octree"), py::arg("depth"),
        py::arg("pts"), py::arg("method") = "linear", py::arg("nempty") = false);
  m.def("octree_align", &octree_align, "align octree data", py::arg("src_data"),
        py::arg("src_octree"), py::arg("des_octree"), py::arg("depth"));
  m.def("octree_align_grad", &octree_align_grad, "backward of align-octree-data");
  m.def("octree_info", &octree_info);
  // (pytorch/cpp/pybind.cpp:35-41)
  m.def("octree_grow", &octree_grow, "octree growing", py::arg("octree"), py::arg("target_depth"),
        py::arg("full_octree") = false);
  m.def("octree_update", &octree_update, "update octree via splitting labels", py::arg("octree"),
        py::arg("label"), py::arg("depth"), py::arg("split") = 1);
  m.def("octree_new", &octree_new, "create a new octree", py::arg("batch_size") = 1,
        py::arg("channel") = 4, py::arg("node_dis") = true, py::arg("adaptive_layer") = 0);
  m.def("feature_node_major", &feature_node_major, py::arg("octree"), py::arg("c_pad"),
        py::arg("bf16") = true, py::arg("half") = false);
  m.def("set_key_bits", &set_key_bits);
  m.def("get_key_bits", &get_key_bits);
  py::class_<NetExecutor>(m, "NetExecutor")
      .def(py::init<>())
      .def("add_feature", &NetExecutor::add_feature)
      .def("add_conv", &NetExecutor::add_conv, py::arg("name"), py::arg("depth"), py::arg("cin"),
           py::arg("cout"), py::arg("kernel_size"), py::arg("stride"), py::arg("weights"),
           py::arg("packed") = py::none(), py::arg("scale") = py::none(),
           py::arg("bias") = py::none(), py::arg("relu") = false, py::arg("input") = 0,
           py::arg("output") = 0, py::arg("residual") = -1, py::arg("pointwise_above") = -1)
      .def("add_conv_pair", &NetExecutor::add_conv_pair)
      .def("add_pool", &NetExecutor::add_pool)
      .def("add_head", &NetExecutor::add_head)
      .def("add_conv_pool", &NetExecutor::add_conv_pool)
      .def("add_chain", &NetExecutor::add_chain)
      .def("set_trace", &NetExecutor::set_trace)
      .def("forward", &NetExecutor::forward, py::call_guard<py::gil_scoped_release>())
      .def("trace_ms", &NetExecutor::trace_ms)
      .def("op_names", &NetExecutor::op_names)
      .def("status", &NetExecutor::status);
  m.def("last_error", []() { return string(ocnn_last_error()); });
  m.def("launch_count", []() { return (int64_t)ocnn_launch_count(); });
}
