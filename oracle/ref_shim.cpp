// TEST INFRASTRUCTURE ONLY — not part of the shipped library.
//
// Thin extern "C" shim around the UNMODIFIED reference CPU sources (octree/octree/*.cpp of
// microsoft/O-CNN).  It is compiled by oracle/Makefile against the reference tree where it
// lies on the build machine, once with 32-bit keys and once with -DKEY64, into
// oracle/_ref/libocnn_ref{32,64}.so.  No reference source is copied: this file only calls
// the reference's public C++ entry points so that ctypes can drive them.
//
// Wrapped entry points (reference file:line):
//   Points::set_points            octree/octree/points.cpp:96-150
//   OctreeInfo::initialize        octree/octree/octree_info.cpp:13-73
//   Octree::build                 octree/octree/octree.cpp:74-121
//   merge_octrees                 octree/octree/merge_octrees.cpp:7-15
//   calc_neigh_cpu (full, split)  octree/octree/octree_nn.cpp:382-424, 357-380
//   octree2col_cpu / octree2colP_cpu   octree/octree/octree_nn.cpp:188-214, 244-271
//   octree_max_pool_cpu           octree/octree/octree_nn.cpp:301-322
//   pad_forward_cpu / pad_backward_cpu octree/octree/octree_nn.cpp:163-185
//   OctreeBaseConv<float>::forward_cpu_gemm  octree/octree/octree_conv.cpp:158-180
//   OctreeBaseConv<float>::backward_cpu_gemm (the deconvolution's forward)  octree_conv.cpp:182-206
//   col2octree_cpu / col2octreeP_cpu   octree/octree/octree_nn.cpp:216-241, 273-298
//   xyz2key_cpu / key2xyz_cpu / search_key_cpu   octree/octree/octree_nn.cpp:540-620
//   PointsParser::displace / rotate / translate / scale / orient_normal / clip
//                                 octree/octree/points_parser.cpp:42-259
//   bounding_box                  octree/octree/math_functions.cpp:113-128
//   NeighHelper tables            octree/octree/octree_nn.cpp:6-108
//   octree::get_one_octree        octree/octree/octree_samples.cpp:2168-2178

#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "merge_octrees.h"
#include "octree.h"
#include "octree_conv.h"
#include "octree_nn.h"
#include "octree_samples.h"
#include "math_functions.h"
#include "points.h"

// OctreeBaseConv's CPU im2col wrapper names OctreeParser::neighbor_gpu on its non-empty branch
// (octree/octree/octree_conv.cpp:135,151); that accessor lives in octree_parser.cu, which
// needs CUDA and is not compiled here.  On the CPU the neighbour table is the same host array
// either way, so the definition forwards to the CPU accessor.
const int* OctreeParser::neighbor_gpu(const int depth) const { return neighbor_cpu(depth); }

namespace {

typedef void (*gemm_cb_t)(int M, int N, int K, const float* A, const float* B, float* C);
gemm_cb_t g_gemm_cb = nullptr;

// C[M,N] = A[M,K] * B[K,N], row-major; the octree library ships no CPU GEMM of its own
// (octree/octree/gemm_engine.h:8-15 is abstract), so the harness supplies one.
class ShimGemm : public octree::GEMMEngine<float> {
 public:
  void gemm(const bool TransA, const bool TransB, const int M, const int N, const int K,
            const float alpha, const float* A, const float* B, const float beta,
            float* C) override {
    if (!TransA && !TransB && alpha == 1.0f && beta == 0.0f && g_gemm_cb != nullptr) {
      g_gemm_cb(M, N, K, A, B, C);
      return;
    }
    for (int m = 0; m < M; ++m) {
      for (int n = 0; n < N; ++n) {
        float acc = 0.0f;
        for (int k = 0; k < K; ++k) {
          float a = TransA ? A[k * M + m] : A[m * K + k];
          float b = TransB ? B[n * K + k] : B[k * N + n];
          acc += a * b;
        }
        C[m * N + n] = alpha * acc + (beta == 0.0f ? 0.0f : beta * C[m * N + n]);
      }
    }
  }
};

// Convolution / deconvolution forward for every stride / nempty combination, driven the way the
// PyTorch binding drives it (pytorch/cpp/octree_conv.cpp:61-120, 137-154, 191-217): setup, reshape,
// child/ichild for the non-empty variant (pad_backward of 0..n-1 through the child array), then
// forward_cpu_gemm for the convolution and backward_cpu_gemm for the deconvolution.
class ShimConvGeneral : public octree::OctreeBaseConv<float> {
 public:
  explicit ShimConvGeneral(bool deconv) : deconv_(deconv) {}
  bool is_deconvolution_layer() override { return deconv_; }

  long run(float* top, const float* bottom, const float* weights, const char* octree_buf,
           int depth, int cin, int cout, const int* ksize, int stride, int nempty, long top_cap) {
    std::vector<int> ks(ksize, ksize + 3);
    this->octree_.set_cpu(octree_buf);
    this->setup(ks, stride, depth, cin, cout, nempty != 0);
    this->engine_cpu_ = &gemm_;
    this->reshape();
    long top_n = (long)this->top_shape_[1] * this->top_shape_[2];
    if (top == nullptr || top_cap < top_n) return top_n;
    std::vector<float> ws((size_t)num_elements(this->workspace_shape_));
    std::vector<float> rb((size_t)num_elements(this->result_buffer_shape_));
    this->workspace_ = ws.data();
    this->result_buffer_ = rb.empty() ? nullptr : rb.data();
    std::vector<int> ich;
    if (nempty) {
      this->child_ = this->octree_.children_cpu(this->workspace_depth_);
      // the binding's pad_backward of 0..child_h-1 through child (only float/double are
      // instantiated in the library, so the same scatter is written out here for ints)
      ich.assign(this->ichild_h_ > 0 ? this->ichild_h_ : 1, 0);
      for (int i = 0; i < this->child_h_; ++i)
        if (this->child_[i] != -1) ich[this->child_[i]] = i;
      this->ichild_ = ich.data();
    }
    if (deconv_) this->backward_cpu_gemm(top, bottom, weights);
    else this->forward_cpu_gemm(top, bottom, weights);
    return top_n;
  }

 private:
  bool deconv_;
  ShimGemm gemm_;
};

class ShimConv : public octree::OctreeBaseConv<float> {
 public:
  bool is_deconvolution_layer() override { return false; }

  long run(float* top, const float* bottom, const float* weights, const char* octree_buf,
           int depth, int cin, int cout, const int* ksize, int stride, long top_cap) {
    std::vector<int> ks(ksize, ksize + 3);
    this->octree_.set_cpu(octree_buf);
    this->setup(ks, stride, depth, cin, cout, false);
    this->engine_cpu_ = &gemm_;
    this->reshape();
    long top_n = (long)this->top_shape_[1] * this->top_shape_[2];
    if (top == nullptr || top_cap < top_n) return top_n;
    std::vector<float> ws((size_t)num_elements(this->workspace_shape_));
    std::vector<float> rb((size_t)num_elements(this->result_buffer_shape_));
    this->workspace_ = ws.data();
    this->result_buffer_ = rb.empty() ? nullptr : rb.data();
    this->forward_cpu_gemm(top, bottom, weights);
    return top_n;
  }

 private:
  ShimGemm gemm_;
};

long emit(const std::vector<char>& src, char* out, long cap) {
  long sz = (long)src.size();
  if (out != nullptr && cap >= sz) memcpy(out, src.data(), sz);
  return sz;
}

}  // namespace

extern "C" {

int ref_key_bits() { return (int)(8 * sizeof(uintk)); }

void ref_set_gemm(gemm_cb_t cb) { g_gemm_cb = cb; }

long ref_points_new(const float* pts, const float* normals, const float* feats,
                    const float* labels, int n, int cf, char* out, long cap) {
  std::vector<float> p(pts, pts + 3 * (size_t)n), nm, ft, lb;
  if (normals) nm.assign(normals, normals + 3 * (size_t)n);
  if (feats) ft.assign(feats, feats + (size_t)cf * n);
  if (labels) lb.assign(labels, labels + (size_t)n);
  Points points;
  if (!points.set_points(p, nm, ft, lb)) return -1;
  return emit(points.get_buffer(), out, cap);
}

// points2octree exactly as pytorch/cpp/point2octree.cpp:5-34 drives it; a non-null bbox
// (6 floats: min xyz, max xyz) overrides the fixed [-1,1]^3 box, which is how the
// reference's own gtest (octree/test/test_octree.cpp:92-100) builds its golden octree.
long ref_points2octree(const char* points_buf, int depth, int full_depth, int node_dis,
                       int node_feature, int split_label, int adaptive, int adp_depth,
                       float th_normal, float th_distance, int extrapolate, int save_pts,
                       int key2xyz, const float* bbox, char* out, long cap) {
  Points pc;
  pc.set(points_buf);
  std::string msg;
  if (!pc.info().check_format(msg)) return -1;
  OctreeInfo info;
  info.initialize(depth, full_depth, node_dis != 0, node_feature != 0, split_label != 0,
                  adaptive != 0, adp_depth, th_distance, th_normal, key2xyz != 0,
                  extrapolate != 0, save_pts != 0, pc);
  if (bbox != nullptr) info.set_bbox(bbox, bbox + 3);
  Octree oct;
  oct.build(info, pc);
  return emit(oct.buffer(), out, cap);
}

long ref_octree_batch(const char* const* octrees, int n, char* out, long cap) {
  std::vector<const char*> in(octrees, octrees + n);
  std::vector<char> merged;
  merge_octrees(merged, in);
  return emit(merged, out, cap);
}

long ref_octree_sample(const char* name, char* out, long cap) {
  size_t size = 0;
  const unsigned char* data = octree::get_one_octree(name, &size);
  if (data == nullptr) return -1;
  if (out != nullptr && cap >= (long)size) memcpy(out, data, size);
  return (long)size;
}

// Header fields through the reference's own accessors: out[0..7] = batch, depth, full_layer,
// sizeof_octree, content_flags, total_nnum, sizeof(OctreeInfo), key bits; then 16 nnum,
// 16 nnum_cum, 16 nnum_nempty, then per property (6): channel, location, ptr_dis(depth 0).
void ref_octree_info(const char* octree_buf, int* out) {
  OctreeParser parser;
  parser.set_cpu(octree_buf);
  const OctreeInfo& info = parser.info();
  out[0] = info.batch_size();
  out[1] = info.depth();
  out[2] = info.full_layer();
  out[3] = info.sizeof_octree();
  out[4] = info.content_flags();
  out[5] = info.total_nnum();
  out[6] = info.sizeof_octinfo();
  out[7] = ref_key_bits();
  for (int d = 0; d < 16; ++d) {
    out[8 + d] = info.node_num(d);
    out[24 + d] = info.node_num_cum(d);
    out[40 + d] = info.node_num_nempty(d);
  }
  for (int i = 0; i < 6; ++i) {
    OctreeInfo::PropType p = static_cast<OctreeInfo::PropType>(1 << i);
    out[56 + 3 * i + 0] = info.channel(p);
    out[56 + 3 * i + 1] = info.locations(p);
    out[56 + 3 * i + 2] = info.ptr_dis(p, 0);
  }
}

void ref_calc_neigh_full(int* neigh, int depth, int batch_size) {
  calc_neigh_cpu(neigh, depth, batch_size);
}

void ref_calc_neigh_split(int* neigh_child, const int* neigh, const int* child, int node_num) {
  calc_neigh_cpu(neigh_child, neigh, child, node_num);
}

int ref_ni_table(const int* ksize, int* out) {
  std::vector<int> ks(ksize, ksize + 3);
  const std::vector<int>& ni = NeighHelper::get_ni(ks);
  if (out != nullptr) memcpy(out, ni.data(), ni.size() * sizeof(int));
  return (int)ni.size();
}

void ref_neigh_tables(int* parent512, int* dis64) {
  memcpy(parent512, NeighHelper::get_parent_array().data(), 512 * sizeof(int));
  memcpy(dis64, NeighHelper::get_dis_array().data(), 64 * sizeof(int));
}

void ref_octree2col(float* col, const float* data, int channel, int height, int kernel_sdim,
                    int stride, const int* neigh, const int* ni, int height_col, int n) {
  octree2col_cpu<float>(col, data, channel, height, kernel_sdim, stride, neigh, ni,
                        height_col, n);
}

void ref_octree2colP(float* col, const float* data, int channel, int height, int octree_h,
                     int kernel_sdim, int stride, const int* neigh, const int* ni,
                     const int* child, const int* ichild, int height_col, int n) {
  octree2colP_cpu<float>(col, data, channel, height, octree_h, kernel_sdim, stride, neigh, ni,
                         child, ichild, height_col, n);
}

void ref_max_pool(float* top, int top_h, int* mask, const float* btm, int btm_h, int channel) {
  octree_max_pool_cpu<float>(top, top_h, mask, btm, btm_h, channel);
}

void ref_pad_forward(float* Y, int Hy, int C, const float* X, int Hx, const int* label,
                     float dval) {
  pad_forward_cpu<float>(Y, Hy, C, X, Hx, label, dval);
}

void ref_pad_backward(float* X, int Hx, int C, const float* Y, int Hy, const int* label) {
  pad_backward_cpu<float>(X, Hx, C, Y, Hy, label);
}

// OctreeConv forward (dense, nempty = false) through the reference's own
// setup/reshape/forward_cpu_gemm.  Returns the number of output floats (Cout * top_h);
// call with top == NULL to size the output.
long ref_octree_conv(float* top, long top_cap, const float* bottom, const float* weights,
                     const char* octree_buf, int depth, int cin, int cout, const int* ksize,
                     int stride) {
  ShimConv conv;
  return conv.run(top, bottom, weights, octree_buf, depth, cin, cout, ksize, stride, top_cap);
}

// OctreeConv / OctreeDeconv forward with any stride and nempty flag.  cin = channels of `bottom`,
// cout = num_output.  Returns the number of output floats; top == NULL sizes the output.
long ref_octree_conv_general(float* top, long top_cap, const float* bottom, const float* weights,
                             const char* octree_buf, int depth, int cin, int cout,
                             const int* ksize, int stride, int nempty, int deconv) {
  ShimConvGeneral conv(deconv != 0);
  return conv.run(top, bottom, weights, octree_buf, depth, cin, cout, ksize, stride, nempty, top_cap);
}

void ref_col2octree(const float* col, float* data, int channel, int height, int kernel_sdim,
                    int stride, const int* neigh, const int* ni, int height_col, int n) {
  col2octree_cpu<float>(col, data, channel, height, kernel_sdim, stride, neigh, ni, height_col, n);
}

void ref_col2octreeP(const float* col, float* data, int channel, int height, int octree_h,
                     int kernel_sdim, int stride, const int* neigh, const int* ni, const int* child,
                     const int* ichild, int height_col, int n) {
  col2octreeP_cpu<float>(col, data, channel, height, octree_h, kernel_sdim, stride, neigh, ni, child,
                         ichild, height_col, n);
}

void ref_xyz2key(uintk* key, const uintk* xyz, int num, int depth) { xyz2key_cpu<uintk>(key, xyz, num, depth); }
void ref_key2xyz(uintk* xyz, const uintk* key, int num, int depth) { key2xyz_cpu<uintk>(xyz, key, num, depth); }
void ref_search_key(int* idx, const uintk* key, int n_key, const uintk* query, int n_query) {
  search_key_cpu<uintk>(idx, key, n_key, query, n_query);
}

// transform_points as pytorch/cpp/transform_points.cpp:71-108 drives the Points methods, in place on
// a copy of the buffer the caller made.
void ref_transform_points(char* buf, const float* angle, const float* scale, const float* jitter,
                          float offset, const char* normal_axis) {
  Points pts;
  pts.set(buf);
  const float kEPS = 1.0e-10f;
  if (offset > kEPS) pts.displace(offset);
  if (std::fabs(angle[0]) > kEPS || std::fabs(angle[1]) > kEPS || std::fabs(angle[2]) > kEPS) pts.rotate(angle);
  if (std::fabs(jitter[0]) > kEPS || std::fabs(jitter[1]) > kEPS || std::fabs(jitter[2]) > kEPS) pts.translate(jitter);
  if (scale[0] != 1.0f || scale[1] != 1.0f || scale[2] != 1.0f) pts.scale(scale);
  std::string axis(normal_axis);
  if (!axis.empty()) pts.orient_normal(axis);
}

// clip_points (transform_points.cpp:110-125): in place; mask receives the in-box flags.
void ref_clip_points(char* buf, const float* bbmin, const float* bbmax, int* mask) {
  Points pts;
  pts.set(buf);
  const std::vector<int> in = pts.clip(bbmin, bbmax);
  memcpy(mask, in.data(), in.size() * sizeof(int));
}

void ref_bounding_box(const float* pt, int npt, float* out6) { bounding_box(out6, out6 + 3, pt, npt); }

// octree_new (pytorch/cpp/octree_grow.cpp:108-148): the same OctreeInfo calls in the same order.
long ref_octree_new(int batch_size, int channel, int node_dis, int adaptive_layer, char* out, long cap) {
  const int node_num = batch_size, depth = 0;
  OctreeInfo oct_info;
  oct_info.set_batch_size(batch_size);
  oct_info.set_depth(depth);
  oct_info.set_full_layer(depth);
  oct_info.set_node_dis(node_dis != 0);
  if (adaptive_layer > 1) {
    oct_info.set_adaptive(true);
    oct_info.set_adaptive_layer(adaptive_layer);
  } else {
    oct_info.set_adaptive(false);
  }
  oct_info.set_key2xyz(true);
  oct_info.set_property(OctreeInfo::kKey, 1, -1);
  oct_info.set_property(OctreeInfo::kChild, 1, -1);
  oct_info.set_property(OctreeInfo::kNeigh, 8, -1);
  oct_info.set_property(OctreeInfo::kFeature, channel, -1);
  float bbmin[] = {0, 0, 0};
  float bbmax[] = {2, 2, 2};
  oct_info.set_bbox(bbmin, bbmax);
  oct_info.set_nnum(depth, node_num);
  oct_info.set_nnum_cum();
  oct_info.set_nempty(depth, node_num);
  oct_info.set_ptr_dis();
  std::vector<char> buf(oct_info.sizeof_octree(), 0);
  OctreeParser octree_out;
  octree_out.set_cpu(buf.data(), &oct_info);
  sequence_cpu(octree_out.mutable_key_cpu(depth), node_num);
  sequence_cpu(octree_out.mutable_children_cpu(depth), node_num);
  return emit(buf, out, cap);
}

// octree_grow (pytorch/cpp/octree_grow.cpp:8-104) with the CPU versions of the functions the
// binding calls on the GPU (calc_neigh_cpu, generate_key_cpu, sequence_cpu: octree_nn.cpp).
long ref_octree_grow(const char* octree_in_buf, int target_depth, int full_octree, char* out, long cap) {
  OctreeParser octree_in;
  octree_in.set_cpu(octree_in_buf);
  const int batch_size = octree_in.info().batch_size();
  const int node_num = octree_in.info().node_num_nempty(target_depth - 1) << 3;
  OctreeInfo oct_info = octree_in.info();
  oct_info.set_depth(target_depth);
  if (full_octree) oct_info.set_full_layer(target_depth);
  float width = 1 << target_depth;
  float bbmin[] = {0, 0, 0};
  float bbmax[] = {width, width, width};
  oct_info.set_bbox(bbmin, bbmax);
  oct_info.set_nnum(target_depth, node_num);
  oct_info.set_nempty(target_depth, node_num);
  oct_info.set_nnum_cum();
  oct_info.set_ptr_dis();
  std::vector<char> buf(oct_info.sizeof_octree(), 0);
  OctreeParser octree_out;
  octree_out.set_cpu(buf.data(), &oct_info);
  const int node_num_cum = octree_in.info().node_num_cum(target_depth);
  memcpy(octree_out.mutable_key_cpu(0), octree_in.key_cpu(0),
         sizeof(uintk) * node_num_cum * octree_in.info().channel(OctreeInfo::kKey));
  memcpy(octree_out.mutable_children_cpu(0), octree_in.children_cpu(0),
         sizeof(int) * node_num_cum * octree_in.info().channel(OctreeInfo::kChild));
  memcpy(octree_out.mutable_neighbor_cpu(0), octree_in.neighbor_cpu(0),
         sizeof(int) * node_num_cum * octree_in.info().channel(OctreeInfo::kNeigh));
  if (octree_in.info().channel(OctreeInfo::kFeature) > 0)
    memcpy(octree_out.mutable_feature_cpu(0), octree_in.feature_cpu(0),
           sizeof(float) * node_num_cum * octree_in.info().channel(OctreeInfo::kFeature));
  if (full_octree) {
    calc_neigh_cpu(octree_out.mutable_neighbor_cpu(target_depth), target_depth, batch_size);
    generate_key_cpu(octree_out.mutable_key_cpu(target_depth), target_depth, batch_size);
    sequence_cpu(octree_out.mutable_children_cpu(target_depth), node_num);
  } else {
    const int* label_ptr = octree_out.children_cpu(target_depth - 1);
    calc_neigh_cpu(octree_out.mutable_neighbor_cpu(target_depth),
                   octree_out.neighbor_cpu(target_depth - 1), label_ptr,
                   octree_out.info().node_num(target_depth - 1));
    generate_key_cpu(octree_out.mutable_key_cpu(target_depth),
                     octree_out.key_cpu(target_depth - 1), label_ptr,
                     octree_out.info().node_num(target_depth - 1));
    sequence_cpu(octree_out.mutable_children_cpu(target_depth), node_num);
  }
  return emit(buf, out, cap);
}

// octree_update (pytorch/cpp/octree_grow.cpp:150-177) with generate_label_cpu.  In place.
void ref_octree_update(char* octree_buf, const int* label, int depth, int split) {
  OctreeParser octree_;
  octree_.set_cpu(octree_buf);
  const int node_num = octree_.info().node_num(depth);
  int split_num = 0;
  int* children = octree_.mutable_children_cpu(depth);
  generate_label_cpu(children, split_num, label, node_num, split);
  if (split_num == 0) {
    split_num = 1;
    children[0] = 0;
  }
  octree_.mutable_info().set_nempty(depth, split_num);
}

}  // extern "C"
