// Host-side reader/writer of the octree wire format: the 716-byte OctreeInfo header followed by
// the Key | Child | Neigh | Feature | Label | Split blocks.  Field offsets follow
// octree/octree/octree_info.h:93-116 of the reference; block offsets follow
// OctreeInfo::set_ptr_dis (octree_info.cpp:254-268).
#include <cstring>

#include "header.h"

namespace ocnn {

static int elem_size(int prop, int key_bits) { return prop == OCNN_PROP_KEY ? key_bits / 8 : 4; }

void finish_meta(ocnn_octree_meta* m) {
  const int depth = m->depth;
  m->nnum_cum[0] = 0;
  for (int d = 1; d < depth + 2; ++d) m->nnum_cum[d] = m->nnum_cum[d - 1] + m->nnum[d - 1];
  m->nnum_cum[depth + 2] = m->nnum_cum[depth + 1];
  m->ptr_dis[0] = OCNN_HEADER_BYTES;
  for (int p = 0; p < OCNN_PROP_COUNT; ++p) {
    const int lc = m->channels[p] != 0 ? m->locations[p] : 0;
    const int64_t n = lc == -1 ? m->nnum_cum[depth + 2] : m->nnum[lc];
    m->ptr_dis[p + 1] = m->ptr_dis[p] + (int64_t)elem_size(p, m->key_bits) * n * m->channels[p];
  }
}

void write_header(const ocnn_octree_meta* m, const HeaderExtras& ex, uint8_t* out) {
  memset(out, 0, OCNN_HEADER_BYTES);
  memcpy(out + kOffMagic, m->key_bits == 64 ? "_OCTREE_2.0_" : "_OCTREE_1.0_", 12);
  auto i32 = [&](int off) { return reinterpret_cast<int32_t*>(out + off); };
  auto f32 = [&](int off) { return reinterpret_cast<float*>(out + off); };
  *i32(kOffBatch) = m->batch_size;
  *i32(kOffDepth) = m->depth;
  *i32(kOffFull) = m->full_depth;
  *i32(kOffAdpLayer) = ex.adp_depth;
  out[kOffIsAdaptive] = (uint8_t)(m->is_adaptive != 0);
  *f32(kOffThDist) = ex.th_distance;
  *f32(kOffThNorm) = ex.th_normal;
  out[kOffKey2Xyz] = (uint8_t)(m->key2xyz != 0);
  out[kOffNodeDis] = (uint8_t)(m->has_node_dis != 0);
  int flags = 0;
  for (int d = 0; d < OCNN_MAX_DEPTH; ++d) {
    i32(kOffNnum)[d] = m->nnum[d];
    i32(kOffNnumCum)[d] = m->nnum_cum[d];
    i32(kOffNnumNempty)[d] = m->nnum_nempty[d];
  }
  for (int p = 0; p < OCNN_PROP_COUNT; ++p) {
    i32(kOffChannels)[p] = m->channels[p];
    i32(kOffLocations)[p] = m->channels[p] != 0 ? m->locations[p] : 0;
    if (m->channels[p] != 0) flags |= 1 << p;
    i32(kOffPtrDis)[p] = (int32_t)m->ptr_dis[p];
  }
  i32(kOffPtrDis)[OCNN_PROP_COUNT] = (int32_t)m->ptr_dis[OCNN_PROP_COUNT];
  *i32(kOffFlags) = flags;
  for (int j = 0; j < 3; ++j) {
    f32(kOffBbmin)[j] = ex.bbmin[j];
    f32(kOffBbmax)[j] = ex.bbmax[j];
  }
  out[kOffExtrapolate] = 0;
  out[kOffSavePts] = (uint8_t)(m->save_pts != 0);
}

}  // namespace ocnn

extern "C" {

int ocnn_parse_header(const void* header_host, size_t nbytes, ocnn_octree_meta* meta) {
  using namespace ocnn;
  OCNN_REQUIRE(header_host != nullptr && meta != nullptr, "ocnn_parse_header: null argument");
  OCNN_REQUIRE(nbytes >= 716, "octree buffer of %zu bytes is shorter than its 716-byte header",
               nbytes);
  const uint8_t* h = static_cast<const uint8_t*>(header_host);
  memset(meta, 0, sizeof(*meta));
  if (memcmp(h, "_OCTREE_1.0_", 13) == 0) {
    meta->key_bits = 32;
  } else if (memcmp(h, "_OCTREE_2.0_", 13) == 0) {
    meta->key_bits = 64;
  } else {
    return fail(OCNN_ERR_INVALID, "not an octree buffer (bad magic string)");
  }
  auto i32 = [&](int off) { return reinterpret_cast<const int32_t*>(h + off); };
  meta->batch_size = *i32(kOffBatch);
  meta->depth = *i32(kOffDepth);
  meta->full_depth = *i32(kOffFull);
  meta->is_adaptive = h[kOffIsAdaptive] != 0;
  meta->key2xyz = h[kOffKey2Xyz] != 0;
  meta->has_node_dis = h[kOffNodeDis] != 0;
  meta->save_pts = h[kOffSavePts] != 0;
  const int max_depth = meta->key_bits == 64 ? 16 : 8;
  OCNN_REQUIRE(meta->batch_size >= 0, "octree header: negative batch size %d", meta->batch_size);
  // (depth 0 with full layer 1 is what octree_new makes: pytorch/cpp/octree_grow.cpp:108-148)
  OCNN_REQUIRE(meta->depth >= 0 && meta->depth <= max_depth && meta->depth < OCNN_MAX_DEPTH,
               "octree header: depth %d outside [0, %d]", meta->depth,
               max_depth < OCNN_MAX_DEPTH ? max_depth : OCNN_MAX_DEPTH - 1);
  OCNN_REQUIRE(meta->full_depth >= 0 && meta->full_depth <= (meta->depth > 1 ? meta->depth : 1),
               "octree header: full layer %d outside [0, depth]", meta->full_depth);
  const int flags = *i32(kOffFlags);
  for (int d = 0; d < OCNN_MAX_DEPTH; ++d) {
    meta->nnum[d] = i32(kOffNnum)[d];
    meta->nnum_cum[d] = i32(kOffNnumCum)[d];
    meta->nnum_nempty[d] = i32(kOffNnumNempty)[d];
  }
  for (int d = 0; d <= meta->depth; ++d) {
    OCNN_REQUIRE(meta->nnum[d] >= 0 && meta->nnum_nempty[d] >= 0 &&
                     meta->nnum_nempty[d] <= meta->nnum[d],
                 "octree header: bad node counts at level %d", d);
  }
  for (int p = 0; p < OCNN_PROP_COUNT; ++p) {
    meta->channels[p] = i32(kOffChannels)[p];
    meta->locations[p] = i32(kOffLocations)[p];
    meta->ptr_dis[p] = i32(kOffPtrDis)[p];
    OCNN_REQUIRE(meta->channels[p] >= 0, "octree header: negative channel count");
    OCNN_REQUIRE((meta->channels[p] == 0) == ((flags & (1 << p)) == 0),
                 "octree header: content flags do not match channels[%d]", p);
    OCNN_REQUIRE(meta->channels[p] == 0 || meta->locations[p] == -1 ||
                     meta->locations[p] == meta->depth,
                 "octree header: locations[%d] must be -1 or the depth", p);
  }
  meta->ptr_dis[OCNN_PROP_COUNT] = i32(kOffPtrDis)[OCNN_PROP_COUNT];
  OCNN_REQUIRE(meta->ptr_dis[0] >= 716 && meta->ptr_dis[OCNN_PROP_COUNT] >= meta->ptr_dis[0],
               "octree header: bad block offsets");
  return OCNN_OK;
}

int64_t ocnn_prop_offset(const ocnn_octree_meta* m, int prop, int depth) {
  if (m == nullptr || prop < 0 || prop >= OCNN_PROP_COUNT || m->channels[prop] == 0) return -1;
  int64_t off = m->ptr_dis[prop];
  if (m->locations[prop] == -1) {
    if (depth < 0 || depth > m->depth) return -1;
    off += (int64_t)m->nnum_cum[depth] * m->channels[prop] * ocnn::elem_size(prop, m->key_bits);
  }
  return off;
}

}  // extern "C"
