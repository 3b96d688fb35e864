// Octree wire-format constants and host helpers shared by the builder and the merge.
#pragma once

#include "common.cuh"

namespace ocnn {

// Byte offsets of the OctreeInfo fields (octree/octree/octree_info.h:93-116; sizeof = 716).
enum : int {
  kOffMagic = 0, kOffBatch = 16, kOffDepth = 20, kOffFull = 24, kOffAdpLayer = 28,
  kOffIsAdaptive = 32, kOffThDist = 36, kOffThNorm = 40, kOffKey2Xyz = 44, kOffNodeDis = 45,
  kOffNnum = 48, kOffNnumCum = 112, kOffNnumNempty = 176, kOffFlags = 240, kOffChannels = 244,
  kOffLocations = 308, kOffBbmin = 372, kOffBbmax = 384, kOffExtrapolate = 396,
  kOffSavePts = 397, kOffPtrDis = 652
};

// Header fields that ocnn_octree_meta does not carry.
struct HeaderExtras {
  int adp_depth = 0;
  float th_distance = 0.f, th_normal = 0.f;
  float bbmin[3] = {-1.f, -1.f, -1.f}, bbmax[3] = {1.f, 1.f, 1.f};
};

// nnum_cum and ptr_dis from nnum / channels / locations
// (OctreeInfo::set_nnum_cum, set_ptr_dis: octree_info.cpp:216-223, 254-268).
void finish_meta(ocnn_octree_meta* meta);
// Serialise the 720 header bytes.
void write_header(const ocnn_octree_meta* meta, const HeaderExtras& extras, uint8_t* out720);

}  // namespace ocnn
