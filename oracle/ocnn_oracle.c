/* TEST INFRASTRUCTURE ONLY — CPU oracle for the octree hot path.
 *
 * A plain-C restatement, written for this repository, of what the reference's CPU code computes
 * for: points -> octree build, batch merge, the neighbour table, octree2col, the convolution,
 * max-pool, pad and depad.  Every function cites the reference lines whose behaviour it restates
 * (paths are relative to the microsoft/O-CNN checkout).  The shipped CUDA library never links or
 * calls this file: only tests, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity pin: tests/test_oracle_vs_reference.py checks every function here, bit for bit, against
 * the reference's own compiled CPU sources (oracle/_ref) where those are present, and against the
 * committed fixtures under tests/golden/ (generated from the reference by
 * tests/golden/make_golden.py) everywhere else.
 *
 * Floating point: compiled with -ffp-contract=off so that no multiply-add is fused, matching the
 * reference built by g++ -O2 for x86-64 (separate mulss/addss).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- wire format ------------------------------------------------------------------------ */
/* OctreeInfo field offsets, octree/octree/octree_info.h:93-116 (sizeof == 716, first block at
 * 720: octree_info.cpp:254-268). */
enum {
  H_MAGIC = 0, H_BATCH = 16, H_DEPTH = 20, H_FULL = 24, H_ADP = 28, H_IS_ADP = 32,
  H_TH_DIST = 36, H_TH_NORM = 40, H_KEY2XYZ = 44, H_NODE_DIS = 45, H_NNUM = 48,
  H_NNUM_CUM = 112, H_NNUM_NE = 176, H_FLAGS = 240, H_CHANNELS = 244, H_LOCATIONS = 308,
  H_BBMIN = 372, H_BBMAX = 384, H_EXTRAP = 396, H_SAVE_PTS = 397, H_PTR_DIS = 652,
  H_SIZE = 716
};
/* property slots, octree_info.h:12-15 */
enum { P_KEY = 0, P_CHILD = 1, P_NEIGH = 2, P_FEATURE = 3, P_LABEL = 4, P_SPLIT = 5, P_COUNT = 6 };

/* PointsInfo, octree/octree/points_info.h:34-39: magic[16] pt_num flags channels[8] ptr_dis[8] */
enum { PT_NUM = 16, PT_FLAGS = 20, PT_CHANNELS = 24, PT_PTR_DIS = 56, PT_SIZE = 88 };

static int32_t *hi(uint8_t *h, int off) { return (int32_t *)(h + off); }
static const int32_t *hci(const uint8_t *h, int off) { return (const int32_t *)(h + off); }

static int key_bytes_of(const uint8_t *h) {
  /* "_OCTREE_1.0_" = 32-bit keys, "_OCTREE_2.0_" = 64-bit (octree_info.cpp:7-11) */
  return h[8] == '2' ? 8 : 4;
}

static int prop_elem_size(int p, int key_bytes) { return p == P_KEY ? key_bytes : 4; }

/* nnum_cum and ptr_dis from nnum/channels/locations: octree_info.cpp:216-223, 254-268 */
static void finish_header(uint8_t *h, int key_bytes) {
  int depth = *hi(h, H_DEPTH);
  int32_t *nnum = hi(h, H_NNUM), *cum = hi(h, H_NNUM_CUM);
  int32_t *ch = hi(h, H_CHANNELS), *loc = hi(h, H_LOCATIONS), *dis = hi(h, H_PTR_DIS);
  cum[0] = 0;
  for (int d = 1; d < depth + 2; ++d) cum[d] = cum[d - 1] + nnum[d - 1];
  cum[depth + 2] = cum[depth + 1];
  int flags = 0;
  for (int p = 0; p < P_COUNT; ++p) if (ch[p] != 0) flags |= 1 << p;
  *hi(h, H_FLAGS) = flags;
  dis[0] = (H_SIZE + 7) / 8 * 8;
  for (int p = 0; p < P_COUNT; ++p) {
    int lc = ch[p] != 0 ? loc[p] : 0;
    int n = lc == -1 ? cum[depth + 2] : nnum[lc];
    dis[p + 1] = dis[p] + prop_elem_size(p, key_bytes) * n * ch[p];
  }
}

/* address of (property, level): octree_info.cpp:157-167 */
static long prop_offset(const uint8_t *h, int p, int d) {
  const int32_t *ch = hci(h, H_CHANNELS);
  if (ch[p] == 0) return -1;
  long off = hci(h, H_PTR_DIS)[p];
  if (hci(h, H_LOCATIONS)[p] == -1)
    off += (long)hci(h, H_NNUM_CUM)[d] * ch[p] * prop_elem_size(p, key_bytes_of(h));
  return off;
}

long oc_prop_offset(const uint8_t *octree, int prop, int d) { return prop_offset(octree, prop, d); }

static void put_key(uint8_t *dst, long i, uint64_t k, int key_bytes) {
  if (key_bytes == 8) ((uint64_t *)dst)[i] = k; else ((uint32_t *)dst)[i] = (uint32_t)k;
}
static uint64_t get_key(const uint8_t *src, long i, int key_bytes) {
  return key_bytes == 8 ? ((const uint64_t *)src)[i] : ((const uint32_t *)src)[i];
}

/* ---- Morton key ------------------------------------------------------------------------- */
/* bit i of x -> key bit 3i+2, of y -> 3i+1, of z -> 3i, for i < depth
 * (compute_key, octree/octree/octree_nn.cpp:551-560) */
uint64_t oc_morton(uint64_t x, uint64_t y, uint64_t z, int depth) {
  uint64_t key = 0;
  for (int i = 0; i < depth; ++i) {
    key |= ((x >> i) & 1ull) << (3 * i + 2);
    key |= ((y >> i) & 1ull) << (3 * i + 1);
    key |= ((z >> i) & 1ull) << (3 * i);
  }
  return key;
}

typedef struct { uint64_t key; uint64_t idx; } KeyIdx;
static int cmp_keyidx(const void *a, const void *b) {
  const KeyIdx *p = (const KeyIdx *)a, *q = (const KeyIdx *)b;
  if (p->key != q->key) return p->key < q->key ? -1 : 1;
  return p->idx < q->idx ? -1 : (p->idx > q->idx ? 1 : 0);
}

/* ---- points -> octree ------------------------------------------------------------------- */
/* Restates Octree::build (octree/octree/octree.cpp:74-121) for the non-adaptive case with the
 * signal stored at the finest level only (node_feature = adaptive = extrapolate = key2xyz = 0),
 * driven the way pytorch/cpp/point2octree.cpp:5-34 drives it.  bbox = NULL means [-1,1]^3
 * (octree_info.cpp:68-69).  Returns the octree size in bytes; writes it when cap is enough. */
long oc_points2octree(const uint8_t *points, int depth, int full_depth, int node_dis,
                      int split_label, int save_pts, int key_bits, int adp_depth,
                      float th_normal, float th_distance, const float *bbox,
                      uint8_t *out, long cap) {
  const int key_bytes = key_bits / 8;
  const int npt = *hci(points, PT_NUM);
  const int pflags = *hci(points, PT_FLAGS);
  const int32_t *pch = hci(points, PT_CHANNELS), *pdis = hci(points, PT_PTR_DIS);
  if (npt <= 0) return -1;
  const float *xyz = (const float *)(points + pdis[0]);
  const float *normals = (pflags & 2) ? (const float *)(points + pdis[1]) : NULL;
  const float *feats = (pflags & 4) ? (const float *)(points + pdis[2]) : NULL;
  const float *labels = (pflags & 8) ? (const float *)(points + pdis[3]) : NULL;
  const int cn = normals ? pch[1] : 0, cf = feats ? pch[2] : 0;

  /* header: OctreeInfo::initialize, octree_info.cpp:13-73 */
  uint8_t hdr[H_SIZE];
  memset(hdr, 0, H_SIZE);
  memcpy(hdr, key_bytes == 8 ? "_OCTREE_2.0_" : "_OCTREE_1.0_", 12);
  *hi(hdr, H_BATCH) = 1;
  *hi(hdr, H_DEPTH) = depth;                       /* set_depth before set_full_layer */
  const int full = full_depth < 1 ? 1 : full_depth;
  *hi(hdr, H_FULL) = full;
  *hi(hdr, H_ADP) = adp_depth;                     /* recorded even when not adaptive */
  *(float *)(hdr + H_TH_DIST) = th_distance;
  *(float *)(hdr + H_TH_NORM) = th_normal;
  hdr[H_NODE_DIS] = node_dis != 0;
  hdr[H_SAVE_PTS] = save_pts != 0;
  int32_t *ch = hi(hdr, H_CHANNELS), *loc = hi(hdr, H_LOCATIONS);
  ch[P_KEY] = 1; loc[P_KEY] = -1;
  ch[P_CHILD] = 1; loc[P_CHILD] = -1;
  if (split_label) { ch[P_SPLIT] = 1; loc[P_SPLIT] = -1; }
  int cfeat = cn + cf;
  if (node_dis) cfeat += normals ? 1 : 4;
  if (save_pts) cfeat += 3;
  ch[P_FEATURE] = cfeat; loc[P_FEATURE] = depth;
  if (labels && pch[3] == 1) { ch[P_LABEL] = 1; loc[P_LABEL] = depth; }
  float *bbmin = (float *)(hdr + H_BBMIN), *bbmax = (float *)(hdr + H_BBMAX);
  for (int j = 0; j < 3; ++j) { bbmin[j] = bbox ? bbox[j] : -1.0f; bbmax[j] = bbox ? bbox[3 + j] : 1.0f; }

  /* normalize_pts: octree.cpp:155-170; width: octree_info.cpp:169-178 */
  float width = bbmax[0] - bbmin[0];
  for (int j = 1; j < 3; ++j) { float w = bbmax[j] - bbmin[j]; if (w > width) width = w; }
  if (width == 0.0f) width = 1.0e-10f;
  const float mul = (float)(1 << depth) / width;
  float *scaled = (float *)malloc(sizeof(float) * 3 * (size_t)npt);
  for (long i = 0; i < 3L * npt; ++i) scaled[i] = (xyz[i] - bbmin[i % 3]) * mul;

  /* sort_keys: octree.cpp:172-203 (truncate toward zero, interleave, sort (key, idx) pairs) */
  KeyIdx *code = (KeyIdx *)malloc(sizeof(KeyIdx) * (size_t)npt);
  const uint64_t cell_mask = key_bytes == 8 ? ~0ull : 0xffffffffull;
  for (long i = 0; i < npt; ++i) {
    uint64_t c[3];
    for (int j = 0; j < 3; ++j) {
      float v = scaled[3 * i + j];
      c[j] = (key_bytes == 8 ? (uint64_t)v : (uint64_t)(uint32_t)v) & cell_mask;
    }
    code[i].key = oc_morton(c[0], c[1], c[2], depth);
    code[i].idx = (uint64_t)i;
  }
  qsort(code, (size_t)npt, sizeof(KeyIdx), cmp_keyidx);

  /* unique_key: octree.cpp:890-904 -> finest non-empty keys + point segments */
  uint64_t *cur = (uint64_t *)malloc(sizeof(uint64_t) * (size_t)npt);
  long *seg = (long *)malloc(sizeof(long) * ((size_t)npt + 1));
  long ncur = 0;
  for (long i = 0; i < npt; ++i)
    if (i == 0 || code[i].key != code[i - 1].key) { seg[ncur] = i; cur[ncur++] = code[i].key; }
  seg[ncur] = npt;
  const long nfinest_keys = ncur;

  /* build_structure: octree.cpp:205-283 */
  uint64_t **keys = (uint64_t **)calloc((size_t)depth + 1, sizeof(uint64_t *));
  int32_t **child = (int32_t **)calloc((size_t)depth + 1, sizeof(int32_t *));
  int32_t *nnum = hi(hdr, H_NNUM), *nne = hi(hdr, H_NNUM_NE);
  for (int d = 0; d <= full; ++d) {
    long n = 1L << (3 * d);
    nnum[d] = (int32_t)n;
    keys[d] = (uint64_t *)malloc(sizeof(uint64_t) * (size_t)n);
    child[d] = (int32_t *)malloc(sizeof(int32_t) * (size_t)n);
    for (long i = 0; i < n; ++i) { keys[d][i] = (uint64_t)i; child[d][i] = d < full ? (int32_t)i : -1; }
  }
  uint64_t *par = (uint64_t *)malloc(sizeof(uint64_t) * (size_t)npt);
  for (int d = depth; d > full; --d) {
    /* parents = unique(cur >> 3); node (8a+j) of level d has key (parent[a] << 3) | j */
    long np = 0;
    long *slot = (long *)malloc(sizeof(long) * (size_t)ncur);
    for (long i = 0; i < ncur; ++i) {
      uint64_t pk = cur[i] >> 3;
      if (i == 0 || pk != par[np - 1]) par[np++] = pk;
      slot[i] = ((np - 1) << 3) | (long)(cur[i] & 7);
    }
    long n = np << 3;
    nnum[d] = (int32_t)n;
    keys[d] = (uint64_t *)malloc(sizeof(uint64_t) * (size_t)n);
    child[d] = (int32_t *)malloc(sizeof(int32_t) * (size_t)n);
    for (long i = 0; i < n; ++i) { keys[d][i] = (par[i >> 3] << 3) | (uint64_t)(i & 7); child[d][i] = -1; }
    for (long i = 0; i < ncur; ++i) child[d][slot[i]] = (int32_t)i;
    free(slot);
    uint64_t *t = cur; cur = par; par = t; ncur = np;
  }
  if (depth > full)
    for (long i = 0; i < ncur; ++i) child[full][cur[i]] = (int32_t)i;

  /* calc_node_num: octree.cpp:285-309 */
  for (int d = 0; d <= depth; ++d) {
    nne[d] = 0;
    for (long i = nnum[d] - 1; i >= 0; --i)
      if (child[d][i] != -1) { nne[d] = child[d][i] + 1; break; }
  }
  finish_header(hdr, key_bytes);
  const long total = hi(hdr, H_PTR_DIS)[P_COUNT];
  long ret = total;
  if (out == NULL || cap < total) goto done;

  memset(out, 0, (size_t)total);
  memcpy(out, hdr, H_SIZE);
  /* serialize: octree.cpp:907-956 */
  for (int d = 0; d <= depth; ++d) {
    uint8_t *kd = out + prop_offset(out, P_KEY, d);
    int32_t *cd = (int32_t *)(out + prop_offset(out, P_CHILD, d));
    for (long i = 0; i < nnum[d]; ++i) { put_key(kd, i, keys[d][i], key_bytes); cd[i] = child[d][i]; }
    if (split_label) {   /* calc_split_label, non-adaptive: octree.cpp:1158-1179 */
      float *sd = (float *)(out + prop_offset(out, P_SPLIT, d));
      for (long i = 0; i < nnum[d]; ++i) sd[i] = child[d][i] == -1 ? 0.0f : 1.0f;
    }
  }

  /* calc_signal at the finest level: octree.cpp:312-452.  Channel rows in the feature block:
   * normals, displacement, point features, average points (serialize, octree.cpp:916-926). */
  {
    const long nn = nnum[depth];
    float *fd = (float *)(out + prop_offset(out, P_FEATURE, depth));
    float *f_normal = fd;
    float *f_dis = f_normal + (long)cn * nn;
    float *f_feat = f_dis + (node_dis ? (normals ? 1 : 4) * nn : 0);
    float *f_pts = f_feat + (long)cf * nn;
    float *ld = ch[P_LABEL] ? (float *)(out + prop_offset(out, P_LABEL, depth)) : NULL;
    int max_label = 0;
    if (ld) {
      float m = labels[0];
      for (long i = 1; i < npt; ++i) if (labels[i] > m) m = labels[i];
      max_label = (int)m + 1;
      for (long i = 0; i < nn; ++i) ld[i] = -1.0f;
    }
    int *votes = max_label > 0 ? (int *)malloc(sizeof(int) * (size_t)max_label) : NULL;
    float *acc = (float *)malloc(sizeof(float) * (size_t)(cn + cf + 3));
    for (long i = 0; i < nn; ++i) {
      const int t = child[depth][i];
      if (t == -1) continue;
      const long s0 = seg[t], s1 = seg[t + 1];
      if (normals) {
        for (int c = 0; c < cn; ++c) acc[c] = 0.0f;
        for (long j = s0; j < s1; ++j)
          for (int c = 0; c < cn; ++c) acc[c] += normals[cn * code[j].idx + c];
        float len = 0.0f;
        for (int c = 0; c < cn; ++c) len += acc[c] * acc[c];
        float factor = sqrtf(len);
        if (factor < 1.0e-6f) {
          for (int c = 0; c < cn; ++c) acc[c] = normals[cn * code[s0].idx + c];
          len = 0.0f;
          for (int c = 0; c < cn; ++c) len += acc[c] * acc[c];
          factor = sqrtf(len) + 1.0e-30f;
        }
        for (int c = 0; c < cn; ++c) f_normal[c * nn + i] = acc[c] / factor;
      }
      if (feats) {
        for (int c = 0; c < cf; ++c) acc[c] = 0.0f;
        for (long j = s0; j < s1; ++j)
          for (int c = 0; c < cf; ++c) acc[c] += feats[cf * code[j].idx + c];
        const float factor = (float)(uint64_t)(s1 - s0) + 1.0e-30f;
        for (int c = 0; c < cf; ++c) f_feat[c * nn + i] = acc[c] / factor;
      }
      if (ld) {
        int valid = 0;
        for (int l = 0; l < max_label; ++l) votes[l] = 0;
        for (long j = s0; j < s1; ++j) {
          int l = (int)labels[code[j].idx];
          if (l < 0) continue;
          votes[l] += 1; valid += 1;
        }
        if (valid > 0) {
          int best = 0;
          for (int l = 1; l < max_label; ++l) if (votes[l] > votes[best]) best = l;
          ld[i] = (float)best;
        }
      }
      if (node_dis || save_pts) {
        float avg[3] = {0.0f, 0.0f, 0.0f}, dis[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (long j = s0; j < s1; ++j)
          for (int c = 0; c < 3; ++c) avg[c] += scaled[3 * code[j].idx + c];
        const float factor = (float)(uint64_t)(s1 - s0) + 1.0e-30f;
        for (int c = 0; c < 3; ++c) {
          avg[c] /= factor;
          float ip;
          dis[c] = modff(avg[c], &ip) - 0.5f;
          if (normals) dis[3] += dis[c] * f_normal[c * nn + i]; else dis[3] = 1.0f;
          if (save_pts) f_pts[c * nn + i] = avg[c];
        }
        if (node_dis) {
          if (normals) {
            f_dis[i] = dis[3] * 1.1547f;
          } else {
            for (int c = 0; c < 3; ++c) f_dis[c * nn + i] = dis[c];
            f_dis[3 * nn + i] = dis[3] * 1.1547f;
          }
        }
      }
    }
    free(acc); free(votes);
  }
  (void)nfinest_keys;

done:
  for (int d = 0; d <= depth; ++d) { free(keys[d]); free(child[d]); }
  free(keys); free(child); free(par); free(cur); free(seg); free(code); free(scaled);
  return ret;
}

/* ---- neighbour table -------------------------------------------------------------------- */
/* ni table of the 3x3x3 kernel: entry (octant o, tap t) is the position, inside the 4x4x4 block of
 * o's sibling group, of the cell at offset (tx-1, ty-1, tz-1) from o
 * (NeighHelper::init_neigh_index, octree/octree/octree_nn.cpp:22-37). */
static int ni333(int o, int t) {
  int ox = o >> 2, oy = (o >> 1) & 1, oz = o & 1;
  int tx = t / 9, ty = (t / 3) % 3, tz = t % 3;
  return ((tx + ox) << 4) | ((ty + oy) << 2) | (tz + oz);
}

/* taps of the 27 selected by each supported kernel shape (octree_nn.cpp:7-19) */
static int kernel_taps(const int ks[3], int taps[27]) {
  static const int t222[8] = {13, 14, 16, 17, 22, 23, 25, 26};
  static const int t311[3] = {4, 13, 22}, t131[3] = {10, 13, 16}, t113[3] = {12, 13, 14};
  static const int t331[9] = {1, 4, 7, 10, 13, 16, 19, 22, 25};
  static const int t313[9] = {3, 4, 5, 12, 13, 14, 21, 22, 23};
  static const int t133[9] = {9, 10, 11, 12, 13, 14, 15, 16, 17};
  const int code = ks[0] * 100 + ks[1] * 10 + ks[2];
  const int *src = NULL; int n = 0;
  switch (code) {
    case 333: for (int i = 0; i < 27; ++i) taps[i] = i; return 27;
    case 111: taps[0] = 13; return 1;
    case 222: src = t222; n = 8; break;
    case 311: src = t311; n = 3; break;
    case 131: src = t131; n = 3; break;
    case 113: src = t113; n = 3; break;
    case 331: src = t331; n = 9; break;
    case 313: src = t313; n = 9; break;
    case 133: src = t133; n = 9; break;
    default: return -1;
  }
  memcpy(taps, src, sizeof(int) * (size_t)n);
  return n;
}

/* ni[o * K + k] for a kernel shape; returns 8*K or -1 (octree_nn.cpp:40-51) */
int oc_ni_table(const int ks[3], int *out) {
  int taps[27];
  const int K = kernel_taps(ks, taps);
  if (K < 0) return -1;
  if (out) for (int o = 0; o < 8; ++o) for (int k = 0; k < K; ++k) out[o * K + k] = ni333(o, taps[k]);
  return 8 * K;
}

/* Full levels (d <= full_depth), closed form: calc_neigh_cpu(neigh, depth, batch),
 * octree/octree/octree_nn.cpp:382-424. */
void oc_calc_neigh_full(int32_t *neigh, int depth, int batch) {
  const long per = 1L << (3 * depth);
  const long side = 1L << depth;
  for (int n = 0; n < batch; ++n) {
    for (long g = 0; g < per; g += 8) {
      long gx = 0, gy = 0, gz = 0;
      for (int b = 0; b < depth; ++b) {
        gx |= ((g >> (3 * b + 2)) & 1) << b;
        gy |= ((g >> (3 * b + 1)) & 1) << b;
        gz |= ((g >> (3 * b)) & 1) << b;
      }
      int32_t *blk = neigh + (g + n * per) * 8;
      for (int j = 0; j < 64; ++j) {
        long x = gx + (j >> 4) - 1, y = gy + ((j >> 2) & 3) - 1, z = gz + (j & 3) - 1;
        if (x < 0 || y < 0 || z < 0 || x >= side || y >= side || z >= side) { blk[j] = -1; continue; }
        blk[j] = (int32_t)(oc_morton((uint64_t)x, (uint64_t)y, (uint64_t)z, depth) + (uint64_t)(n * per));
      }
    }
  }
}

/* Deeper levels from the parent level: calc_neigh_cpu(neigh_split, neigh, children, node_num),
 * octree/octree/octree_nn.cpp:357-380; parent/displacement tables octree_nn.cpp:53-81.
 * Blocks of empty parents do not exist in the output (it has one block per non-empty parent). */
void oc_calc_neigh_split(int32_t *out, const int32_t *neigh, const int32_t *child, int nnum_parent) {
  for (int i = 0; i < nnum_parent; ++i) {
    const int l0 = child[i];
    if (l0 < 0) continue;
    const int32_t *blk0 = neigh + ((long)(i >> 3) << 6);
    int32_t *blk1 = out + ((long)l0 << 6);
    for (int j = 0; j < 64; ++j) {
      /* child-level offset j = (x,y,z) in 0..3 -> parent-level tap and the octant inside it */
      int x = (j >> 4) + 1, y = ((j >> 2) & 3) + 1, z = (j & 3) + 1;
      int tap = (x >> 1) * 9 + (y >> 1) * 3 + (z >> 1);
      int oct = ((x & 1) << 2) | ((y & 1) << 1) | (z & 1);
      int k = blk0[ni333(i & 7, tap)];
      int v = -1;
      if (k != -1 && child[k] != -1) v = (child[k] << 3) + oct;
      blk1[j] = v;
    }
  }
}

/* ---- batch merge ------------------------------------------------------------------------ */
/* merge_octrees, octree/octree/merge_octrees.cpp:7-198: level-wise concatenation, batch index in
 * the top key lane, children rebased by the cumulative non-empty count, features re-interleaved
 * per channel, and the neighbour property (8 ints per node) added. */
long oc_octree_batch(const uint8_t *const *in, int batch, uint8_t *out, long cap) {
  const uint8_t *h0 = in[0];
  const int key_bytes = key_bytes_of(h0);
  const int depth = *hci(h0, H_DEPTH), full = *hci(h0, H_FULL);
  uint8_t hdr[H_SIZE];
  memcpy(hdr, h0, H_SIZE);
  *hi(hdr, H_BATCH) = batch < 1 ? 1 : batch;
  int32_t *ch = hi(hdr, H_CHANNELS), *loc = hi(hdr, H_LOCATIONS);
  ch[P_NEIGH] = 8; loc[P_NEIGH] = -1;
  int32_t *nnum = hi(hdr, H_NNUM), *nne = hi(hdr, H_NNUM_NE);
  for (int d = 0; d <= depth; ++d) {
    nnum[d] = 0; nne[d] = 0;
    for (int b = 0; b < batch; ++b) { nnum[d] += hci(in[b], H_NNUM)[d]; nne[d] += hci(in[b], H_NNUM_NE)[d]; }
  }
  finish_header(hdr, key_bytes);
  const long total = hi(hdr, H_PTR_DIS)[P_COUNT];
  if (out == NULL || cap < total) return total;
  memset(out, 0, (size_t)total);
  memcpy(out, hdr, H_SIZE);

  for (int d = 0; d <= depth; ++d) {
    long node0 = 0, ne0 = 0;
    for (int b = 0; b < batch; ++b) {
      const uint8_t *src = in[b];
      const long n = hci(src, H_NNUM)[d];
      /* keys: batch id into byte 3 (32-bit) / uint16 lane 3 (64-bit): merge_octrees.cpp:120-132 */
      if (ch[P_KEY]) {
        const uint8_t *ks = src + prop_offset(src, P_KEY, d);
        uint8_t *kd = out + prop_offset(out, P_KEY, d);
        for (long j = 0; j < n; ++j) {
          uint64_t k = get_key(ks, j, key_bytes);
          if (key_bytes == 8) k = (k & 0x0000ffffffffffffull) | ((uint64_t)(b & 0xffff) << 48);
          else k = (k & 0x00ffffffull) | ((uint64_t)(b & 0xff) << 24);
          put_key(kd, node0 + j, k, key_bytes);
        }
      }
      if (ch[P_CHILD]) {   /* merge_octrees.cpp:136-144 */
        const int32_t *cs = (const int32_t *)(src + prop_offset(src, P_CHILD, d));
        int32_t *cd = (int32_t *)(out + prop_offset(out, P_CHILD, d));
        for (long j = 0; j < n; ++j) cd[node0 + j] = cs[j] == -1 ? -1 : cs[j] + (int32_t)ne0;
      }
      if (ch[P_FEATURE] && (loc[P_FEATURE] == -1 || d == depth)) {   /* :147-158 */
        const float *fs = (const float *)(src + prop_offset(src, P_FEATURE, d));
        float *fd = (float *)(out + prop_offset(out, P_FEATURE, d));
        for (int c = 0; c < ch[P_FEATURE]; ++c)
          for (long j = 0; j < n; ++j) fd[(long)c * nnum[d] + node0 + j] = fs[(long)c * n + j];
      }
      if (ch[P_LABEL] && (loc[P_LABEL] == -1 || d == depth)) {       /* :161-170 */
        const float *ls = (const float *)(src + prop_offset(src, P_LABEL, d));
        float *ld = (float *)(out + prop_offset(out, P_LABEL, d));
        for (long j = 0; j < n; ++j) ld[node0 + j] = ls[j];
      }
      if (ch[P_SPLIT] && (loc[P_SPLIT] == -1 || d == depth)) {       /* :173-181 */
        const float *ss = (const float *)(src + prop_offset(src, P_SPLIT, d));
        float *sd = (float *)(out + prop_offset(out, P_SPLIT, d));
        for (long j = 0; j < n; ++j) sd[node0 + j] = ss[j];
      }
      node0 += n;
      ne0 += hci(src, H_NNUM_NE)[d];
    }
  }
  for (int d = 1; d <= depth; ++d) {                                  /* :184-197 */
    int32_t *nd = (int32_t *)(out + prop_offset(out, P_NEIGH, d));
    if (d <= full) {
      oc_calc_neigh_full(nd, d, batch);
    } else {
      oc_calc_neigh_split(nd, (const int32_t *)(out + prop_offset(out, P_NEIGH, d - 1)),
                          (const int32_t *)(out + prop_offset(out, P_CHILD, d - 1)), nnum[d - 1]);
    }
  }
  return total;
}

/* top[m, h] = sum_k w[m, k] * src[k, h], k ascending, in fp32 without fused multiply-add: the
 * same sequence of operations per output element as a plain dot-product loop, arranged so that the
 * inner loop runs along h (contiguous) instead of along k. */
static void gemm_rows(float *top, const float *w, const float *src, int M, long K, long H) {
  for (int m = 0; m < M; ++m) {
    float *row = top + (long)m * H;
    for (long h = 0; h < H; ++h) row[h] = 0.0f;
    for (long k = 0; k < K; ++k) {
      const float a = w[(long)m * K + k];
      const float *s = src + k * H;
      for (long h = 0; h < H; ++h) row[h] += a * s[h];
    }
  }
}

/* ---- octree2col / convolution ----------------------------------------------------------- */
/* col[(c*K + k)*H + h] = data[c*octree_h + neigh[...]] or 0:
 * octree2col_cpu, octree/octree/octree_nn.cpp:188-214 (single workspace chunk, n = 0). */
void oc_octree2col(float *col, const float *data, int channel, int height, int kdim, int stride,
                   const int32_t *neigh, const int32_t *ni) {
  const long octree_h = (long)height << (3 * (stride - 1));
  for (int c = 0; c < channel; ++c)
    for (int k = 0; k < kdim; ++k) {
      float *row = col + ((long)c * kdim + k) * height;
      for (long h = 0; h < height; ++h) {
        long at = stride == 2 ? (h << 6) + ni[k] : ((h >> 3) << 6) + ni[(h & 7) * kdim + k];
        int p = neigh[at];
        row[h] = p == -1 ? 0.0f : data[c * octree_h + p];
      }
    }
}

/* Y[Cout, Htop] = W[Cout, Cin*K] x col[Cin*K, Htop]: OctreeBaseConv::reshape / forward_cpu_gemm,
 * octree/octree/octree_conv.cpp:48-122, 158-180 (dense variant, nempty = false).  Stride 1:
 * Htop = nnum[depth]; stride 2: Htop = nnum_nempty[depth-1] (= nnum[depth]/8), un-padded; an
 * empty level is given height 1 (octree_conv.cpp:80).  The inner product runs over
 * k = cin*K + tap in increasing order in fp32.  Returns Cout*Htop. */
long oc_octree_conv(float *top, long cap, const float *bottom, const float *weights,
                    const uint8_t *octree, int depth, int cin, int cout, const int ks[3],
                    int stride) {
  int taps[27];
  const int K = kernel_taps(ks, taps);
  if (K < 0 || stride < 1 || stride > 2) return -1;
  const int32_t *nnum = hci(octree, H_NNUM), *nne = hci(octree, H_NNUM_NE);
  long top_h = stride == 2 ? nne[depth - 1] : nnum[depth];
  const long work_h = stride == 2 ? nnum[depth] / 8 : top_h;
  if (top_h == 0) top_h = 1;
  const long count = (long)cout * top_h;
  if (top == NULL || cap < count) return count;
  const int one = ks[0] == 1 && ks[1] == 1 && ks[2] == 1 && stride == 1;
  const long kd = (long)cin * K;
  float *col = NULL;
  const float *src = bottom;
  if (!one) {
    int ni[216];
    oc_ni_table(ks, ni);
    col = (float *)calloc((size_t)(kd * top_h), sizeof(float));
    float *tmp = (float *)malloc(sizeof(float) * (size_t)(kd * (work_h > 0 ? work_h : 1)));
    oc_octree2col(tmp, bottom, cin, (int)work_h, K, stride,
                  (const int32_t *)(octree + prop_offset(octree, P_NEIGH, depth)), ni);
    for (long r = 0; r < kd; ++r) memcpy(col + r * top_h, tmp + r * work_h, sizeof(float) * (size_t)work_h);
    free(tmp);
    src = col;
  }
  gemm_rows(top, weights, src, cout, kd, top_h);
  free(col);
  return count;
}

/* The same on non-empty nodes only (nempty = true, stride 1): octree2colP_cpu,
 * octree/octree/octree_nn.cpp:244-271.  data: [channel, octree_h] over the non-empty nodes of the
 * level, col: [channel*kdim, height] with height = number of non-empty nodes; ichild[i] = node of
 * the i-th non-empty node, child[node] = its rank among the non-empty nodes or -1. */
void oc_octree2col_p(float *col, const float *data, int channel, int height, int octree_h, int kdim,
                     const int32_t *neigh, const int32_t *ni, const int32_t *child,
                     const int32_t *ichild) {
  for (int c = 0; c < channel; ++c)
    for (int k = 0; k < kdim; ++k) {
      float *row = col + ((long)c * kdim + k) * height;
      for (long h = 0; h < height; ++h) {
        const long hp = ichild[h];
        int p = neigh[((hp >> 3) << 6) + ni[(hp & 7) * kdim + k]];
        if (p >= 0) p = child[p];
        row[h] = p < 0 ? 0.0f : data[(long)c * octree_h + p];
      }
    }
}

/* ichild as the PyTorch binding builds it: pad_backward of 0..nnum-1 through the child array
 * (pytorch/cpp/octree_conv.cpp:109-116). */
void oc_ichild(int32_t *ichild, const int32_t *child, int nnum) {
  for (int h = 0; h < nnum; ++h) if (child[h] != -1) ichild[child[h]] = h;
}

/* OctreeConv with nempty = true, stride 1: Y[Cout, nne] = W x colP (octree_conv.cpp:48-122 with
 * nempty_, 125-140).  Returns Cout * max(nne, 1). */
long oc_octree_conv_nempty(float *top, long cap, const float *bottom, const float *weights,
                           const uint8_t *octree, int depth, int cin, int cout, const int ks[3]) {
  int taps[27];
  const int K = kernel_taps(ks, taps);
  if (K < 0) return -1;
  const int32_t *nnum = hci(octree, H_NNUM), *nne = hci(octree, H_NNUM_NE);
  const long h_ne = nne[depth];
  const long top_h = h_ne == 0 ? 1 : h_ne;
  const long count = (long)cout * top_h;
  if (top == NULL || cap < count) return count;
  const long kd = (long)cin * K;
  const int one = ks[0] == 1 && ks[1] == 1 && ks[2] == 1;
  float *col = NULL;
  const float *src = bottom;
  if (!one && h_ne > 0) {
    int ni[216];
    oc_ni_table(ks, ni);
    const int32_t *child = (const int32_t *)(octree + prop_offset(octree, P_CHILD, depth));
    int32_t *ichild = (int32_t *)calloc((size_t)h_ne, sizeof(int32_t));
    oc_ichild(ichild, child, nnum[depth]);
    col = (float *)malloc(sizeof(float) * (size_t)(kd * h_ne));
    oc_octree2col_p(col, bottom, cin, (int)h_ne, (int)h_ne, K,
                    (const int32_t *)(octree + prop_offset(octree, P_NEIGH, depth)), ni, child, ichild);
    free(ichild);
    src = col;
  }
  if (h_ne > 0) gemm_rows(top, weights, src, cout, kd, top_h);
  else memset(top, 0, sizeof(float) * (size_t)count);
  free(col);
  return count;
}

/* ---- general convolution / deconvolution (all strides, dense or non-empty) ------------------ */
/* col2octree_cpu, octree/octree/octree_nn.cpp:216-241 (single chunk): the transpose of octree2col,
 * data[c*octree_h + p] += col[(c*K + k)*H + h], visited in (c, k, h) order. */
void oc_col2octree(const float *col, float *data, int channel, int height, int kdim, int stride,
                   const int32_t *neigh, const int32_t *ni) {
  const long octree_h = (long)height << (3 * (stride - 1));
  memset(data, 0, sizeof(float) * (size_t)(channel * octree_h));
  for (int c = 0; c < channel; ++c)
    for (int k = 0; k < kdim; ++k) {
      const float *row = col + ((long)c * kdim + k) * height;
      for (long h = 0; h < height; ++h) {
        long at = stride == 2 ? (h << 6) + ni[k] : ((h >> 3) << 6) + ni[(h & 7) * kdim + k];
        int p = neigh[at];
        if (p != -1) data[c * octree_h + p] += row[h];
      }
    }
}

/* octree2colP_cpu with either stride, octree/octree/octree_nn.cpp:244-271: at stride 2 the column
 * rows are the sibling groups themselves (no ichild), the gathered node still goes through child. */
void oc_octree2col_p2(float *col, const float *data, int channel, int height, int octree_h, int kdim,
                      int stride, const int32_t *neigh, const int32_t *ni, const int32_t *child,
                      const int32_t *ichild) {
  for (int c = 0; c < channel; ++c)
    for (int k = 0; k < kdim; ++k) {
      float *row = col + ((long)c * kdim + k) * height;
      for (long h = 0; h < height; ++h) {
        const long hp = ichild[h];
        const long at = stride == 2 ? (h << 6) + ni[k] : ((hp >> 3) << 6) + ni[(hp & 7) * kdim + k];
        int p = neigh[at];
        if (p >= 0) p = child[p];
        row[h] = p < 0 ? 0.0f : data[(long)c * octree_h + p];
      }
    }
}

/* col2octreeP_cpu, octree/octree/octree_nn.cpp:273-298 */
void oc_col2octree_p(const float *col, float *data, int channel, int height, int octree_h, int kdim,
                     int stride, const int32_t *neigh, const int32_t *ni, const int32_t *child,
                     const int32_t *ichild) {
  memset(data, 0, sizeof(float) * (size_t)((long)channel * octree_h));
  for (int c = 0; c < channel; ++c)
    for (int k = 0; k < kdim; ++k) {
      const float *row = col + ((long)c * kdim + k) * height;
      for (long h = 0; h < height; ++h) {
        const long hp = ichild[h];
        const long at = stride == 2 ? (h << 6) + ni[k] : ((hp >> 3) << 6) + ni[(hp & 7) * kdim + k];
        int p = neigh[at];
        if (p >= 0) p = child[p];
        if (p >= 0) data[(long)c * octree_h + p] += row[h];
      }
    }
}

/* OctreeConv / OctreeDeconv forward for every combination of stride (1, 2), nempty and
 * transposition: OctreeBaseConv::setup / reshape (octree/octree/octree_conv.cpp:10-122) followed
 * by forward_cpu_gemm (:158-180) for the convolution or backward_cpu_gemm (:182-206) for the
 * deconvolution (pytorch/cpp/octree_conv.cpp:191-217 runs the deconvolution's forward through
 * backward_gpu_gemm).  channel_in = channels of `bottom`, num_output = channels of `top`;
 * weights: [conv_out, conv_in*K] with (conv_in, conv_out) = (channel_in, num_output) for the
 * convolution and swapped for the deconvolution.  Bottom height: nnum[depth], or nnum_nempty[depth]
 * when nempty or for a stride-2 deconvolution.  Returns num_output * top_h; call with top == NULL
 * to size the output. */
long oc_octree_conv_general(float *top, long cap, const float *bottom, const float *weights,
                            const uint8_t *octree, int depth, int channel_in, int num_output,
                            const int ks[3], int stride, int nempty, int deconv) {
  int taps[27];
  const int K = kernel_taps(ks, taps);
  if (K < 0 || stride < 1 || stride > 2) return -1;
  const int32_t *nnum = hci(octree, H_NNUM), *nne = hci(octree, H_NNUM_NE);
  const int odepth = *hci(octree, H_DEPTH);
  int top_depth = depth, work_depth = depth;
  if (stride == 2) {
    if (deconv) top_depth = work_depth = depth + 1; else top_depth = depth - 1;
    if (top_depth < 0 || top_depth > odepth) return -1;
  }
  const int conv_in = deconv ? num_output : channel_in, conv_out = deconv ? channel_in : num_output;
  const long kd = (long)K * conv_in;
  long top_h = nempty ? nne[top_depth] : nnum[top_depth];
  if (!nempty && stride == 2 && !deconv) top_h = nne[top_depth];
  if (top_h == 0) top_h = 1;
  long work_h = top_h;
  if (stride == 2) work_h = deconv ? nnum[top_depth] / 8 : nnum[depth] / 8;
  const long count = (long)num_output * top_h;
  if (top == NULL || cap < count) return count;
  const int one = ks[0] == 1 && ks[1] == 1 && ks[2] == 1 && stride == 1;
  int ni[216];
  oc_ni_table(ks, ni);
  const int32_t *neigh = one ? NULL : (const int32_t *)(octree + prop_offset(octree, P_NEIGH, work_depth));
  const int32_t *child = NULL;
  int32_t *ichild = NULL;
  long octree_h = 0;
  if (nempty) {
    child = (const int32_t *)(octree + prop_offset(octree, P_CHILD, work_depth));
    const long ich = nne[work_depth] > 0 ? nne[work_depth] : 1;
    /* at stride 2 the column rows outnumber nothing: ichild is read for h < work_h only at
     * stride 1, but the reference indexes it unconditionally, so size it for both */
    ichild = (int32_t *)calloc((size_t)(ich > work_h ? ich : work_h), sizeof(int32_t));
    oc_ichild(ichild, child, nnum[work_depth]);
    octree_h = (stride == 2 && deconv) ? nne[top_depth] : nne[depth];
  }
  float *col = one ? NULL : (float *)calloc((size_t)(kd * (work_h > 0 ? work_h : 1)), sizeof(float));
  if (!deconv) {
    const float *src = bottom;
    if (!one) {
      if (nempty)
        oc_octree2col_p2(col, bottom, conv_in, (int)work_h, (int)octree_h, K, stride, neigh, ni, child, ichild);
      else
        oc_octree2col(col, bottom, conv_in, (int)work_h, K, stride, neigh, ni);
      src = col;
    }
    gemm_rows(top, weights, src, conv_out, kd, work_h);
  } else {
    float *dst = one ? top : col;
    for (long m = 0; m < kd; ++m)
      for (long h = 0; h < work_h; ++h) {
        float acc = 0.0f;
        for (int k = 0; k < conv_out; ++k) acc += weights[k * kd + m] * bottom[k * work_h + h];
        dst[m * work_h + h] = acc;
      }
    if (!one) {
      if (nempty)
        oc_col2octree_p(col, top, conv_in, (int)work_h, (int)octree_h, K, stride, neigh, ni, child, ichild);
      else
        oc_col2octree(col, top, conv_in, (int)work_h, K, stride, neigh, ni);
    }
  }
  free(col);
  free(ichild);
  return count;
}

/* ---- keys ------------------------------------------------------------------------------------- */
/* xyz2key_cpu / key2xyz_cpu / search_key_cpu, octree/octree/octree_nn.cpp:540-620, for 64-bit keys
 * (four 16-bit lanes x, y, z, id) or 32-bit keys (four bytes).  Only `depth` bits of each
 * coordinate enter the key (compute_key, :551-560). */
void oc_xyz2key(uint64_t *key, const uint64_t *xyz, long num, int depth, int key_bits) {
  const int B = key_bits == 64 ? 16 : 8;
  const uint64_t lane = (1ull << B) - 1, low3 = (1ull << (3 * B)) - 1;
  for (long i = 0; i < num; ++i) {
    const uint64_t v = xyz[i], pt[3] = {v & lane, (v >> B) & lane, (v >> (2 * B)) & lane};
    uint64_t k = 0;
    for (int b = 0; b < depth; ++b)
      for (int j = 0; j < 3; ++j) k |= (pt[j] & (1ull << b)) << (2 * b + 2 - j);
    key[i] = (k & low3) | (v & ~low3);
  }
}

void oc_key2xyz(uint64_t *xyz, const uint64_t *key, long num, int depth, int key_bits) {
  const int B = key_bits == 64 ? 16 : 8;
  const uint64_t lane = (1ull << B) - 1, low3 = (1ull << (3 * B)) - 1;
  for (long i = 0; i < num; ++i) {
    uint64_t pt[3] = {0, 0, 0};
    for (int b = 0; b < depth; ++b)
      for (int j = 0; j < 3; ++j) pt[j] |= (key[i] & (1ull << (3 * b + 2 - j))) >> (2 * b + 2 - j);
    xyz[i] = (pt[0] & lane) | ((pt[1] & lane) << B) | ((pt[2] & lane) << (2 * B)) | (key[i] & ~low3);
  }
}

void oc_search_key(int32_t *idx, const uint64_t *key, long n_key, const uint64_t *query, long n_query) {
  for (long i = 0; i < n_query; ++i) {
    long lo = 0, hi = n_key;
    while (lo < hi) { long mid = (lo + hi) / 2; if (key[mid] < query[i]) lo = mid + 1; else hi = mid; }
    idx[i] = (lo >= n_key || key[lo] != query[i]) ? -1 : (int32_t)lo;
  }
}

/* ---- pool / pad ------------------------------------------------------------------------- */
/* octree_max_pool_cpu, octree/octree/octree_nn.cpp:301-322: strict '>' so the first maximum
 * wins; mask holds the absolute bottom row. */
void oc_max_pool(float *top, int top_h, int32_t *mask, const float *btm, int btm_h, int channel) {
  for (int c = 0; c < channel; ++c)
    for (int h = 0; h < top_h; ++h) {
      const float *b = btm + (long)c * btm_h;
      int at = 8 * h;
      for (int j = 8 * h + 1; j < 8 * h + 8; ++j) if (b[j] > b[at]) at = j;
      top[(long)c * top_h + h] = b[at];
      mask[(long)c * top_h + h] = at;
    }
}

/* pad_forward_cpu, octree/octree/octree_nn.cpp:163-172 */
void oc_pad(float *y, int hy, int channel, const float *x, int hx, const int32_t *child, float val) {
  for (int c = 0; c < channel; ++c)
    for (int h = 0; h < hy; ++h)
      y[(long)c * hy + h] = child[h] == -1 ? val : x[(long)c * hx + child[h]];
}

/* pad_backward_cpu, octree/octree/octree_nn.cpp:174-185 (rows never written keep their value) */
void oc_depad(float *x, int hx, int channel, const float *y, int hy, const int32_t *child) {
  for (int c = 0; c < channel; ++c)
    for (int h = 0; h < hy; ++h)
      if (child[h] != -1) x[(long)c * hx + child[h]] = y[(long)c * hy + h];
}
