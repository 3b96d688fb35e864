"""Pins the CPU oracle (oracle/ocnn_oracle.c) on (1) the known-answer vectors held by the
reference's own tests and (2) fixtures produced by the reference's compiled CPU code
(tests/golden/reference_vectors.npz).  Runs without a GPU and without the reference checkout."""
import os

import numpy as np
import pytest

from conftest import same_bits
from oracle import oracle as oc

KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [1, 3, 1], [1, 1, 3], [3, 3, 1], [3, 1, 3], [1, 3, 3],
           [1, 1, 1]]


def kname(ks):
  return ''.join(map(str, ks))


# ---- known answers from the reference's own tests ------------------------------------------
def test_morton_known_answers():
  # caffe/src/caffe/test/test_octree_util.cpp:255-272 (xyz -> key at depth 5)
  assert oc.morton(0, 0, 0, 5) == 0
  assert oc.morton(1, 1, 1, 5) == 7
  assert oc.morton(1, 2, 3, 5) == 29


def test_build_known_answers_three_points():
  # octree/test/test_octree.cpp:92-170: 3 points, box [0,2]^3, depth 5, full layer 1,
  # node displacement on, split labels on.
  pts = [0.0, 0.0, 0.0, 1.0, 1.0, 0.0, 1.0625, 1.0625, 0.0]
  normals = [1.0, 0.0, 0.0, -1.0, 0.0, 0.0, 0.0, 1.0, 0.0]
  feats = [1.0, -1.0, 2.0, -2.0, 3.0, -3.0]
  labels = [0.0, 2.0, 2.0]
  points = oc.points_new(pts, normals, feats, labels)
  for kb in (32, 64):
    buf = oc.points2octree(points, 5, 1, node_dis=True, split_label=True, key_bits=kb,
                           bbox=[0, 0, 0, 2, 2, 2])
    v = oc.OctreeView(buf)
    assert (v.depth, v.full_depth) == (5, 1)
    assert list(v.nnum[:6]) == [1, 8, 16, 16, 16, 16]                       # :106
    assert list(v.nnum_cum[:7]) == [0, 1, 9, 25, 41, 57, 73]                # :107
    assert list(v.nnum_nempty[:6]) == [1, 2, 2, 2, 2, 3]                    # :108
    keys = [0, 0, 1, 2, 3, 4, 5, 6, 7]                                      # :117-123
    for base in (48, 384, 3072, 24576):
      keys += list(range(8)) + list(range(base, base + 8))
    got = np.concatenate([v.prop('key', d) for d in range(6)])
    assert list(got) == keys
    e = [-1] * 7
    children = [0, 0, -1, -1, -1, -1, -1, 1, -1]                            # :133-139
    for _ in range(3):
      children += [0] + e + [1] + e
    children += [0] + e + [1, -1, -1, -1, -1, -1, 2, -1]
    got = np.concatenate([v.prop('child', d) for d in range(6)])
    assert list(got) == children
    f = v.prop('feature', 5)                                                # :149-156
    assert f.shape == (6, 16)
    z16 = np.zeros(16, np.float32)
    want = np.stack([z16.copy() for _ in range(6)])
    want[0, [0, 8]] = [1.0, -1.0]
    want[1, 14] = 1.0
    want[3, [0, 8, 14]] = [-0.57735, 0.57735, -0.57735]
    want[4, [0, 8, 14]] = [1.0, 2.0, 3.0]
    want[5, [0, 8, 14]] = [-1.0, -2.0, -3.0]
    assert np.array_equal(f[[0, 1, 2, 4, 5]], want[[0, 1, 2, 4, 5]])
    # the test writes the displacement as the literal -0.57735f and compares with EXPECT_EQ on
    # values computed as (+-0.5) * 1.1547f, which is that literal in fp32
    assert np.array_equal(f[3], np.float32(want[3]))
    lab = v.prop('label', 5)                                                # :163-166
    assert list(lab) == [0.0] + [-1.0] * 7 + [2.0] + [-1.0] * 5 + [2.0, -1.0]
    split = np.concatenate([v.prop('split', d) for d in range(6)])          # :172-178
    assert list(split) == [1.0 if c >= 0 else 0.0 for c in children]


def octree2col_bruteforce(data, ks, stride, taps):
  """Direct neighbour walk on one fully occupied 2x2x2 level (the closed-form check of
  pytorch/test/test_octree2col.py:23-50, restated)."""
  channel = data.shape[0]
  kdim = int(np.prod(ks))
  top_h = 8 if stride == 1 else 1
  col = np.zeros((channel, kdim, top_h), np.float32)
  for h in range(top_h):
    hx, hy, hz = h >> 2, (h >> 1) & 1, h & 1
    for k, tap in enumerate(taps):
      x, y, z = hx + tap // 9 - 1, hy + (tap // 3) % 3 - 1, hz + tap % 3 - 1
      if 0 <= x < 2 and 0 <= y < 2 and 0 <= z < 2:
        col[:, k, h] = data[:, 4 * x + 2 * y + z]
  return col


TAPS = {'333': list(range(27)), '111': [13], '222': [13, 14, 16, 17, 22, 23, 25, 26],
        '311': [4, 13, 22], '131': [10, 13, 16], '113': [12, 13, 14],
        '331': [1, 4, 7, 10, 13, 16, 19, 22, 25], '313': [3, 4, 5, 12, 13, 14, 21, 22, 23],
        '133': [9, 10, 11, 12, 13, 14, 15, 16, 17]}


@pytest.mark.parametrize('ks', KERNELS)
@pytest.mark.parametrize('stride', [1, 2])
def test_octree2col_known_answer_depth1(golden, ks, stride):
  # pytorch/test/test_octree2col.py:52-67 on octree_1, depth 1
  merged = oc.octree_batch([golden['k32_octree_1']])
  v = oc.OctreeView(merged)
  rng = np.random.default_rng(5)
  data = rng.uniform(-1, 1, size=(3, 8)).astype(np.float32)
  got = oc.octree2col(data, v.prop('neigh', 1), ks, stride, 8 if stride == 1 else 1)
  assert np.array_equal(got, octree2col_bruteforce(data, ks, stride, TAPS[kname(ks)]))


def test_pool_known_answer():
  # pytorch/test/test_octree_pool.py:10-39 (forward part): data, pooled values and mask
  row0 = [1.1, 2.2, 3.3, 4.4, 5.5, 6.6, 7.7, 8.8]
  row1 = [8.1, 7.2, 6.3, 5.4, 4.5, 3.6, 2.7, 1.8]
  data = np.array([row0 + row0, row1 + row1], np.float32)
  top, mask = oc.max_pool(data)
  assert np.array_equal(mask, np.array([[7, 15], [0, 8]], np.int32))
  assert np.array_equal(top, np.array([[8.8, 8.8], [8.1, 8.1]], np.float32))
  # OctreeMaxPool pads the pooled rows to the parent level (octree_pool.py:84-87)
  merged = oc.octree_batch([_g('k32_octree_1')] * 2)
  child4 = oc.OctreeView(merged).prop('child', 4)
  padded = oc.pad(top, child4, 0.0)
  want = np.zeros((2, 16), np.float32)
  want[:, 0], want[:, 8] = [8.8, 8.1], [8.8, 8.1]
  assert np.array_equal(padded, want)


_GOLD = {}


def _g(name):
  if not _GOLD:
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden',
                        'reference_vectors.npz')
    _GOLD.update(np.load(path))
  return _GOLD[name]


def test_property_known_answers(golden):
  # pytorch/test/test_octree_property.py:10-55 on a batch of two octree_1 (64-bit keys, as the
  # PyTorch binding is built)
  merged = oc.octree_batch([golden['k64_octree_1']] * 2)
  v = oc.OctreeView(merged)
  assert list(v.nnum[:6]) == [2, 16, 128, 16, 16, 16]
  assert list(v.nnum_cum[:7]) == [0, 2, 18, 146, 162, 178, 194]
  assert (v.batch_size, v.depth, v.full_depth) == (2, 5, 2)
  child = v.prop('child', 5)
  want = -np.ones(16, np.int32)
  want[0], want[8] = 0, 1
  assert np.array_equal(child, want)
  f = v.prop('feature', 5)
  wantf = np.zeros((3, 16), np.float32)
  wantf[:, [0, 8]] = 3.0 ** 0.5 / 3.0
  assert np.allclose(f, wantf)
  # batch index lives in the top 16-bit lane of the key ('index' property)
  assert list(v.prop('key', 5) >> np.uint64(48)) == [0] * 8 + [1] * 8
  # the embedded samples store packed (x, y, z, batch) uint16 lanes instead of Morton keys
  # (key2xyz = true); finest nodes of octree_1: pytorch/test/test_octree_key.py:14-18
  assert merged[44] == 1
  key = v.prop('key', 5)
  lanes = np.stack([(key >> np.uint64(16 * i)) & np.uint64(0xffff) for i in range(4)], 1)
  want_xyz = [[x, y, z] for x in (16, 17) for y in (16, 17) for z in (16, 17)]
  assert lanes[:8, :3].tolist() == want_xyz and lanes[8:, :3].tolist() == want_xyz
  # their Morton keys, as searched for in test_octree_key.py:33-41 (28673 -> node 1,
  # (1 << 48) | 28679 -> node 15)
  mort = [oc.morton(x, y, z, 5) for x, y, z in want_xyz]
  assert mort == list(range(28672, 28680))
  assert mort[1] == 28673 and (1 << 48) | mort[7] == 281474976739335


def test_conv_equals_octree2col_times_weights(golden):
  # pytorch/test/test_octree_conv.py:10-82: OctreeConv == octree2col + mm on octree_1 + octree_2,
  # depth 4, 3 -> 5 channels, every kernel shape and stride
  merged = oc.octree_batch([golden['k32_octree_1'], golden['k32_octree_2']])
  v = oc.OctreeView(merged)
  depth, cin, cout = 4, 3, 5
  H = int(v.nnum[depth])
  assert H == 152
  rng = np.random.default_rng(9)
  data = rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)
  for ks in [[3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]]:
    for stride in (1, 2):
      kd = int(np.prod(ks))
      w = rng.normal(size=(cout, cin * kd)).astype(np.float32)
      out = oc.octree_conv(data, w, merged, depth, cout, ks, stride)
      hc = H if stride == 1 else H // 8
      col = oc.octree2col(data, v.prop('neigh', depth), ks, stride, hc).reshape(cin * kd, hc)
      assert out.shape == (cout, hc)
      assert np.allclose(out, w @ col, rtol=1e-5, atol=1e-5)


# ---- fixtures produced by the reference's CPU code ----------------------------------------
@pytest.mark.parametrize('kb', [32, 64])
def test_build_matches_reference_fixture(golden, kb):
  tag = 'k%d_' % kb
  pts = oc.points_new(golden['a_xyz'], golden['a_normal'], golden['a_feat'], golden['a_label'])
  assert same_bits(pts, golden['a_points'])
  assert same_bits(oc.points2octree(pts, 5, 2, key_bits=kb), golden[tag + 'a_octree'])
  assert same_bits(oc.points2octree(pts, 5, 2, node_dis=True, split_label=True, save_pts=True,
                                    key_bits=kb), golden[tag + 'a_octree_flags'])
  pts_nn = oc.points_new(golden['a_xyz'], None, golden['a_feat'])
  assert same_bits(oc.points2octree(pts_nn, 4, 1, node_dis=True, key_bits=kb),
                   golden[tag + 'a_octree_nonormal'])


@pytest.mark.parametrize('kb', [32, 64])
def test_merge_matches_reference_fixture(golden, kb):
  tag = 'k%d_' % kb
  singles = []
  for i in range(3):
    pts = oc.points_new(golden['b%d_xyz' % i], golden['b%d_normal' % i])
    singles.append(oc.points2octree(pts, 4, 2, key_bits=kb))
    assert same_bits(singles[-1], golden[tag + 'b%d_octree' % i])
  assert same_bits(oc.octree_batch(singles), golden[tag + 'b_merged'])
  assert same_bits(oc.octree_batch([golden[tag + 'octree_1'], golden[tag + 'octree_2']]),
                   golden[tag + 'merge_samples_12'])
  assert same_bits(oc.octree_batch([golden[tag + 'octree_1']] * 2),
                   golden[tag + 'merge_samples_11'])


def test_tables_match_reference_fixture(golden):
  for ks in KERNELS:
    assert np.array_equal(oc.ni_table(ks), golden['tbl_ni' + kname(ks)])
  for d in (1, 2, 3):
    assert np.array_equal(oc.calc_neigh_full(d, 2), golden['neigh_full_d%d_b2' % d])
  # the parent / displacement tables are implicit in calc_neigh_split; check them through it
  v = oc.OctreeView(golden['k32_b_merged'])
  for d in (3, 4):
    got = oc.calc_neigh_split(v.prop('neigh', d - 1), v.prop('child', d - 1), int(v.nnum[d]))
    assert np.array_equal(got.reshape(-1, 64), v.prop('neigh', d))


def test_ops_match_reference_fixture(golden):
  merged = golden['k32_b_merged']
  v = oc.OctreeView(merged)
  d = 4
  x, xne = golden['b_x'], golden['b_xne']
  H = int(v.nnum[d])
  for ks in KERNELS:
    for stride in (1, 2):
      got = oc.octree_conv(x, golden['b_w' + kname(ks)], merged, d, 5, ks, stride)
      assert same_bits(got, golden['b_conv%s_s%d' % (kname(ks), stride)]), (ks, stride)
  assert same_bits(oc.octree2col(x, v.prop('neigh', d), [3, 1, 1], 1, H), golden['b_col311_s1'])
  assert same_bits(oc.octree2col(x, v.prop('neigh', d), [2, 2, 2], 2, H // 8),
                   golden['b_col222_s2'])
  top, mask = oc.max_pool(x)
  assert same_bits(top, golden['b_pool']) and same_bits(mask, golden['b_pool_mask'])
  child = v.prop('child', d)
  assert same_bits(oc.pad(xne, child, 0.25), golden['b_pad'])
  assert same_bits(oc.depad(x, child, xne.shape[1]), golden['b_depad'])


# ---- convolution / deconvolution for every stride / nempty combination ----------------------
GENERAL_KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]]


@pytest.fixture(scope='module')
def golden_general():
  import os
  path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden',
                      'reference_vectors_general.npz')
  return dict(np.load(path))


@pytest.mark.parametrize('ks', GENERAL_KERNELS)
def test_conv_general_matches_reference_fixture(golden, golden_general, ks):
  """Outputs of the reference's OctreeBaseConv (forward_cpu_gemm / backward_cpu_gemm with
  octree2col(P) / col2octree(P)) on the merged batch of the first fixture file, depth 3."""
  g = golden_general
  merged = golden['k32_b_merged']
  name = kname(ks)
  for stride in (1, 2):
    for nempty in (0, 1):
      for deconv in (0, 1):
        x = g['g_x_ne'] if (nempty or (deconv and stride == 2)) else g['g_x_full']
        w = g['g_wd' + name] if deconv else g['g_wc' + name]
        got = oc.octree_conv_general(x, w, merged, 3, 5, ks, stride, bool(nempty), bool(deconv))
        assert same_bits(got, g['g_y%s_s%d_n%d_t%d' % (name, stride, nempty, deconv)]), \
            (ks, stride, nempty, deconv)


def test_octree_samples_api(golden):
  """`ocnn.octree_samples` hands out the reference's embedded test octrees in the current key
  width (pytorch/cpp/octree_samples.cpp:5-22)."""
  import ocnn
  for kb in (64, 32):
    ocnn.set_key_bits(kb)
    try:
      got = ocnn.octree_samples(['octree_1', 'octree_2'])
      for t, name in zip(got, ('octree_1', 'octree_2')):
        assert same_bits(t.numpy(), golden['k%d_%s' % (kb, name)])
      assert len(ocnn.nn.octree_samples(['octree_%d' % i for i in range(1, 7)])) == 6
    finally:
      ocnn.set_key_bits(64)
  with pytest.raises(ValueError):
    ocnn.octree_samples(['octree_7'])


@pytest.mark.parametrize('kb', [32, 64])
def test_octree_new_grow_update_match_reference_fixture(kb):
  """octree_new / octree_grow / octree_update against outputs of the compiled reference
  (tests/golden/reference_vectors_grow.npz, made by make_golden.py grow)."""
  g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden',
                           'reference_vectors_grow.npz'))
  cur = oc.octree_new(2, 4, True, 0, kb)
  assert np.array_equal(cur, g['k%d_new' % kb])
  for d in range(1, 5):
    cur = oc.octree_grow(cur, d, d <= 2)
    assert np.array_equal(cur, g['k%d_grow%d' % (kb, d)]), d
    if d >= 2:
      cur = oc.octree_update(cur, g['k%d_label%d' % (kb, d)], d, 1)
      assert np.array_equal(cur, g['k%d_update%d' % (kb, d)]), d
