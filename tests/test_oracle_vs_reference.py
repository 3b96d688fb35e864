"""Differential test: the C oracle against the reference's own CPU code compiled unmodified
(oracle/_ref, built by `make -C oracle ref` where the reference checkout exists).  Bit-exact on
every output.  Skipped where the compiled reference is absent; the committed fixtures
(test_oracle_golden.py) pin the oracle there."""
import numpy as np
import pytest

from conftest import same_bits
from oracle import oracle as oc
from oracle import ref
from ocnn_harness import synth

pytestmark = pytest.mark.skipif(not (ref.available(32) and ref.available(64)),
                                reason='compiled reference (oracle/_ref) not present')

KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [1, 3, 1], [1, 1, 3], [3, 3, 1], [3, 1, 3], [1, 3, 3],
           [1, 1, 1]]


@pytest.fixture(scope='module', params=[32, 64])
def batch(request):
  kb = request.param
  R = ref.get(kb)
  rng = np.random.default_rng(3 + kb)
  singles_r, singles_o = [], []
  for i in range(3):
    p, q = synth.primitive_union(4000 + 500 * i, 70 + i)
    f = rng.normal(size=(p.shape[0], 2)).astype(np.float32)
    pr, po = R.points_new(p, q, f), oc.points_new(p, q, f)
    assert same_bits(pr, po)
    singles_r.append(R.points2octree(pr, 6, 2))
    singles_o.append(oc.points2octree(po, 6, 2, key_bits=kb))
    assert same_bits(singles_r[-1], singles_o[-1])
  return kb, R, R.octree_batch(singles_r), oc.octree_batch(singles_o)


@pytest.mark.parametrize('kb', [32, 64])
@pytest.mark.parametrize('flags', [(0, 0, 0), (1, 1, 0), (1, 0, 1), (0, 1, 1)])
def test_build_flags(kb, flags):
  R = ref.get(kb)
  nd, sl, sp = flags
  rng = np.random.default_rng(17)
  p, q = synth.primitive_union(6000, 5, jitter_frac=0.05, jitter_sigma=0.005)
  f = rng.normal(size=(p.shape[0], 3)).astype(np.float32)
  lab = rng.integers(-1, 6, size=p.shape[0]).astype(np.float32)
  for normals in (q, None):
    pts = oc.points_new(p, normals, f, lab)
    for depth, full in ((7, 2), (4, 3), (3, 3), (5, 1)):
      a = R.points2octree(pts, depth, full, node_dis=nd, split_label=sl, save_pts=sp)
      b = oc.points2octree(pts, depth, full, node_dis=nd, split_label=sl, save_pts=sp,
                           key_bits=kb)
      assert same_bits(a, b), (depth, full, normals is None)


def test_build_deep_64bit():
  R = ref.get(64)
  p, q, c = synth.indoor_scene(20000, 5000)
  pts = oc.points_new(p, q, c)
  assert same_bits(R.points2octree(pts, 9, 2), oc.points2octree(pts, 9, 2, key_bits=64))
  assert same_bits(R.points2octree(pts, 12, 3, node_dis=True),
                   oc.points2octree(pts, 12, 3, node_dis=True, key_bits=64))


def test_degenerate_clouds():
  for kb in (32, 64):
    R = ref.get(kb)
    one = oc.points_new([0.3, -0.2, 0.1], [0.0, 0.0, 1.0])
    assert same_bits(R.points2octree(one, 5, 2), oc.points2octree(one, 5, 2, key_bits=kb))
    # all points in one cell, cancelling normals (falls back to the first point's normal)
    p = np.tile(np.array([[0.5, 0.5, 0.5]], np.float32), (4, 1))
    q = np.array([[1, 0, 0], [-1, 0, 0], [0, 1, 0], [0, -1, 0]], np.float32)
    same = oc.points_new(p, q)
    assert same_bits(R.points2octree(same, 6, 2), oc.points2octree(same, 6, 2, key_bits=kb))
    single = R.points2octree(one, 5, 2)
    assert same_bits(R.octree_batch([single]), oc.octree_batch([single]))


def test_merge(batch):
  kb, R, merged_r, merged_o = batch
  assert same_bits(merged_r, merged_o)
  info = R.octree_info(merged_o)
  v = oc.OctreeView(merged_o)
  assert info['key_bits'] == kb and info['sizeof_octree'] == merged_o.size == v.sizeof_octree
  assert np.array_equal(info['nnum'], v.nnum) and np.array_equal(info['nnum_cum'], v.nnum_cum)
  assert np.array_equal(info['nnum_nempty'], v.nnum_nempty)
  for i, p in enumerate(oc.PROPS):
    assert info['channel'][p] == v.channels[i]
    if v.channels[i]:
      assert info['ptr_dis'][p] == v.ptr_dis[i] and info['location'][p] == v.locations[i]


def test_neighbour_tables(batch):
  kb, R, merged_r, _ = batch
  v = oc.OctreeView(merged_r)
  for d in (1, 2, 3):
    assert np.array_equal(R.calc_neigh_full(d, 3), oc.calc_neigh_full(d, 3))
  for d in range(3, 7):
    a = R.calc_neigh_split(v.prop('neigh', d - 1), v.prop('child', d - 1), int(v.nnum[d]))
    b = oc.calc_neigh_split(v.prop('neigh', d - 1), v.prop('child', d - 1), int(v.nnum[d]))
    assert np.array_equal(a, b)
  for ks in KERNELS:
    assert np.array_equal(R.ni_table(ks), oc.ni_table(ks))


@pytest.mark.parametrize('ks', KERNELS)
@pytest.mark.parametrize('stride', [1, 2])
def test_conv_and_octree2col(batch, ks, stride):
  kb, R, merged_r, merged_o = batch
  v = oc.OctreeView(merged_o)
  rng = np.random.default_rng(sum(ks) * 10 + stride)
  for d in (6, 4):
    H = int(v.nnum[d])
    cin, cout = 3, 5
    x = rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)
    w = rng.normal(size=(cout, cin * int(np.prod(ks)))).astype(np.float32)
    assert same_bits(R.octree_conv(x, w, merged_r, d, cout, ks, stride),
                     oc.octree_conv(x, w, merged_o, d, cout, ks, stride))
    hc = H if stride == 1 else H // 8
    assert same_bits(R.octree2col(x, v.prop('neigh', d), ks, stride, hc),
                     oc.octree2col(x, v.prop('neigh', d), ks, stride, hc))


@pytest.mark.parametrize('ks', [[3, 3, 3], [3, 1, 1], [2, 2, 2], [1, 1, 1]])
def test_octree2col_nempty(batch, ks):
  """octree2colP (the convolution restricted to non-empty nodes): the restatement against the
  reference's octree2colP_cpu, and the convolution built on it against the identity the
  reference's own test uses (pytorch/test/test_octree_conv.py: OctreeConv(nempty=True) equals the
  dense convolution of the zero-padded data, read back at the non-empty nodes)."""
  kb, R, _, merged_o = batch
  v = oc.OctreeView(merged_o)
  rng = np.random.default_rng(21)
  for d in (6, 4):
    nne = int(v.nnum_nempty[d])
    child, neigh = v.prop('child', d), v.prop('neigh', d)
    x = rng.uniform(-1, 1, size=(3, nne)).astype(np.float32)
    assert same_bits(R.octree2col_p(x, neigh, child, ks), oc.octree2col_p(x, neigh, child, ks))
    w = rng.normal(size=(5, 3 * int(np.prod(ks)))).astype(np.float32)
    got = oc.octree_conv_nempty(x, w, merged_o, d, 5, ks)
    dense = oc.octree_conv(oc.pad(x, child, 0.0), w, merged_o, d, 5, ks, 1)
    assert same_bits(got, oc.depad(dense, child, nne))


def test_pool_pad_depad(batch):
  kb, R, _, merged_o = batch
  v = oc.OctreeView(merged_o)
  rng = np.random.default_rng(8)
  for d in (6, 5, 3):
    H, Hne = int(v.nnum[d]), int(v.nnum_nempty[d])
    x = rng.uniform(-1, 1, size=(4, H)).astype(np.float32)
    x[0, :16] = 1.0            # ties: the first maximum must win
    x[1, 8:16] = np.nan        # NaN never wins a '>' comparison
    a, b = R.max_pool(x), oc.max_pool(x)
    assert same_bits(a[0], b[0]) and same_bits(a[1], b[1])
    child = v.prop('child', d)
    xs = rng.uniform(-1, 1, size=(4, Hne)).astype(np.float32)
    assert same_bits(R.pad_forward(xs, child, 0.5), oc.pad(xs, child, 0.5))
    assert same_bits(R.pad_backward(x, child, Hne), oc.depad(x, child, Hne))


GENERAL_KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]]   # pytorch/test/test_octree_deconv.py


def _bottom_height(v, d, stride, nempty, deconv):
  return int(v.nnum_nempty[d]) if (nempty or (deconv and stride == 2)) else int(v.nnum[d])


@pytest.mark.parametrize('ks', GENERAL_KERNELS)
@pytest.mark.parametrize('stride', [1, 2])
@pytest.mark.parametrize('nempty', [False, True])
@pytest.mark.parametrize('deconv', [False, True])
def test_conv_general(batch, ks, stride, nempty, deconv):
  """OctreeConv / OctreeDeconv forward for every stride / nempty combination: the restatement
  against the reference's setup + reshape + forward_cpu_gemm / backward_cpu_gemm, bit for bit."""
  kb, R, merged_r, merged_o = batch
  v = oc.OctreeView(merged_o)
  rng = np.random.default_rng(sum(ks) * 100 + stride * 10 + nempty * 2 + deconv)
  cin, cout = 3, 5
  kd = int(np.prod(ks))
  for d in (5, 4):
    x = rng.uniform(-1, 1, size=(cin, _bottom_height(v, d, stride, nempty, deconv))).astype(np.float32)
    wshape = (cin, cout * kd) if deconv else (cout, cin * kd)
    w = rng.normal(size=wshape).astype(np.float32)
    a = R.octree_conv_general(x, w, merged_r, d, cout, ks, stride, nempty, deconv)
    b = oc.octree_conv_general(x, w, merged_o, d, cout, ks, stride, nempty, deconv)
    assert a.shape == b.shape and same_bits(a, b), (d, a.shape)
    if not nempty and not deconv:
      assert same_bits(b, oc.octree_conv(x, w, merged_o, d, cout, ks, stride))


@pytest.mark.parametrize('ks', GENERAL_KERNELS)
@pytest.mark.parametrize('stride', [1, 2])
def test_col2octree_and_octree2colP(batch, ks, stride):
  kb, R, _, merged_o = batch
  v = oc.OctreeView(merged_o)
  rng = np.random.default_rng(5 + sum(ks) + stride)
  d = 5
  H, nne = int(v.nnum[d]), int(v.nnum_nempty[d])
  neigh, child = v.prop('neigh', d), v.prop('child', d)
  kd = int(np.prod(ks))
  hc = H if stride == 1 else H // 8
  col = rng.uniform(-1, 1, size=(3, kd, hc)).astype(np.float32)
  assert same_bits(R.col2octree_general(col, neigh, ks, stride, H),
                   oc.col2octree_general(col, neigh, ks, stride, H))
  hcp = nne if stride == 1 else H // 8
  colp = rng.uniform(-1, 1, size=(3, kd, hcp)).astype(np.float32)
  assert same_bits(R.col2octree_general(colp, neigh, ks, stride, nne, child),
                   oc.col2octree_general(colp, neigh, ks, stride, nne, child))
  x = rng.uniform(-1, 1, size=(3, nne)).astype(np.float32)
  assert same_bits(R.octree2col_general(x, neigh, ks, stride, hcp, child),
                   oc.octree2col_general(x, neigh, ks, stride, hcp, child))


def test_deconv_identities(batch):
  """The identities of the reference's own test (pytorch/test/test_octree_deconv.py:44-57):
  OctreeDeconv(nempty=True) on the non-empty rows equals the dense deconvolution of the masked
  data read back at the non-empty nodes of the output level."""
  kb, R, _, merged_o = batch
  v = oc.OctreeView(merged_o)
  rng = np.random.default_rng(77)
  d, cin, cout = 4, 3, 5
  H, nne = int(v.nnum[d]), int(v.nnum_nempty[d])
  child = v.prop('child', d)
  for ks in GENERAL_KERNELS:
    kd = int(np.prod(ks))
    w = rng.normal(size=(cin, cout * kd)).astype(np.float32)
    x = rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)
    xne = oc.depad(x, child, nne)
    for stride in (1, 2):
      d_out = d if stride == 1 else d + 1
      child_out = v.prop('child', d_out)
      nne_out = int(v.nnum_nempty[d_out])
      got = oc.octree_conv_general(xne, w, merged_o, d, cout, ks, stride, True, True)
      masked = oc.pad(xne, child, 0.0)
      dense_in = masked if stride == 1 else xne      # OctreeDeconv depads before a stride-2 call
      dense = oc.octree_conv_general(dense_in, w, merged_o, d, cout, ks, stride, False, True)
      want = oc.depad(dense, child_out, nne_out)
      assert np.allclose(got, want, atol=1e-6), (ks, stride)


def test_keys_and_search(batch):
  """xyz2key / key2xyz / search_key against the reference's CPU functions, and the known answers
  of pytorch/test/test_octree_key.py:43-52 (round trip of coordinates wider than 32 key bits)."""
  kb, R, merged_r, merged_o = batch
  v = oc.OctreeView(merged_o)
  rng = np.random.default_rng(4)
  depth = 6
  keys = v.prop('key', depth)
  lane = 16 if kb == 64 else 8
  xyz = R.key2xyz(keys, depth)
  assert np.array_equal(xyz.astype(np.uint64), oc.key2xyz(keys, depth, kb))
  assert np.array_equal(R.xyz2key(xyz, depth).astype(np.uint64), oc.xyz2key(xyz, depth, kb))
  assert np.array_equal(oc.xyz2key(oc.key2xyz(keys, depth, kb), depth, kb), keys.astype(np.uint64))
  # coordinates outside [0, 2^depth) wrap: only `depth` bits of each lane are used
  wild = rng.integers(0, 1 << (4 * lane - 1), size=200).astype(np.uint64)
  assert np.array_equal(R.xyz2key(wild, depth).astype(np.uint64), oc.xyz2key(wild, depth, kb))
  query = np.concatenate([keys[::7], keys[:5] + 1, rng.integers(0, 1 << 20, size=50).astype(keys.dtype)])
  assert np.array_equal(R.search_key(keys, query), oc.search_key(keys, query))
  if kb == 64:
    xyz64 = np.array([[2049, 4095, 8011, 1], [511, 4095, 8011, 0]], np.uint64)
    word = xyz64[:, 0] | (xyz64[:, 1] << 16) | (xyz64[:, 2] << 32) | (xyz64[:, 3] << 48)
    assert np.array_equal(oc.key2xyz(oc.xyz2key(word, 13), 13), word)
    assert np.array_equal(R.xyz2key(word, 13), oc.xyz2key(word, 13))


def test_point_preparation():
  """transform_points / clip_points / bounding_box: the numpy restatement against the reference's
  Points methods, bit for bit."""
  R = ref.get(64)
  rng = np.random.default_rng(12)
  p, q = synth.primitive_union(3000, 31)
  f = rng.normal(size=(3000, 2)).astype(np.float32)
  lab = rng.integers(0, 5, size=3000).astype(np.float32)
  for normals in (q, None):
    pts = oc.points_new(p, normals, f, lab)
    cases = [([0.3, -0.2, 1.1], [1.0, 1.0, 1.0], [0.0, 0.0, 0.0], 0.0, ''),
             ([0.0, 0.0, 0.0], [0.8, 0.8, 0.8], [0.01, -0.02, 0.03], 0.02, 'x'),
             ([0.5, 0.25, -0.75], [0.9, 1.1, 0.7], [0.05, 0.0, 0.0], 0.0, 'xyz'),
             ([0.0, 0.0, 0.2], [1.0, 2.0, 1.0], [0.0, 0.0, 0.0], 0.001, 'z')]
    for angle, scale, jitter, offset, axis in cases:
      a = R.transform_points(pts, angle, scale, jitter, offset, axis)
      b = oc.transform_points(pts, angle, scale, jitter, offset, axis)
      assert same_bits(a, b), (angle, scale, jitter, offset, axis, normals is None)
    for lo, hi in (([-1, -1, -1], [1, 1, 1]), ([-0.3, -0.5, -0.2], [0.4, 0.6, 0.9]), ([2, 2, 2], [3, 3, 3])):
      a, ma = R.clip_points(pts, lo, hi)
      b, mb = oc.clip_points(pts, lo, hi)
      assert np.array_equal(ma, mb)
      kept = int(b[16:20].view(np.int32)[0])
      assert int(a[16:20].view(np.int32)[0]) == kept == max(1, int(mb.sum()))
      (xa, na, fa, la), _ = oc._points_blocks(a)
      (xb, nb, fb, lb), _ = oc._points_blocks(b)
      for u, v in ((xa, xb), (na, nb), (fa, fb), (la, lb)):
        assert (u is None) == (v is None)
        if u is not None:
          assert same_bits(u[:kept], v[:kept])
  assert same_bits(R.bounding_box(p), oc.bounding_box(p))


@pytest.mark.parametrize('kb', [32, 64])
@pytest.mark.parametrize('setup', [(1, 3, False, 0), (2, 4, True, 0), (3, 0, False, 4)])
def test_octree_new_grow_update(kb, setup):
  """The generative path's octree editing (pytorch/cpp/octree_grow.cpp): octree_new, full and
  label-driven octree_grow, octree_update incl. the degenerate all-empty case."""
  R = ref.get(kb)
  batch, channel, node_dis, adp = setup
  cur = R.octree_new(batch, channel, node_dis, adp)
  assert same_bits(cur, oc.octree_new(batch, channel, node_dis, adp, kb))
  rng = np.random.default_rng(batch)
  for d in range(1, 6):
    full = d <= 2
    grown = R.octree_grow(cur, d, full)
    assert same_bits(grown, oc.octree_grow(cur, d, full)), (d, full)
    cur = grown
    if d >= 2:
      n = int(oc.OctreeView(grown).nnum[d])
      label = (rng.random(n) < 0.4).astype(np.int32)
      if d == 5 and batch == 1:
        label[:] = 0                       # nothing splits: one node is kept
      cur = R.octree_update(grown, label, d, 1)
      assert same_bits(cur, oc.octree_update(grown, label, d, 1)), d
