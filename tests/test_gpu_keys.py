"""GPU parity of key conversion, key search, interpolation at points and octree alignment against
the CPU oracle, plus the known answers of the reference's own tests
(pytorch/test/test_octree_key.py, test_octree_align.py, test_octree_trilinear.py)."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import oracle as oc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def ocnn():
  import ocnn as mod
  mod.set_key_bits(64)
  return mod


@pytest.fixture(scope='module')
def batch():
  clouds = gu.small_clouds(3, 4000, 400)
  singles, merged, _ = gu.oracle_batch(clouds, 6, 2, 64)
  return merged, gu.to_cuda_u8(merged), oc.OctreeView(merged), clouds


def samples(golden, names):
  return [torch.from_numpy(golden['k64_' + n]) for n in names]


def i64(a):
  return torch.from_numpy(np.asarray(a).astype(np.uint64).view(np.int64)).cuda()


def test_key_known_answers(ocnn, golden):
  octree = ocnn.octree_batch(samples(golden, ['octree_1', 'octree_1'])).cuda()
  xyz = ocnn.octree_property(octree, 'xyz', 5)
  pts = ocnn.octree_decode_key(xyz)
  gt = torch.tensor([[16, 16, 16, 0], [16, 16, 17, 0], [16, 17, 16, 0], [16, 17, 17, 0],
                     [17, 16, 16, 0], [17, 16, 17, 0], [17, 17, 16, 0], [17, 17, 17, 0],
                     [16, 16, 16, 1], [16, 16, 17, 1], [16, 17, 16, 1], [16, 17, 17, 1],
                     [17, 16, 16, 1], [17, 16, 17, 1], [17, 17, 16, 1], [17, 17, 17, 1]],
                    dtype=torch.int16, device='cuda')                 # test_octree_key.py:15-19
  assert torch.equal(pts, gt)
  assert torch.equal(ocnn.octree_encode_key(pts), xyz)
  key = ocnn.octree_xyz2key(xyz, 5)
  assert torch.equal(key, ocnn.octree_property(octree, 'key', 5))
  assert torch.equal(ocnn.octree_key2xyz(key, 5), xyz)
  q = torch.tensor([28673, 281474976739335, 10], dtype=torch.int64, device='cuda')     # :35-38
  assert ocnn.octree_search_key(q, octree, 5, False, False).tolist() == [1, 15, -1]
  q = torch.tensor([28672, 28673, 281474976739328, 10], dtype=torch.int64, device='cuda')   # :40-43
  assert ocnn.octree_search_key(q, octree, 5, False, True).tolist() == [0, -1, 1, -1]
  xyz = torch.tensor([[2049, 4095, 8011, 1], [511, 4095, 8011, 0]], dtype=torch.int16, device='cuda')
  enc = ocnn.octree_encode_key(xyz)
  assert torch.equal(ocnn.octree_decode_key(ocnn.octree_key2xyz(ocnn.octree_xyz2key(enc, 13), 13)), xyz)


def test_keys_and_search_vs_oracle(ocnn, batch):
  merged, octree, v, _ = batch
  rng = np.random.default_rng(2)
  for d in (6, 4):
    keys = v.prop('key', d).astype(np.uint64)
    xyz = ocnn.octree_key2xyz(i64(keys), d)
    assert np.array_equal(xyz.cpu().numpy().view(np.uint64), oc.key2xyz(keys, d))
    assert np.array_equal(ocnn.octree_xyz2key(xyz, d).cpu().numpy().view(np.uint64), keys)
    wild = rng.integers(0, 1 << 62, size=500).astype(np.uint64)
    assert np.array_equal(ocnn.octree_xyz2key(i64(wild), d).cpu().numpy().view(np.uint64),
                          oc.xyz2key(wild, d))
    query = np.concatenate([keys[::5], keys[:9] + np.uint64(1), wild[:50]])
    for nempty in (False, True):
      want = oc.search_key(oc.level_keys(merged, d, nempty), query)
      got = ocnn.octree_search_key(i64(query), octree, d, False, nempty)
      assert np.array_equal(got.cpu().numpy(), want)
    qx = oc.key2xyz(query, d)
    got = ocnn.octree_search_key(i64(qx), octree, d, True, False)
    assert np.array_equal(got.cpu().numpy(), oc.search_key(oc.level_keys(merged, d), oc.xyz2key(qx, d)))


@pytest.mark.parametrize('method', ['nearest', 'linear'])
@pytest.mark.parametrize('nempty', [False, True])
@pytest.mark.parametrize('mode', ['fp32_cm', 'fp32_nm', 'bf16_nm'])
def test_interp_vs_oracle(ocnn, batch, method, nempty, mode):
  merged, octree, v, clouds = batch
  rng = np.random.default_rng(11)
  d, C = 5, 12
  H = int(v.nnum_nempty[d] if nempty else v.nnum[d])
  data = rng.uniform(-1, 1, size=(C, H)).astype(np.float32)
  if mode == 'bf16_nm':
    data = gu.bf16_round(data)
  # the clouds' own points (every one sits in an occupied cell), points near the cube's faces
  # (corner cells that do not exist, lanes that wrap) and random points
  pts = np.concatenate([np.concatenate([c[0][:300], np.full((300, 1), i, np.float32)], 1)
                        for i, c in enumerate(clouds)] +
                       [np.concatenate([rng.uniform(-1, 1, size=(200, 3)), rng.integers(0, 3, (200, 1))], 1),
                        np.array([[-0.999, -0.999, -0.999, 0], [0.999, 0.999, 0.999, 2],
                                  [-0.999, 0.5, 0.999, 1]])]).astype(np.float32)
  interp = ocnn.OctreeInterp(d, method, nempty)
  got = interp(gu.data_cuda(data, mode != 'fp32_cm', mode == 'bf16_nm'), octree, torch.from_numpy(pts).cuda())
  scaled = pts.copy()
  scaled[:, :3] = (pts[:, :3] + np.float32(1.0)) * np.float32(2 ** (d - 1))
  want = oc.octree_interp(data, merged, d, scaled, method, nempty)
  assert got.shape == (1, C, pts.shape[0], 1)
  tol = 1e-5 if mode != 'bf16_nm' else 8e-3
  assert np.abs(gu.to_np(got) - want).max() < tol
  if method == 'nearest':
    assert np.abs(want[:, :900]).sum(0).min() > 0 or nempty      # the clouds' own points are found


def test_trilinear_known_answer(ocnn, golden):
  # pytorch/test/test_octree_trilinear.py:10-16: constant data stays constant
  octree = ocnn.octree_batch(samples(golden, ['octree_1', 'octree_1'])).cuda()
  data = torch.ones(1, 3, 16, 1, device='cuda')
  out = ocnn.octree_trilinear(data, octree, 4, 5)
  assert out.shape == (1, 3, 16, 1) and bool((out == 1).all())


def test_align_known_answers(ocnn, golden):
  # pytorch/test/test_octree_align.py:14-78
  one = ocnn.octree_batch(samples(golden, ['octree_1'])).cuda()
  two = ocnn.octree_batch(samples(golden, ['octree_1', 'octree_1'])).cuda()
  x = torch.rand(1, 3, 16, 1, device='cuda')
  out, idx = ocnn.octree_align(x, two, two, 5)
  assert torch.equal(out, x) and idx.tolist() == list(range(16))
  x8 = torch.rand(1, 3, 8, 1, device='cuda')
  out, idx = ocnn.octree_align(x8, one, two, 5)
  assert torch.equal(out, torch.cat([x8, torch.zeros_like(x8)], 2)) and idx.tolist() == list(range(8))
  out, idx = ocnn.octree_align(x, two, one, 5)
  assert torch.equal(out, x[:, :, :8]) and idx.tolist() == list(range(8)) + [-1] * 8
  grad = ocnn.nn.octree_align_grad(torch.ones(1, 3, 8, 1, device='cuda'), idx)
  assert torch.equal(grad, torch.cat([torch.ones(1, 3, 8, 1), torch.zeros(1, 3, 8, 1)], 2).cuda())


def test_align_between_different_octrees(ocnn, batch):
  merged, octree, v, clouds = batch
  rng = np.random.default_rng(4)
  other_clouds = [(c[0][::2], c[1][::2]) for c in clouds]
  _, other, _ = gu.oracle_batch(other_clouds, 6, 2, 64)
  vo = oc.OctreeView(other)
  d, C = 5, 6
  x = rng.uniform(-1, 1, size=(C, int(v.nnum[d]))).astype(np.float32)
  want_idx = oc.search_key(oc.level_keys(other, d), oc.level_keys(merged, d))
  want = np.zeros((C, int(vo.nnum[d])), np.float32)
  want[:, want_idx[want_idx >= 0]] = x[:, want_idx >= 0]
  for nm in (False, True):
    out, idx = ocnn.octree_align(gu.data_cuda(x, nm), octree, gu.to_cuda_u8(other), d)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.array_equal(gu.to_np(out), want)
    assert 0 < (want_idx >= 0).sum() < want_idx.size
