"""GPU parity tests of the bandwidth operators and the neighbour table against the CPU oracle.
Bit-exact for every integer / index / copy result."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import oracle as oc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def ocnn():
  import ocnn as mod
  return mod


@pytest.fixture(scope='module', params=[32, 64])
def batch(request):
  kb = request.param
  clouds = gu.small_clouds(3, 4000, 100)
  singles, merged, pts = gu.oracle_batch(clouds, 6, 2, kb)
  return kb, singles, merged, gu.to_cuda_u8(merged), oc.OctreeView(merged)


# ---- known answers of the reference's own tests, on the GPU ---------------------------------
def test_pool_known_answer(ocnn, golden):
  # pytorch/test/test_octree_pool.py:10-39: pooled values, mask [[7],[15]],[[0],[8]], padded output
  octree = ocnn.octree_batch([torch.from_numpy(golden['k64_octree_1'])] * 2)
  row0 = [1.1, 2.2, 3.3, 4.4, 5.5, 6.6, 7.7, 8.8]
  row1 = [8.1, 7.2, 6.3, 5.4, 4.5, 3.6, 2.7, 1.8]
  data = np.array([row0 + row0, row1 + row1], np.float32)
  out, mask = ocnn.OctreeMaxPool(5, return_indices=True)(gu.data_cuda(data), octree)
  want = np.zeros((2, 16), np.float32)
  want[:, 0], want[:, 8] = [8.8, 8.1], [8.8, 8.1]
  assert np.array_equal(mask.cpu().numpy(), np.array([[[[7], [15]], [[0], [8]]]], np.int32))
  assert np.array_equal(gu.to_np(out), want)


def test_property_known_answers(ocnn, golden):
  # pytorch/test/test_octree_property.py:10-55
  octree = ocnn.octree_batch([torch.from_numpy(golden['k64_octree_1'])] * 2)
  assert octree.is_cuda
  assert ocnn.octree_property(octree, 'index', 5).cpu().tolist() == [0] * 8 + [1] * 8
  f = ocnn.octree_property(octree, 'feature', 5).cpu().numpy()
  want = np.zeros((3, 16), np.float32)
  want[:, [0, 8]] = 3.0 ** 0.5 / 3.0
  assert f.shape == (1, 3, 16, 1) and np.allclose(f[0, :, :, 0], want)
  child = -np.ones(16)
  child[0], child[8] = 0, 1
  assert np.array_equal(ocnn.octree_property(octree, 'child', 5).cpu().numpy(), child)
  cat = torch.cat([ocnn.octree_property(octree, 'child', d) for d in range(1, 6)])
  assert torch.equal(ocnn.octree_property(octree, 'child')[2:], cat)
  assert ocnn.octree_property(octree, 'node_num').cpu().tolist() == [2, 16, 128, 16, 16, 16]
  assert ocnn.octree_property(octree, 'node_num_cum').cpu().tolist() == [0, 2, 18, 146, 162, 178, 194]
  assert ocnn.octree_property(octree, 'node_num', 5).item() == 16
  assert ocnn.octree_property(octree, 'node_num_cum', 5).item() == 178
  assert ocnn.octree_property(octree, 'batch_size').item() == 2
  assert ocnn.octree_property(octree, 'depth').item() == 5
  assert ocnn.octree_property(octree, 'full_depth').item() == 2
  # same answers from a host tensor
  host = octree.cpu()
  assert ocnn.octree_property(host, 'node_num').tolist() == [2, 16, 128, 16, 16, 16]


def octree2col_bruteforce(data, ks, stride, taps):
  channel = data.shape[0]
  top_h = 8 if stride == 1 else 1
  col = np.zeros((channel, len(taps), top_h), np.float32)
  for h in range(top_h):
    hx, hy, hz = h >> 2, (h >> 1) & 1, h & 1
    for k, tap in enumerate(taps):
      x, y, z = hx + tap // 9 - 1, hy + (tap // 3) % 3 - 1, hz + tap % 3 - 1
      if 0 <= x < 2 and 0 <= y < 2 and 0 <= z < 2:
        col[:, k, h] = data[:, 4 * x + 2 * y + z]
  return col


TAPS = {'333': list(range(27)), '111': [13], '222': [13, 14, 16, 17, 22, 23, 25, 26],
        '311': [4, 13, 22], '331': [1, 4, 7, 10, 13, 16, 19, 22, 25]}


def test_octree2col_known_answer(ocnn, golden):
  # pytorch/test/test_octree2col.py:52-67: octree_1, depth 1, 5 kernel shapes x 2 strides
  octree = ocnn.octree_batch([torch.from_numpy(golden['k64_octree_1'])])
  rng = np.random.default_rng(1)
  data = rng.uniform(-1, 1, size=(3, 8)).astype(np.float32)
  for stride in (1, 2):
    for ks in ([3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]):
      out = ocnn.octree2col(gu.data_cuda(data), octree, 1, ks, stride, False)
      want = octree2col_bruteforce(data, ks, stride, TAPS[''.join(map(str, ks))])
      assert np.array_equal(out.cpu().numpy(), want), (ks, stride)


# ---- differential tests against the oracle ----------------------------------------------------
@pytest.mark.parametrize('layout', ['channel_major', 'node_major'])
@pytest.mark.parametrize('bf16', [False, True])
def test_pad_depad_pool(ocnn, batch, layout, bf16):
  kb, _, merged, octree, v = batch
  nm = layout == 'node_major'
  rng = np.random.default_rng(4)
  for d, C in ((6, 5), (5, 16), (3, 8), (2, 3)):
    H, Hne = int(v.nnum[d]), int(v.nnum_nempty[d])
    x = rng.uniform(-1, 1, size=(C, H)).astype(np.float32)
    x[0, :16] = 0.5                      # ties -> first maximum
    if not bf16:
      x[1, 8:16] = np.nan                # NaN never wins
    xs = rng.uniform(-1, 1, size=(C, Hne)).astype(np.float32)
    if bf16:
      x, xs = gu.bf16_round(x), gu.bf16_round(xs)
    child = v.prop('child', d)
    got = ocnn.octree_pad(gu.data_cuda(xs, nm, bf16), octree, d, 0.25)
    assert got.shape == (1, C, H, 1)
    assert np.array_equal(gu.to_np(got), oc.pad(xs, child, 0.25))
    got = ocnn.octree_depad(gu.data_cuda(x, nm, bf16), octree, d)
    assert np.array_equal(gu.to_np(got), oc.depad(x, child, Hne), equal_nan=True)
    if d > 1:
      top, mask = ocnn.octree_max_pool(gu.data_cuda(x, nm, bf16), octree, d)
      wt, wm = oc.max_pool(x)
      assert np.array_equal(gu.to_np(top), wt, equal_nan=True)
      m = mask.contiguous().view(C, H // 8).cpu().numpy()
      assert np.array_equal(m, wm)


@pytest.mark.parametrize('C', [8, 32, 40])
def test_max_pool_pad_fused(ocnn, batch, C):
  """ocnn_octree_max_pool_pad == octree_max_pool followed by octree_pad(0), bit for bit, on every
  level; also through the OctreeMaxPool module, which takes the fused path for such data."""
  _, _, _, octree, v = batch
  rng = np.random.default_rng(11)
  for d in range(2, v.depth + 1):
    H = int(v.nnum[d])
    x = gu.bf16_round(rng.uniform(-1, 1, size=(C, H)).astype(np.float32))
    x[0, :16] = 0.5
    data = gu.data_cuda(x, True, True)
    want = oc.pad(oc.max_pool(x)[0], v.prop('child', d - 1), 0.0)
    got = ocnn.nn.octree_max_pool_pad(data, octree, d)
    assert got.shape == (1, C, int(v.nnum[d - 1]), 1)
    assert np.array_equal(gu.to_np(got), want)
    assert np.array_equal(gu.to_np(ocnn.OctreeMaxPool(d)(data, octree)), want)
  with pytest.raises(RuntimeError, match='node-major'):
    ocnn.nn.octree_max_pool_pad(torch.zeros(1, 8, int(v.nnum[3]), 1, device='cuda'), octree, 3)


@pytest.mark.parametrize('nm,bf16,C', [(False, False, 5), (True, False, 6), (True, True, 8), (True, True, 40),
                                       (True, True, 12)])
def test_octree_tile(ocnn, batch, nm, bf16, C):
  """OctreeTile = octree_depad + eightfold repeat, bit for bit, on every level that has a finer one."""
  _, _, _, octree, v = batch
  rng = np.random.default_rng(13)
  for d in range(1, v.depth):
    H = int(v.nnum[d])
    x = rng.uniform(-1, 1, size=(C, H)).astype(np.float32)
    if bf16:
      x = gu.bf16_round(x)
    want = np.repeat(oc.depad(x, v.prop('child', d), int(v.nnum_nempty[d])), 8, axis=1)
    got = ocnn.octree_tile(gu.data_cuda(x, nm, bf16), octree, d)
    assert got.shape == (1, C, int(v.nnum[d + 1]), 1)
    assert np.array_equal(gu.to_np(got), want)
    assert np.array_equal(gu.to_np(ocnn.OctreeTile(d)(gu.data_cuda(x, nm, bf16), octree)), want)
  with pytest.raises(RuntimeError, match='no finer level'):
    ocnn.octree_tile(torch.zeros(1, 2, int(v.nnum[v.depth]), 1, device='cuda'), octree, v.depth)


def test_pad_shape_errors(ocnn, batch):
  _, _, _, octree, v = batch
  with pytest.raises(RuntimeError, match='data height'):
    ocnn.octree_pad(torch.zeros(1, 2, 7, 1, device='cuda'), octree, 4)
  with pytest.raises(RuntimeError, match='data height'):
    ocnn.octree_depad(torch.zeros(1, 2, 7, 1, device='cuda'), octree, 4)
  with pytest.raises(RuntimeError, match='larger than 1'):
    ocnn.octree_max_pool(torch.zeros(1, 2, int(v.nnum[1]), 1, device='cuda'), octree, 1)
  with pytest.raises(RuntimeError, match='CUDA tensor'):
    ocnn.octree_pad(torch.zeros(1, 2, int(v.nnum_nempty[4]), 1), octree, 4)


def test_neighbour_table(ocnn, batch):
  """ocnn_calc_neigh through octree_batch: merge on the GPU, compare every level's table."""
  kb, singles, merged, _, v = batch
  got = ocnn.octree_batch([torch.from_numpy(s) for s in singles])
  assert got.is_cuda and np.array_equal(got.cpu().numpy(), merged)
  g = oc.OctreeView(got.cpu().numpy())
  for d in range(1, v.depth + 1):
    assert np.array_equal(g.prop('neigh', d), v.prop('neigh', d)), d
  neigh = ocnn.octree_property(got, 'neigh', 4).cpu().numpy()
  assert neigh.shape == (int(v.nnum[4]), 8)
  assert np.array_equal(neigh.reshape(-1, 64), v.prop('neigh', 4))


def test_merge_samples_matches_reference_fixture(ocnn, golden):
  for kb in (32, 64):
    tag = 'k%d_' % kb
    got = ocnn.octree_batch([torch.from_numpy(golden[tag + 'octree_1']),
                             torch.from_numpy(golden[tag + 'octree_2']).cuda()])
    assert np.array_equal(got.cpu().numpy(), golden[tag + 'merge_samples_12'])
    got = ocnn.octree_batch([torch.from_numpy(golden[tag + 'b%d_octree' % i]) for i in range(3)])
    assert np.array_equal(got.cpu().numpy(), golden[tag + 'b_merged'])
  with pytest.raises(RuntimeError, match='not consistent'):
    ocnn.octree_batch([torch.from_numpy(golden['k32_octree_1']),
                       torch.from_numpy(golden['k32_a_octree'])])


def test_octree2col_matches_oracle(ocnn, batch):
  _, _, _, octree, v = batch
  rng = np.random.default_rng(6)
  for d in (6, 4, 2):
    H = int(v.nnum[d])
    x = rng.uniform(-1, 1, size=(3, H)).astype(np.float32)
    for ks in ([3, 3, 3], [2, 2, 2], [1, 3, 3], [3, 1, 3], [1, 1, 3], [1, 3, 1]):
      for stride in (1, 2):
        hc = H if stride == 1 else H // 8
        got = ocnn.octree2col(gu.data_cuda(x), octree, d, ks, stride, False)
        assert np.array_equal(got.cpu().numpy(), oc.octree2col(x, v.prop('neigh', d), ks, stride, hc))


@pytest.mark.parametrize('half', [False, True], ids=['bf16', 'fp16'])
@pytest.mark.parametrize('shape', [(32, 64, 512, 40), (3, 8, 32, 7), (1, 512, 96, 20)])
def test_global_pool_fc(shape, half):
  """FullOctreeGlobalPool + Linear (pytorch/ocnn/octree_pool.py:106-115, resnet.py:18-21) in one launch
  against the mean over each shape's rows and a float64 matrix product."""
  import ocnn
  batch, per, C, nout = shape
  rng = np.random.default_rng(batch + C)
  rnd = gu.half_round if half else gu.bf16_round
  x = rnd(rng.uniform(-1, 1, size=(C, batch * per)).astype(np.float32))
  w = rng.normal(size=(nout, C)).astype(np.float32)
  b = rng.normal(size=nout).astype(np.float32)
  want = x.reshape(C, batch, per).astype(np.float64).mean(axis=2).T @ w.T.astype(np.float64) + b
  got = ocnn.nn.global_pool_fc(gu.data_cuda(x, True, not half, half), torch.from_numpy(w).cuda(),
                               torch.from_numpy(b).cuda(), batch)
  assert got.shape == (batch, nout) and got.dtype == torch.float32
  assert np.abs(got.cpu().numpy() - want).max() < 1e-4 * max(1.0, np.abs(want).max())
  with pytest.raises(RuntimeError, match='rows'):
    ocnn.nn.global_pool_fc(gu.data_cuda(x, True, not half, half), torch.from_numpy(w).cuda(), None, batch * per + 1)
