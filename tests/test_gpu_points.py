"""GPU parity of the point-cloud preparation steps (transform / normalize / clip / bounding box)
against the CPU oracle, bit for bit, and the `.points` / `.octree` file round trip."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from conftest import same_bits
from oracle import oracle as oc
from ocnn_harness import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def ocnn():
  import ocnn as mod
  mod.set_key_bits(64)
  return mod


@pytest.fixture(scope='module')
def cloud():
  rng = np.random.default_rng(12)
  p, q = synth.primitive_union(30000, 31)
  f = rng.normal(size=(30000, 2)).astype(np.float32)
  lab = rng.integers(0, 5, size=30000).astype(np.float32)
  return p, q, f, lab


CASES = [([0.3, -0.2, 1.1], [1.0, 1.0, 1.0], [0.0, 0.0, 0.0], 0.0, ''),
         ([0.0, 0.0, 0.0], [0.8, 0.8, 0.8], [0.01, -0.02, 0.03], 0.02, 'x'),
         ([0.5, 0.25, -0.75], [0.9, 1.1, 0.7], [0.05, 0.0, 0.0], 0.0, 'xyz'),
         ([0.0, 0.0, 0.2], [1.0, 2.0, 1.0], [0.0, 0.0, 0.0], 0.001, 'z')]


@pytest.mark.parametrize('with_normals', [True, False])
def test_transform_points(ocnn, cloud, with_normals):
  p, q, f, lab = cloud
  pts = oc.points_new(p, q if with_normals else None, f, lab)
  for device in ('cpu', 'cuda'):
    src = torch.from_numpy(pts).to(device)
    for angle, scale, jitter, offset, axis in CASES:
      got = ocnn.transform_points(src, angle, scale, jitter, offset, axis)
      assert got.is_cuda
      want = oc.transform_points(pts, angle, scale, jitter, offset, axis)
      assert same_bits(got.cpu().numpy(), want), (angle, scale, axis, device)
  assert same_bits(src.cpu().numpy(), pts)            # the input is left alone


def test_normalize_and_bounding_box(ocnn, cloud):
  p, q, f, lab = cloud
  shifted = (p * np.float32(3.0) + np.array([1.0, -2.0, 0.5], np.float32)).astype(np.float32)
  pts = oc.points_new(shifted, q, f, lab)
  sphere = ocnn.bounding_sphere(torch.from_numpy(pts), 'box')
  box = oc.bounding_box(shifted)
  center = (box[3:] + box[:3]) / np.float32(2)
  half = (box[3:] - box[:3]) / np.float32(2)
  radius = np.sqrt(np.float32(half[0] * half[0]) + np.float32(half[1] * half[1]) +
                   np.float32(half[2] * half[2]) + np.float32(1e-20))
  assert np.allclose(sphere, [radius, center[0], center[1], center[2]], rtol=1e-6)
  got = ocnn.normalize_points(torch.from_numpy(pts), sphere[0], sphere[1:])
  inv = np.float32(1.0) / np.float32(sphere[0])
  want = oc.transform_points(pts, [0, 0, 0], [inv, inv, inv], [-np.float32(c) for c in sphere[1:]], 0.0)
  assert same_bits(got.cpu().numpy(), want)
  xyz = ocnn.points_property(got, 'xyz')
  assert float(xyz.abs().max()) <= 1.0 + 1e-6
  with pytest.raises(RuntimeError, match='Miniball'):
    ocnn.bounding_sphere(torch.from_numpy(pts), 'sphere')


@pytest.mark.parametrize('box', [([-1, -1, -1], [1, 1, 1]), ([-0.3, -0.5, -0.2], [0.4, 0.6, 0.9]),
                                 ([2, 2, 2], [3, 3, 3])])
def test_clip_points(ocnn, cloud, box):
  p, q, f, lab = cloud
  pts = oc.points_new(p, q, f, lab)
  lo, hi = box
  got, mask = ocnn.clip_points(torch.from_numpy(pts), [float(v) for v in lo], [float(v) for v in hi])
  want, wmask = oc.clip_points(pts, lo, hi)
  assert np.array_equal(mask.cpu().numpy(), wmask)
  g = got.cpu().numpy()
  kept = int(want[16:20].view(np.int32)[0])
  assert int(g[16:20].view(np.int32)[0]) == kept
  (xa, na, fa, la), _ = oc._points_blocks(g)
  (xb, nb, fb, lb), _ = oc._points_blocks(want)
  for u, v in ((xa, xb), (na, nb), (fa, fb), (la, lb)):
    assert same_bits(u[:kept], v[:kept])
  # the clipped cloud builds the octree of the kept points
  octree = ocnn.points2octree(got, 5, 2, False, False, False, False, 4, 0.1, 2.0, False, False, False)
  assert np.array_equal(octree.cpu().numpy(), oc.points2octree(want, 5, 2, key_bits=64))


def test_points_property_and_files(ocnn, cloud, tmp_path):
  p, q, f, lab = cloud
  pts = torch.from_numpy(oc.points_new(p, q, f, lab))
  assert torch.equal(ocnn.points_property(pts, 'xyz'), torch.from_numpy(p))
  assert torch.equal(ocnn.points_property(pts, 'normal'), torch.from_numpy(q))
  assert torch.equal(ocnn.points_property(pts, 'feature'), torch.from_numpy(f))
  assert torch.equal(ocnn.points_property(pts, 'label').view(-1), torch.from_numpy(lab))
  both = ocnn.points_batch_property([pts, pts], 'xyzi')
  assert both.shape == (60000, 4) and float(both[30000:, 3].min()) == 1.0
  changed = ocnn.points_set_property(pts, torch.from_numpy(q * 2), 'normal')
  assert torch.equal(ocnn.points_property(changed, 'normal'), torch.from_numpy(q * 2))
  path = str(tmp_path / 'cloud.points')
  ocnn.write_points(pts, path)
  assert torch.equal(ocnn.read_points(path), pts)
  octree = ocnn.points2octree(pts, 6, 2, False, False, False, False, 4, 0.1, 2.0, False, False, False)
  opath = str(tmp_path / 'cloud.octree')
  ocnn.write_octree(octree, opath)
  back = ocnn.read_octree(opath, 'cuda')
  assert torch.equal(back, octree)
  with open(path, 'r+b') as fh:
    fh.write(b'XX')
  with pytest.raises(ValueError):
    ocnn.read_points(path)


def test_transform_compose(ocnn, cloud):
  p, q, f, lab = cloud
  np.random.seed(5)
  flags = dict(depth=5, full_depth=2, distort=True, angle=[10, 180, 10], scale=0.2, jitter=0.1,
               bsphere='box', normal_axis='')
  tf = ocnn.TransformCompose(flags)
  np.random.seed(5)
  angle, scale, jitter = tf.transform_points.draw()
  np.random.seed(5)
  out = tf(torch.from_numpy(oc.points_new(p * np.float32(0.5), q, f, lab)))
  pts = oc.points_new(p * np.float32(0.5), q, f, lab)
  sphere = ocnn.bounding_sphere(torch.from_numpy(pts), 'box')
  inv = np.float32(1.0) / np.float32(sphere[0])
  step1 = oc.transform_points(pts, [0, 0, 0], [inv] * 3, [-np.float32(c) for c in sphere[1:]], 0.0)
  step2 = oc.transform_points(step1, angle, scale, jitter, 0.0, '')
  step3, wmask = oc.clip_points(step2, [-1] * 3, [1] * 3)
  assert np.array_equal(out['inbox_mask'].cpu().numpy(), wmask)
  assert np.array_equal(out['octree'].cpu().numpy(), oc.points2octree(step3, 5, 2, key_bits=64))
