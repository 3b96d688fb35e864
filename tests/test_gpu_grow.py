"""The generative path's octree editing on the GPU (octree_new / octree_grow / octree_update,
pytorch/cpp/octree_grow.cpp) against the oracle's restatement, which is pinned on the compiled
reference: byte-identical octrees along a decoder-like chain of levels."""
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


@pytest.mark.parametrize('kb', [64, 32])
@pytest.mark.parametrize('setup', [(1, 3, False, 0), (2, 4, True, 0), (5, 0, False, 4)])
def test_new_grow_update_chain(ocnn, kb, setup):
  batch, channel, node_dis, adp = setup
  ocnn.set_key_bits(kb)
  try:
    rng = np.random.default_rng(batch + kb)
    got = ocnn.octree_new(batch, channel, node_dis, adp)
    want = oc.octree_new(batch, channel, node_dis, adp, kb)
    assert got.is_cuda and np.array_equal(got.cpu().numpy(), want)
    for d in range(1, 7):
      full = d <= 2
      got = ocnn.octree_grow(got, d, full)
      want = oc.octree_grow(want, d, full)
      assert np.array_equal(got.cpu().numpy(), want), (d, full)
      if d >= 2:
        n = int(oc.OctreeView(want).nnum[d])
        label = (rng.random(n) < 0.45).astype(np.int32)
        if d == 6 and batch == 1:
          label[:] = 0                     # nothing splits: one node is kept
        got = ocnn.octree_update(got, torch.from_numpy(label).cuda(), d, 1)
        want = oc.octree_update(want, label, d, 1)
        assert np.array_equal(got.cpu().numpy(), want), d
        # the cached header follows the edit
        assert int(ocnn.octree_property(got, 'node_num_ne', d)[0]) == int(oc.OctreeView(want).nnum_nempty[d])
  finally:
    ocnn.set_key_bits(64)


def test_create_full_octree_and_convolution_on_it(ocnn):
  """create_full_octree (pytorch/ocnn/modules.py:325-330) and a convolution over the grown
  octree's neighbour table: the grown octree is a working input of the operators."""
  octree = ocnn.create_full_octree(3, 4, batch_size=2, node_dis=True)
  want = oc.octree_new(2, 4, True, 0, 64)
  for d in (1, 2, 3):
    want = oc.octree_grow(want, d, True)
  assert np.array_equal(octree.cpu().numpy(), want)
  rng = np.random.default_rng(9)
  H = int(oc.OctreeView(want).nnum[3])
  x = rng.uniform(-1, 1, size=(4, H)).astype(np.float32)
  w = rng.normal(scale=0.2, size=(6, 4 * 27)).astype(np.float32)
  got = ocnn.octree_conv(gu.data_cuda(x), torch.from_numpy(w).cuda(), octree, 3, 6, [3, 3, 3], 1)
  ref = oc.octree_conv(x, w, want, 3, 6, [3, 3, 3], 1)
  assert gu.rel_err(gu.to_np(got), ref) < 1e-5


def test_grow_errors(ocnn):
  octree = ocnn.octree_new(2, 4, True, 0)
  with pytest.raises(RuntimeError, match='skips a level'):
    ocnn.octree_grow(octree, 2, True)
  grown = ocnn.octree_grow(ocnn.octree_grow(octree, 1, True), 2, True)
  with pytest.raises(RuntimeError, match='labels for'):
    ocnn.octree_update(grown, torch.zeros(5, dtype=torch.int32, device='cuda'), 2, 1)
