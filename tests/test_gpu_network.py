"""Whole-network parity: the ResNet / LeNet forward passes of the benchmark configurations on the
GPU operators against the same networks chained over the CPU oracle."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import oracle as oc
from ocnn_harness import models, synth

pytestmark = pytest.mark.gpu


def logits_pair(net, clouds, depth, mode, tensor_core=True):
  import ocnn
  ocnn.set_key_bits(64)
  pts = [oc.points_new(p, q) for p, q in clouds]
  merged = oc.octree_batch([oc.points2octree(p, depth, 2, key_bits=64) for p in pts])
  want = models.CpuNet(net, oc, oc.OctreeView).forward(merged)
  octree = ocnn.points2octree_batch([torch.from_numpy(p) for p in pts], depth, 2, False, False,
                                    False, False, 4, 0.1, 2.0, False, False, False)
  gnet = models.GpuNet(net, mode, tensor_core=tensor_core)
  got = gnet.forward(octree).float().cpu().numpy()
  torch.cuda.synchronize()
  assert int(gnet.status.item()) == 0
  return got, want


def test_resnet_fp32_matches_cpu_chain():
  clouds = [synth.primitive_union(5000, 600 + i) for i in range(4)]
  net = models.resnet_params(6, 3, 40, 2, seed=1)
  got, want = logits_pair(net, clouds, 6, 'fp32')
  assert got.shape == want.shape == (4, 40)
  assert gu.rel_err(got, want) < 1e-4


def test_lenet_fp32_matches_cpu_chain():
  clouds = [synth.primitive_union(4000, 700 + i) for i in range(3)]
  net = models.lenet_params(5, 3, 40, seed=2)
  got, want = logits_pair(net, clouds, 5, 'fp32')
  assert got.shape == want.shape == (3, 40)
  assert gu.rel_err(got, want) < 1e-4


@pytest.mark.parametrize('tensor_core', [False, True])
def test_resnet_bf16_close_to_cpu_chain(tensor_core):
  # bf16 activations through ~35 layers: the per-layer tolerance of 2e-2 compounds, so the
  # end-to-end bound on the logits is looser
  clouds = [synth.primitive_union(5000, 600 + i) for i in range(4)]
  net = models.resnet_params(6, 3, 40, 2, seed=1)
  got, want = logits_pair(net, clouds, 6, 'bf16', tensor_core)
  assert gu.rel_err(got, want) < 6e-2
  assert np.array_equal(got.argmax(1), want.argmax(1)) or gu.rel_err(got, want) < 3e-2


# ---- scene segmentation U-Net (normals + RGB input, per-node class scores) -------------------------
def unet_pair(net, scene, depth, mode):
  import ocnn
  ocnn.set_key_bits(64)
  xyz, nrm, rgb = scene
  merged = oc.octree_batch([oc.points2octree(oc.points_new(xyz, nrm, rgb), depth, 2, key_bits=64)])
  want = models.CpuNet(net, oc, oc.OctreeView).forward(merged)
  pts = ocnn.points_new(torch.from_numpy(xyz), torch.from_numpy(nrm), torch.from_numpy(rgb),
                        torch.zeros(0))
  octree = ocnn.points2octree_batch([pts], depth, 2, False, False, False, False, 4, 0.1, 2.0,
                                    False, False, False)
  assert np.array_equal(octree.cpu().numpy(), merged)
  gnet = models.GpuNet(net, mode)
  got = gnet.forward(octree).cpu().numpy()
  torch.cuda.synchronize()
  assert gnet.error_status() == 0
  return got, want


def test_unet_matches_cpu_chain():
  scene = synth.indoor_scene(6000, 5)
  net = models.unet_params(6, 6, 20, seed=3, channels=(16, 32, 64, 128))
  got, want = unet_pair(net, scene, 6, 'fp32')
  assert got.shape == want.shape and got.shape[1] == 20
  assert gu.rel_err(got, want) < 1e-4
  got, want = unet_pair(net, scene, 6, 'bf16')
  assert gu.rel_err(got, want) < 6e-2


def test_unet_scene_scale_runs():
  """The scene configuration at full size (200k points, depth 9, channels 32-64-128-256): every
  layer on the bf16 kernels; finite scores for every finest node."""
  import ocnn
  ocnn.set_key_bits(64)
  xyz, nrm, rgb = synth.config_clouds(5, 1)[0]
  pts = ocnn.points_new(torch.from_numpy(xyz), torch.from_numpy(nrm), torch.from_numpy(rgb),
                        torch.zeros(0))
  octree = ocnn.points2octree_batch([pts], 9, 2, False, False, False, False, 4, 0.1, 2.0, False,
                                    False, False)
  net = models.unet_params(9, 6, 20, seed=4)
  gnet = models.GpuNet(net, 'bf16')
  scores = gnet.forward(octree)
  torch.cuda.synchronize()
  assert gnet.error_status() == 0
  nnum = int(ocnn.octree_info(octree)[4 + 9])
  assert scores.shape == (nnum, 20)
  assert bool(torch.isfinite(scores).all())
  # every layer has a tensor-core weight image (the 20-class head is widened to 32 channels)
  assert all(p.get('_packed') is not None for _, p in models.conv_layers(net))
