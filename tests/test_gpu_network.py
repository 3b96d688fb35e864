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
