"""The module route — `ocnn.ResNet` / `ocnn.UNet` assembled from `ocnn.OctreeConv`,
`ocnn.OctreeDeconv`, `ocnn.OctreeMaxPool` and the reference's building blocks — against the same
networks walked on the CPU over the oracle (ocnn_harness.cpu_modules)."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import oracle as oc
from ocnn_harness import cpu_modules, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def ocnn():
  import ocnn as mod
  mod.set_key_bits(64)
  return mod


def randomize_bn(net, seed):
  g = torch.Generator().manual_seed(seed)
  for m in net.modules():
    if isinstance(m, (torch.nn.BatchNorm1d, torch.nn.BatchNorm2d)):
      with torch.no_grad():
        m.weight.copy_(torch.rand(m.weight.shape, generator=g) + 0.5)
        m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.1)
        m.running_mean.copy_(torch.randn(m.running_mean.shape, generator=g) * 0.1)
        m.running_var.copy_(torch.rand(m.running_var.shape, generator=g) + 0.5)


def build(ocnn, clouds, depth, feats=None):
  pts = [oc.points_new(c[0], c[1], None if feats is None else feats[i]) for i, c in enumerate(clouds)]
  merged = oc.octree_batch([oc.points2octree(p, depth, 2, key_bits=64) for p in pts])
  octree = ocnn.points2octree_batch([torch.from_numpy(p) for p in pts], depth, 2, False, False, False,
                                    False, 4, 0.1, 2.0, False, False, False)
  assert np.array_equal(octree.cpu().numpy(), merged)
  return merged, octree


def test_resnet_module_matches_cpu(ocnn):
  """The reference's own ResNet (blocks on depths 6..3, pool to depth 2, average, FC 256 -> 40)."""
  torch.manual_seed(0)
  clouds = [synth.primitive_union(5000, 610 + i) for i in range(4)]
  merged, octree = build(ocnn, clouds, 6)
  net = ocnn.ResNet(6, 3, 40, 2).cuda().eval()
  randomize_bn(net, 1)
  want = cpu_modules.CpuModules(oc, oc.OctreeView).resnet(net, merged)
  with torch.no_grad():
    got = net(octree).cpu().numpy()
    assert got.shape == want.shape == (4, 40)
    assert gu.rel_err(got, want) < 1e-4
    # torch BatchNorm / ReLU modules after every kernel instead of the fused epilogue
    ocnn.modules.FUSE_EVAL_BN = False
    try:
      plain = net(octree).cpu().numpy()
    finally:
      ocnn.modules.FUSE_EVAL_BN = True
    assert gu.rel_err(plain, want) < 1e-4
    # bf16 channels_last activations: every convolution on the tensor-core kernel
    feat = ocnn.nn.feature_node_major(octree, 8, True)
    net8 = ocnn.ResNet(6, 8, 40, 2).cuda().eval()
    sd = net.state_dict()
    w = sd['conv1.conv.weights'].view(32, 3, 27)
    sd['conv1.conv.weights'] = torch.cat([w, w.new_zeros(32, 5, 27)], 1).reshape(32, 8 * 27)
    net8.load_state_dict(sd)
    got16 = net8(octree, feat).float().cpu().numpy()
  torch.cuda.synchronize()
  assert int(ocnn.tc_status('cuda').item()) == 0
  assert gu.rel_err(got16, want) < 6e-2


@pytest.mark.parametrize('nempty', [True, False])
def test_unet_module_matches_cpu(ocnn, nempty):
  """The reference's U-Net (kernel-2 stride-2 convolutions down, deconvolutions up, skip
  concatenation, interpolation at the input points, 1x1 head), on non-empty nodes as its ScanNet
  configuration runs it, and on all nodes."""
  torch.manual_seed(1)
  xyz, nrm, rgb = synth.indoor_scene(8000, 7)
  merged, octree = build(ocnn, [(xyz, nrm)], 7, feats=[rgb])
  net = ocnn.UNet(7, 6, 20, nempty=nempty).cuda().eval()
  randomize_bn(net, 2)
  pts = np.concatenate([xyz[:500], np.zeros((500, 1), np.float32)], 1)
  cpu = cpu_modules.CpuModules(oc, oc.OctreeView)
  want = cpu.unet(net, merged, pts)
  with torch.no_grad():
    got = net(octree, torch.from_numpy(pts).cuda()).cpu().numpy()
  assert got.shape == want.shape == (500, 20)
  assert gu.rel_err(got, want) < 1e-4
  want_nodes = cpu.unet(net, merged)
  with torch.no_grad():
    got_nodes = net(octree).cpu().numpy()
    assert gu.rel_err(got_nodes, want_nodes) < 1e-4
    # bf16: input channels padded to 8
    feat = ocnn.octree_feature(octree, 7, nempty)
    feat = torch.cat([feat, feat.new_zeros(1, 2, feat.shape[2], 1)], 1).to(torch.bfloat16)
    feat = feat.contiguous(memory_format=torch.channels_last)
    net8 = ocnn.UNet(7, 8, 20, nempty=nempty).cuda().eval()
    sd = net.state_dict()
    w = sd['conv1.conv.weights'].view(32, 6, 27)
    sd['conv1.conv.weights'] = torch.cat([w, w.new_zeros(32, 2, 27)], 1).reshape(32, 8 * 27)
    net8.load_state_dict(sd)
    got16 = net8(octree, data=feat).float().cpu().numpy()
  torch.cuda.synchronize()
  assert int(ocnn.tc_status('cuda').item()) == 0
  assert gu.rel_err(got16, want_nodes) < 8e-2


def test_unet_scene_depth8_parity(ocnn):
  """A reduced scene of the scene-scale configuration (40k points, depth 8, nempty, bf16) checked
  against the CPU chain, layer by layer: each stage's GPU output against the CPU stage fed
  bf16-rounded inputs."""
  torch.manual_seed(2)
  xyz, nrm, rgb = synth.indoor_scene(40000, 5000)
  merged, octree = build(ocnn, [(xyz, nrm)], 8, feats=[rgb])
  net = ocnn.UNet(8, 8, 20, nempty=True).cuda().eval()
  randomize_bn(net, 3)
  cpu = cpu_modules.CpuModules(oc, oc.OctreeView, round_fn=gu.bf16_round)
  cpu.trace = []
  want = cpu.unet(net, merged)
  feat = ocnn.octree_feature(octree, 8, True)
  feat = torch.cat([feat, feat.new_zeros(1, 2, feat.shape[2], 1)], 1).to(torch.bfloat16)
  feat = feat.contiguous(memory_format=torch.channels_last)
  stages = {}

  def hook(name):
    return lambda mod, inp, out: stages.__setitem__(name, out)
  net.conv1.register_forward_hook(hook('conv1'))
  for i in range(net.stages):
    net.downsample[i].register_forward_hook(hook('down%d' % (8 - i - 1)))
    net.encoder[i].register_forward_hook(hook('enc%d' % (8 - i - 1)))
    net.upsample[i].register_forward_hook(hook('up%d' % (8 - net.stages + i + 1)))
    net.decoder[i].register_forward_hook(hook('dec%d' % (8 - net.stages + i + 1)))
  with torch.no_grad():
    got = net(octree, data=feat).float().cpu().numpy()
  torch.cuda.synchronize()
  assert int(ocnn.tc_status('cuda').item()) == 0
  assert got.shape == want.shape
  assert gu.rel_err(got, want) < 8e-2
  assert len(cpu.trace) == 1 + 4 * net.stages
  for name, ref in cpu.trace:
    assert gu.rel_err(gu.to_np(stages[name]), ref) < 6e-2, name
