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


# ---- the benchmark configurations at full size ---------------------------------------------------------
def test_config1_single_conv_exact():
  """BASELINE configuration 1: 10,000 points uniform on the unit sphere with outward normals as
  the 3-channel signal, depth 5, full depth 2; 3x3x3 convolution at depth 5, stride 1, 3 -> 32,
  weights N(0, 0.02).  Octree bytes equal, convolution within 1e-5."""
  import ocnn
  ocnn.set_key_bits(64)
  xyz, nrm, _ = synth.config_clouds(1)[0]
  pts = oc.points_new(xyz, nrm)
  want_octree = oc.octree_batch([oc.points2octree(pts, 5, 2, key_bits=64)])
  octree = ocnn.points2octree_batch([torch.from_numpy(pts)], 5, 2, False, False, False, False, 4, 0.1,
                                    2.0, False, False, False)
  assert np.array_equal(octree.cpu().numpy(), want_octree)
  v = oc.OctreeView(want_octree)
  x = np.ascontiguousarray(v.prop('feature', 5))
  assert x.shape == (3, int(v.nnum[5]))
  w = np.random.default_rng(1000).normal(scale=0.02, size=(32, 81)).astype(np.float32)
  want = oc.octree_conv(x, w, want_octree, 5, 32, [3, 3, 3], 1)
  feat = ocnn.octree_property(octree, 'feature', 5)
  got = ocnn.OctreeConv(5, 3, 32).cuda()
  with torch.no_grad():
    got.weights.copy_(torch.from_numpy(w))
  y = got(feat, octree)
  assert gu.rel_err(gu.to_np(y), want) < 1e-5


@pytest.fixture(scope='module')
def full_batch():
  """The benchmark batch: 32 shapes x 20k points, depth 6, and the CPU forward over the oracle
  (fp32 and with bf16-rounded layer inputs, traced per layer)."""
  clouds = [synth.primitive_union(20000, 3000 + i) for i in range(32)]
  pts = [oc.points_new(p, q) for p, q in clouds]
  merged = oc.octree_batch([oc.points2octree(p, 6, 2, key_bits=64) for p in pts])
  net = models.resnet_params(6, 3, 40, 2, seed=0)
  want = models.CpuNet(net, oc, oc.OctreeView).forward(merged)
  rounded = models.CpuNet(net, oc, oc.OctreeView, round_fn=gu.bf16_round)
  rounded.trace = []
  rounded.forward(merged)
  return pts, merged, net, want, rounded.trace


def test_full_size_forward_parity(full_batch):
  """ResNet O-CNN d6 on the very batch the benchmark times: GPU fp32, GPU bf16 through the recorded
  executor and GPU bf16 through the operator-by-operator route, against the CPU chain."""
  import ocnn
  ocnn.set_key_bits(64)
  pts, merged, net, want, _ = full_batch
  octree = ocnn.points2octree_batch([torch.from_numpy(p) for p in pts], 6, 2, False, False, False,
                                    False, 4, 0.1, 2.0, False, False, False)
  assert np.array_equal(octree.cpu().numpy(), merged)
  got32 = models.GpuNet(net, 'fp32').forward(octree).cpu().numpy()
  assert gu.rel_err(got32, want) < 1e-4
  for executor in (True, False):
    gnet = models.GpuNet(net, 'bf16', executor=executor)
    got = gnet.forward(octree).float().cpu().numpy()
    torch.cuda.synchronize()
    assert gnet.error_status() == 0
    assert got.shape == want.shape == (32, 40)
    assert gu.rel_err(got, want) < 6e-2, executor       # compounded over ~45 bf16 layers
    assert (got.argmax(1) == want.argmax(1)).mean() > 0.9


def test_full_size_per_layer_parity(full_batch):
  """Every convolution of the network at the benchmark size, one at a time: the GPU kernel (the
  tensor-core one wherever the benchmark uses it) fed the very input the CPU layer saw (rounded to
  bf16), against that CPU layer's output: rel < 2e-2 per layer."""
  import ocnn
  ocnn.set_key_bits(64)
  pts, merged, net, _, trace = full_batch
  octree = gu.to_cuda_u8(merged)
  gnet = models.GpuNet(net, 'bf16', executor=False)
  layers = {p['name']: p for _, p in models.conv_layers(net)}
  worst = 0.0
  for name, d, x, y in trace:
    p = layers[name]
    xin = x
    if p['_cin'] != x.shape[0]:
      xin = np.concatenate([x, np.zeros((p['_cin'] - x.shape[0], x.shape[1]), np.float32)])
    got = gnet._conv(gu.data_cuda(xin, True, True), p, octree, d, False)
    err = gu.rel_err(gu.to_np(got)[:p['cout']], y)
    worst = max(worst, err)
    assert err < 2e-2, (name, err)
  torch.cuda.synchronize()
  assert gnet.error_status() == 0
  assert worst > 0


BENCH_SIZE_TC = [(8, 32, [3, 3, 3]), (32, 32, [3, 3, 3]), (24, 40, [3, 3, 3]), (64, 64, [3, 3, 3]),
                 (128, 128, [3, 3, 3]), (192, 64, [3, 3, 3]), (64, 512, [3, 3, 3]), (128, 256, [3, 3, 3]),
                 (192, 256, [3, 3, 3])]


@pytest.mark.parametrize('case', BENCH_SIZE_TC, ids=lambda c: '%dto%d' % (c[0], c[1]))
def test_tensor_core_at_benchmark_size(full_batch, case):
  """The launch configurations the benchmark runs (many waves; two or three CTAs per SM with
  two-stage rings and 128-row tiles, or, where Cin is a multiple of 64, the persistent kernel with
  256-row tiles and a ragged last tile) on the depth-6 level of the benchmark batch: the tensor-core kernel with
  its fused epilogue against the fp32 kernel on the same GPU (every row) and against the CPU oracle
  on a sample of rows."""
  import ocnn
  pts, merged, _, _, _ = full_batch
  cin, cout, ks = case
  octree = gu.to_cuda_u8(merged)
  v = oc.OctreeView(merged)
  H = int(v.nnum[6])
  g = torch.Generator(device='cuda').manual_seed(cin + cout)
  x = (torch.rand(1, cin, H, 1, device='cuda', generator=g) * 2 - 1).to(torch.bfloat16)
  x = x.contiguous(memory_format=torch.channels_last)
  w = (torch.randn(cout, cin * 27, device='cuda', generator=g) * 0.1).to(torch.bfloat16).float()
  scale = torch.rand(cout, device='cuda', generator=g) + 0.5
  bias = torch.randn(cout, device='cuda', generator=g)
  res = torch.randn(1, cout, H, 1, device='cuda', generator=g).to(torch.bfloat16)
  res = res.contiguous(memory_format=torch.channels_last)
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights(w, cin, cout, ks)
  got = ocnn.nn.octree_conv_tc(x, packed, octree, 6, cout, ks, 1, scale, bias, res, True, status)
  ref = ocnn.nn.octree_conv_fused(x.float().contiguous(), w, octree, 6, cout, ks, 1, scale, bias,
                                  res.float().contiguous(), True)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  err = float((got.float() - ref).abs().max()) / float(ref.abs().max())
  assert err < 8e-3, err
  # a few hundred rows against the CPU: rows of the first, a middle and the last tile
  rows = np.unique(np.concatenate([np.arange(0, 128), np.arange(H // 2, H // 2 + 128), np.arange(H - 128, H)]))
  xn = x.float().contiguous().view(cin, H).cpu().numpy()
  neigh = v.prop('neigh', 6).reshape(-1)
  ni = oc.ni_table(ks).reshape(8, 27)
  wn = w.cpu().numpy().reshape(cout, cin, 27)
  sc, bi = scale.cpu().numpy(), bias.cpu().numpy()
  rn = res.float().contiguous().view(cout, H).cpu().numpy()
  gn = got.float().contiguous().view(cout, H).cpu().numpy()
  for h in rows:
    nb = neigh[(h >> 3) * 64 + ni[h & 7]]
    col = np.where(nb[None, :] >= 0, xn[:, np.maximum(nb, 0)], 0.0)          # [cin, 27]
    y = np.maximum(np.einsum('oct,ct->o', wn, col) * sc + bi + rn[:, h], 0)
    assert np.abs(gn[:, h] - y).max() < 2e-2 * max(1.0, np.abs(y).max()), h


PERSISTENT_CASES = [
    # (depth of the output, cin, cout, kernel, stride, nempty, fp16)
    (6, 64, 256, [3, 3, 3], 1, True, False),     # non-empty nodes only: rows through ichild / child
    (5, 64, 256, [3, 3, 3], 2, False, True),     # stride 2 (output on depth 5), fp16
    (6, 128, 256, [1, 1, 1], 1, False, False),   # 1x1: the identity table
    (5, 128, 512, [3, 3, 3], 1, False, True),    # two slices of 256 columns, fp16
    # sibling-group layers with 8 / 16 channels: tile rows are groups, indices from the neighbour blocks
    (6, 8, 32, [3, 3, 3], 1, False, False),
    (6, 8, 8, [3, 3, 3], 1, False, True),
    (6, 16, 16, [3, 3, 3], 1, False, False),
    (6, 16, 32, [3, 1, 3], 1, False, False),     # 9 taps
]


@pytest.mark.parametrize('case', PERSISTENT_CASES, ids=lambda c: 'd%d_%dto%d_k%s_s%d_ne%d_h%d' % (
    c[0], c[1], c[2], ''.join(map(str, c[3])), c[4], c[5], c[6]))
def test_persistent_kernel_layer_kinds(full_batch, case):
  """The persistent tensor-core kernel (256 output columns, levels of many tiles) on the layer kinds
  it serves besides the plain convolution, against the CUDA-core fp32-accumulating kernel on the
  same 16-bit data (that kernel is checked against the CPU code on the small batch)."""
  import ocnn
  pts, merged, _, _, _ = full_batch
  d_out, cin, cout, ks, stride, nempty, half = case
  d_in = d_out + 1 if stride == 2 else d_out
  octree = gu.to_cuda_u8(merged)
  v = oc.OctreeView(merged)
  H = int(v.nnum_nempty[d_in]) if nempty else int(v.nnum[d_in])
  dt = torch.float16 if half else torch.bfloat16
  g = torch.Generator(device='cuda').manual_seed(cin + cout + stride)
  x = (torch.rand(1, cin, H, 1, device='cuda', generator=g) * 2 - 1).to(dt)
  x = x.contiguous(memory_format=torch.channels_last)
  kd = int(np.prod(ks))
  w = (torch.randn(cout, cin * kd, device='cuda', generator=g) * 0.1)
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights_general(w, cin, cout, ks, stride, False, nempty, half)
  got = ocnn.nn.octree_conv_tc_general(x, packed, octree, d_in, cout, ks, stride, nempty, False,
                                       None, None, None, False, status)
  ref = ocnn.nn.octree_conv_general(x, w, octree, d_in, cout, ks, stride, nempty, False)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  assert got.shape == ref.shape and got.shape[2] >= 3 * 148 * 256
  err = float((got.float() - ref.float()).abs().max()) / float(ref.float().abs().max())
  assert err < 1.2e-2, err
