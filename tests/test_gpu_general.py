"""GPU parity of every OctreeConv / OctreeDeconv variant (stride 1 or 2, all or non-empty nodes),
the column operators behind them, and the fp16 data type, against the CPU oracle.
Tolerances (max |y - y_ref| / max |y_ref| per tensor): 1e-5 for fp32, 2e-2 for bf16 / fp16 data."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import oracle as oc

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
HALF_TOL = 2e-2
KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]]   # pytorch/test/test_octree_deconv.py:84


@pytest.fixture(scope='module')
def ocnn():
  import ocnn as mod
  mod.set_key_bits(64)
  return mod


@pytest.fixture(scope='module')
def batch():
  clouds = gu.small_clouds(3, 4000, 300)
  singles, merged, _ = gu.oracle_batch(clouds, 6, 2, 64)
  return merged, gu.to_cuda_u8(merged), oc.OctreeView(merged)


def bottom_height(v, d, stride, nempty, deconv):
  return int(v.nnum_nempty[d]) if (nempty or (deconv and stride == 2)) else int(v.nnum[d])


def weight_shape(cin, cout, kd, deconv):
  return (cin, cout * kd) if deconv else (cout, cin * kd)


@pytest.mark.parametrize('ks', KERNELS, ids=lambda k: ''.join(map(str, k)))
@pytest.mark.parametrize('stride', [1, 2])
@pytest.mark.parametrize('nempty', [False, True])
@pytest.mark.parametrize('deconv', [False, True])
def test_conv_general_fp32(ocnn, batch, ks, stride, nempty, deconv):
  merged, octree, v = batch
  rng = np.random.default_rng(sum(ks) * 100 + stride * 10 + nempty * 2 + deconv)
  cin, cout, kd = 5, 7, int(np.prod(ks))
  for d in (5, 3):
    x = rng.uniform(-1, 1, size=(cin, bottom_height(v, d, stride, nempty, deconv))).astype(np.float32)
    w = rng.normal(scale=0.2, size=weight_shape(cin, cout, kd, deconv)).astype(np.float32)
    want = oc.octree_conv_general(x, w, merged, d, cout, ks, stride, nempty, deconv)
    wt = torch.from_numpy(w).cuda()
    for node_major in (False, True):
      got = ocnn.nn.octree_conv_general(gu.data_cuda(x, node_major), wt, octree, d, cout, ks, stride,
                                        nempty, deconv)
      assert got.shape == (1, cout, want.shape[1], 1), (d, got.shape, want.shape)
      assert gu.rel_err(gu.to_np(got), want) < FP32_TOL, (d, node_major)
  # the reference-named entry points
  d = 4
  x = rng.uniform(-1, 1, size=(cin, bottom_height(v, d, stride, nempty, deconv))).astype(np.float32)
  w = rng.normal(scale=0.2, size=weight_shape(cin, cout, kd, deconv)).astype(np.float32)
  fn = ocnn.nn.octree_deconv if deconv else ocnn.nn.octree_conv
  got = fn(gu.data_cuda(x), torch.from_numpy(w).cuda(), octree, d, cout, ks, stride, nempty)
  want = oc.octree_conv_general(x, w, merged, d, cout, ks, stride, nempty, deconv)
  assert gu.rel_err(gu.to_np(got), want) < FP32_TOL


TC_GENERAL = [
    # (depth, cin, cout, kernel, stride, nempty, deconv)
    (5, 16, 32, [2, 2, 2], 2, False, False),    # folded: one row of 8*Cin channels per sibling group
    (5, 32, 64, [2, 2, 2], 2, True, False),     # the U-Net's down-sampling layer
    (4, 64, 64, [2, 2, 2], 2, True, False),
    (5, 24, 40, [2, 2, 2], 2, True, False),
    (4, 32, 32, [2, 2, 2], 2, False, True),     # expanded: 8*Cout columns per parent, dense rows
    (4, 64, 32, [2, 2, 2], 2, True, True),      # the U-Net's up-sampling layer: scattered rows
    (3, 256, 256, [2, 2, 2], 2, True, True),    # 2048 columns in 8 slices
    (4, 32, 96, [2, 2, 2], 2, True, True),
    (4, 16, 24, [2, 2, 2], 2, True, True),      # 8*24 = 192 columns in one launch
    (4, 16, 40, [2, 2, 2], 2, True, True),      # 8*40 = 320 is no multiple of 256: gather form
    (5, 16, 16, [3, 3, 3], 1, False, True),     # deconvolution through the mirrored taps
    (4, 64, 64, [3, 3, 3], 1, True, True),
    (5, 32, 16, [3, 1, 1], 1, True, True),
    (4, 32, 32, [3, 3, 3], 2, False, True),     # stride-2 deconvolution in gather form
    (4, 64, 32, [3, 3, 3], 2, True, True),
    (4, 16, 32, [3, 3, 1], 2, True, True),
    (5, 32, 32, [3, 3, 3], 2, True, False),     # stride-2 convolution on non-empty nodes
    (5, 64, 32, [3, 3, 1], 2, True, False),
    (5, 16, 8, [1, 1, 1], 2, True, True),
    (5, 16, 8, [1, 1, 1], 2, False, False),
]


@pytest.mark.parametrize('half', [False, True], ids=['bf16', 'fp16'])
@pytest.mark.parametrize('case', TC_GENERAL, ids=lambda c: 'd%d_%dto%d_k%s_s%d_n%d_t%d' % (
    c[0], c[1], c[2], ''.join(map(str, c[3])), c[4], c[5], c[6]))
def test_conv_general_tensor_core(ocnn, batch, case, half):
  merged, octree, v = batch
  d, cin, cout, ks, stride, nempty, deconv = case
  rng = np.random.default_rng(cin * 1000 + cout + stride + 7 * nempty + 13 * deconv)
  kd = int(np.prod(ks))
  rnd = gu.half_round if half else gu.bf16_round
  x = rnd(rng.uniform(-1, 1, size=(cin, bottom_height(v, d, stride, nempty, deconv))).astype(np.float32))
  w = rng.normal(scale=0.1, size=weight_shape(cin, cout, kd, deconv)).astype(np.float32)
  wt = torch.from_numpy(w).cuda()
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights_general(wt, cin, cout, ks, stride, deconv, nempty, half)
  got = ocnn.nn.octree_conv_tc_general(gu.data_cuda(x, True, not half, half), packed, octree, d, cout,
                                       ks, stride, nempty, deconv, None, None, None, False, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0, 'kernel gave up on a wait (code %d)' % int(status.item())
  want = oc.octree_conv_general(x, w, merged, d, cout, ks, stride, nempty, deconv)
  assert got.shape == (1, cout, want.shape[1], 1)
  assert got.dtype == (torch.float16 if half else torch.bfloat16)
  assert gu.rel_err(gu.to_np(got), want) < HALF_TOL
  tight = oc.octree_conv_general(x, rnd(w), merged, d, cout, ks, stride, nempty, deconv)
  assert gu.rel_err(gu.to_np(got), tight) < 6e-3
  # the CUDA-core kernel on the same 16-bit data
  simt = ocnn.nn.octree_conv_general(gu.data_cuda(x, True, not half, half), wt, octree, d, cout, ks,
                                     stride, nempty, deconv)
  assert gu.rel_err(gu.to_np(simt), want) < 6e-3


def test_deconv_tensor_core_epilogue(ocnn, batch):
  """Scale / bias / ReLU in the epilogue of the scattered up-sampling layer."""
  merged, octree, v = batch
  rng = np.random.default_rng(5)
  d, cin, cout, ks = 4, 32, 32, [2, 2, 2]
  x = gu.bf16_round(rng.uniform(-1, 1, size=(cin, int(v.nnum_nempty[d]))).astype(np.float32))
  w = rng.normal(scale=0.1, size=(cin, cout * 8)).astype(np.float32)
  scale = rng.uniform(0.5, 1.5, size=cout).astype(np.float32)
  bias = rng.normal(size=cout).astype(np.float32)
  ref = oc.octree_conv_general(x, gu.bf16_round(w), merged, d, cout, ks, 2, True, True)
  want = np.maximum(ref * scale[:, None] + bias[:, None], 0)
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights_general(torch.from_numpy(w).cuda(), cin, cout, ks, 2, True, True)
  got = ocnn.nn.octree_conv_tc_general(gu.data_cuda(x, True, True), packed, octree, d, cout, ks, 2, True,
                                       True, torch.from_numpy(scale).cuda(), torch.from_numpy(bias).cuda(),
                                       None, True, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  assert gu.rel_err(gu.to_np(got), want) < 8e-3


@pytest.mark.parametrize('ks', KERNELS, ids=lambda k: ''.join(map(str, k)))
@pytest.mark.parametrize('stride', [1, 2])
def test_octree2col_nempty_and_col2octree(ocnn, batch, ks, stride):
  merged, octree, v = batch
  rng = np.random.default_rng(31 + sum(ks) + stride)
  d = 5
  H, nne = int(v.nnum[d]), int(v.nnum_nempty[d])
  neigh, child = v.prop('neigh', d), v.prop('child', d)
  kd = int(np.prod(ks))
  hc = nne if stride == 1 else H // 8
  x = rng.uniform(-1, 1, size=(3, nne)).astype(np.float32)
  got = ocnn.nn.octree2col(gu.data_cuda(x), octree, d, ks, stride, True)
  assert np.array_equal(got.cpu().numpy(), oc.octree2col_general(x, neigh, ks, stride, hc, child))
  # octree2colP = octree2col of the padded data, depadded (pytorch/test/test_octree2col.py:99-132)
  dense = ocnn.nn.octree2col(ocnn.nn.octree_pad(gu.data_cuda(x), octree, d, 0.0), octree, d, ks, stride, False)
  if stride == 1:
    dense = ocnn.nn.octree_depad(dense.view(1, 3 * kd, H, 1), octree, d).view(3, kd, nne)
  assert torch.equal(got, dense)
  for nempty in (False, True):
    h_col = (nne if nempty else H) if stride == 1 else H // 8
    col = rng.uniform(-1, 1, size=(3, kd, h_col)).astype(np.float32)
    back = ocnn.nn.col2octree(torch.from_numpy(col).cuda(), octree, d, ks, stride, nempty)
    want = oc.col2octree_general(col, neigh, ks, stride, nne if nempty else H, child if nempty else None)
    assert back.shape == (1, 3, want.shape[1], 1)
    assert np.allclose(gu.to_np(back), want, atol=1e-5)


@pytest.mark.parametrize('ks', KERNELS, ids=lambda k: ''.join(map(str, k)))
@pytest.mark.parametrize('stride', [1, 2])
def test_deconv_modules(ocnn, batch, ks, stride):
  """The reference's own check (pytorch/test/test_octree_deconv.py): OctreeDeconv against
  OctreeDeconvFast (dense product + col2octree), and nempty=True against the dense layer on masked
  data read back at the non-empty nodes."""
  merged, octree, v = batch
  torch.manual_seed(3)
  d, cin, cout = 4, 3, 5
  H = int(v.nnum[d])
  data = torch.rand(1, cin, H, 1, device='cuda') * 2 - 1
  conv1 = ocnn.OctreeDeconv(d, cin, cout, ks, stride).cuda()
  conv2 = ocnn.OctreeDeconvFast(d, cin, cout, ks, stride).cuda()
  conv3 = ocnn.OctreeDeconv(d, cin, cout, ks, stride, True).cuda()
  with torch.no_grad():
    conv2.weights.copy_(conv1.weights)
    conv3.weights.copy_(conv1.weights)
  out1, out2 = conv1(data, octree), conv2(data, octree)
  assert torch.allclose(out1, out2, atol=1e-5)
  mask3 = ocnn.octree_property(octree, 'child', d) >= 0
  out3 = conv3(data[:, :, mask3].contiguous(), octree)
  d_out = d if stride == 1 else d + 1
  mask4 = ocnn.octree_property(octree, 'child', d_out) >= 0
  out4 = conv1(data * mask3.view(1, 1, -1, 1).float(), octree)[:, :, mask4]
  assert torch.allclose(out3, out4, atol=1e-5)


# ---- fp16 through the bandwidth kernels and the pointwise kernel ----------------------------------------
@pytest.mark.parametrize('layout', ['channel_major', 'node_major'])
def test_fp16_pad_depad_pool_tile(ocnn, batch, layout):
  merged, octree, v = batch
  rng = np.random.default_rng(9)
  d, C = 5, 16
  H, Hne = int(v.nnum[d]), int(v.nnum_nempty[d])
  child = v.prop('child', d)
  nm = layout == 'node_major'
  x = gu.half_round(rng.uniform(-1, 1, size=(C, H)).astype(np.float32))
  xne = gu.half_round(rng.uniform(-1, 1, size=(C, Hne)).astype(np.float32))
  got = ocnn.nn.octree_pad(gu.data_cuda(xne, nm, half=True), octree, d, 0.25)
  assert got.dtype == torch.float16 and np.array_equal(gu.to_np(got), oc.pad(xne, child, 0.25))
  got = ocnn.nn.octree_depad(gu.data_cuda(x, nm, half=True), octree, d)
  assert np.array_equal(gu.to_np(got), oc.depad(x, child, Hne))
  top, mask = ocnn.nn.octree_max_pool(gu.data_cuda(x, nm, half=True), octree, d)
  wtop, wmask = oc.max_pool(x)
  assert np.array_equal(gu.to_np(top), wtop)
  assert np.array_equal(mask.contiguous().view(C, -1).cpu().numpy(), wmask)
  tile = ocnn.nn.octree_tile(gu.data_cuda(x, nm, half=True), octree, d)
  assert np.array_equal(gu.to_np(tile), np.repeat(oc.depad(x, child, Hne), 8, axis=1))
  if nm:
    fused = ocnn.nn.octree_max_pool_pad(gu.data_cuda(x, True, half=True), octree, d)
    assert np.array_equal(gu.to_np(fused), oc.pad(wtop, v.prop('child', d - 1), 0.0))


@pytest.mark.parametrize('shape', [(6, 32, 8), (5, 16, 64), (4, 24, 16)])
def test_fp16_pointwise_and_feature(ocnn, batch, shape):
  merged, octree, v = batch
  d, cin, cout = shape
  rng = np.random.default_rng(cin + cout)
  H = int(v.nnum[d])
  x = gu.half_round(rng.uniform(-1, 1, size=(cin, H)).astype(np.float32))
  w = rng.normal(scale=0.2, size=(cout, cin)).astype(np.float32)
  res = gu.half_round(rng.normal(size=(cout, H)).astype(np.float32))
  got = ocnn.nn.pointwise_conv(gu.data_cuda(x, True, half=True), torch.from_numpy(w).cuda(), None, None,
                               gu.data_cuda(res, True, half=True), True)
  want = np.maximum(w @ x + res, 0)
  assert got.dtype == torch.float16 and gu.rel_err(gu.to_np(got), want) < 4e-3
  feat = ocnn.nn.feature_node_major(octree, 8, False, True)
  assert feat.dtype == torch.float16
  f = v.prop('feature', 6)
  assert np.array_equal(gu.to_np(feat)[:f.shape[0]], gu.half_round(f))
