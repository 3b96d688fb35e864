"""Gradients of the octree operators (training support): the data gradient of OctreeConv /
OctreeDeconv is the transposed operator, the weight gradient a reduction over the nodes; pooling,
padding, octree2col and octree_align differentiate through their transposes.  Checked against
the CPU oracle and, as the reference's own tests do (pytorch/test/test_octree_conv.py,
test_octree_deconv.py, test_octree_pool.py), against the column-matrix formulation under autograd."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import oracle as oc

pytestmark = pytest.mark.gpu
KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]]


@pytest.fixture(scope='module')
def ocnn():
  import ocnn as mod
  mod.set_key_bits(64)
  return mod


@pytest.fixture(scope='module')
def batch():
  clouds = gu.small_clouds(3, 3000, 500)
  singles, merged, _ = gu.oracle_batch(clouds, 5, 2, 64)
  return merged, gu.to_cuda_u8(merged), oc.OctreeView(merged)


def heights(v, d, stride, nempty, deconv):
  h_in = int(v.nnum_nempty[d]) if (nempty or (deconv and stride == 2)) else int(v.nnum[d])
  return h_in


@pytest.mark.parametrize('ks', KERNELS, ids=lambda k: ''.join(map(str, k)))
@pytest.mark.parametrize('stride', [1, 2])
@pytest.mark.parametrize('nempty', [False, True])
@pytest.mark.parametrize('deconv', [False, True])
def test_conv_gradients_vs_oracle(ocnn, batch, ks, stride, nempty, deconv):
  merged, octree, v = batch
  rng = np.random.default_rng(sum(ks) + 10 * stride + 3 * nempty + 5 * deconv)
  d, cin, cout, kd = 4, 4, 6, int(np.prod(ks))
  x = rng.uniform(-1, 1, size=(cin, heights(v, d, stride, nempty, deconv))).astype(np.float32)
  w = rng.normal(scale=0.3, size=(cin, cout * kd) if deconv else (cout, cin * kd)).astype(np.float32)
  y = oc.octree_conv_general(x, w, merged, d, cout, ks, stride, nempty, deconv)
  g = rng.uniform(-1, 1, size=y.shape).astype(np.float32)
  # data gradient = the transposed operator with the same weights, from the output level back
  back_depth = d if stride == 1 else (d + 1 if deconv else d - 1)
  want_gx = oc.octree_conv_general(g, w, merged, back_depth, cin, ks, stride, nempty, not deconv)
  # weight gradient by finite structure: dL/dW = sum over outputs, via the linear map y(W)
  # (y is linear in W: probe with the basis would be slow; use the column formulation instead)
  work_d = d + 1 if (deconv and stride == 2) else d
  neigh = v.prop('neigh', work_d)
  child = v.prop('child', work_d) if nempty else None
  src, a = (g, x) if deconv else (x, g)
  h_col = a.shape[1]
  if kd == 1 and stride == 1:
    col = src[:, None, :]
  else:
    col = oc.octree2col_general(src, neigh, ks, stride, h_col, child)
  want_gw = a @ col.reshape(-1, h_col).T
  fn = ocnn.nn.octree_deconv_grad if deconv else ocnn.nn.octree_conv_grad
  for nm in (False, True):
    gx, gw = fn(gu.data_cuda(x, nm), torch.from_numpy(w).cuda(), octree, gu.data_cuda(g, nm), d, cout, ks,
                stride, nempty)
    assert gu.rel_err(gu.to_np(gx), want_gx) < 1e-5
    assert gw.shape == w.shape and gu.rel_err(gw.cpu().numpy(), want_gw) < 2e-5


@pytest.mark.parametrize('stride', [1, 2])
@pytest.mark.parametrize('deconv', [False, True])
def test_module_gradients_match_column_formulation(ocnn, batch, stride, deconv):
  merged, octree, v = batch
  torch.manual_seed(4)
  d, cin, cout, ks = 4, 3, 5, [3, 3, 3]
  data = torch.rand(1, cin, int(v.nnum[d]), 1, device='cuda')
  fast = (ocnn.OctreeDeconvFast if deconv else ocnn.OctreeConvFast)(d, cin, cout, ks, stride).cuda()
  conv = (ocnn.OctreeDeconv if deconv else ocnn.OctreeConv)(d, cin, cout, ks, stride).cuda()
  with torch.no_grad():
    fast.weights.copy_(conv.weights)
  d1 = data.clone().requires_grad_()
  d2 = data.clone().requires_grad_()
  out1, out2 = conv(d1, octree), fast(d2, octree)
  assert torch.allclose(out1, out2, atol=1e-5)
  g = torch.rand_like(out1)
  out1.backward(g)
  out2.backward(g)
  assert torch.allclose(d1.grad, d2.grad, atol=1e-5)
  assert torch.allclose(conv.weights.grad, fast.weights.grad, atol=1e-4)


def test_pool_pad_align_gradients(ocnn, batch):
  merged, octree, v = batch
  torch.manual_seed(6)
  d, C = 4, 5
  H, Hne = int(v.nnum[d]), int(v.nnum_nempty[d])
  x = torch.rand(1, C, H, 1, device='cuda', requires_grad=True)
  pooled, mask = ocnn.octree_max_pool(x, octree, d)
  g = torch.rand_like(pooled)
  pooled.backward(g)
  want = np.zeros((C, H), np.float32)
  m = mask.view(C, -1).cpu().numpy()
  for c in range(C):
    want[c, m[c]] = g.view(C, -1).cpu().numpy()[c]
  assert np.array_equal(gu.to_np(x.grad), want)
  assert torch.equal(ocnn.octree_mask_pool(x.detach(), mask, octree, d), pooled.detach())
  up = ocnn.octree_max_unpool(pooled.detach(), mask, octree, d)
  assert torch.equal(up, torch.from_numpy(np.where(want != 0, gu.to_np(x.detach()), 0)).cuda().view(1, C, H, 1)
                     * 0 + up)          # shape / dtype
  assert np.array_equal(gu.to_np(up)[want != 0], gu.to_np(x.detach())[want != 0])
  # pad / depad are each other's transposes
  xs = torch.rand(1, C, Hne, 1, device='cuda', requires_grad=True)
  y = ocnn.octree_pad(xs, octree, d)
  gy = torch.rand_like(y)
  y.backward(gy)
  assert torch.equal(xs.grad, ocnn.octree_depad(gy, octree, d))
  xf = torch.rand(1, C, H, 1, device='cuda', requires_grad=True)
  z = ocnn.octree_depad(xf, octree, d)
  gz = torch.rand_like(z)
  z.backward(gz)
  assert torch.equal(xf.grad, ocnn.octree_pad(gz, octree, d))
  # align
  xa = torch.rand(1, C, H, 1, device='cuda', requires_grad=True)
  out, idx = ocnn.octree_align(xa, octree, octree, d)
  out.sum().backward()
  assert torch.equal(out, xa) and torch.equal(xa.grad, torch.ones_like(xa))


def test_training_step_runs(ocnn, batch):
  """One optimisation step of a small residual network assembled from the modules."""
  merged, octree, v = batch
  torch.manual_seed(8)
  d = 5
  blocks = ocnn.OctreeResBlocks(d, 3, 16, 1, bottleneck=1, resblk=ocnn.OctreeResBlock2).cuda().train()
  pool = ocnn.OctreeMaxPool(d)
  head = ocnn.OctreeConv1x1(16, 4, use_bias=True).cuda().train()
  opt = torch.optim.SGD(list(blocks.parameters()) + list(head.parameters()), lr=0.05)
  data = ocnn.octree_property(octree, 'feature', d)
  losses = []
  for _ in range(3):
    opt.zero_grad()
    out = head(pool(blocks(data, octree), octree))
    loss = (out ** 2).mean()
    loss.backward()
    opt.step()
    losses.append(float(loss))
  assert all(np.isfinite(losses)) and losses[-1] < losses[0]
