"""GPU parity tests of the octree convolution against the CPU oracle.
Tolerances (max |y - y_ref| / max |y_ref| per tensor): 1e-5 for fp32, 2e-2 for bf16 data."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import oracle as oc

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
BF16_TOL = 2e-2
KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [1, 3, 1], [1, 1, 3], [3, 3, 1], [3, 1, 3], [1, 3, 3],
           [1, 1, 1]]


@pytest.fixture(scope='module')
def ocnn():
  import ocnn as mod
  return mod


@pytest.fixture(scope='module')
def batch():
  clouds = gu.small_clouds(3, 4000, 200)
  singles, merged, _ = gu.oracle_batch(clouds, 6, 2, 64)
  return merged, gu.to_cuda_u8(merged), oc.OctreeView(merged)


def test_conv_matches_reference_fixture(ocnn, golden):
  """Every kernel shape and stride against outputs of the reference's own CPU convolution."""
  merged = golden['k32_b_merged']
  octree = gu.to_cuda_u8(merged)
  for ks in KERNELS:
    name = ''.join(map(str, ks))
    w = torch.from_numpy(golden['b_w' + name]).cuda()
    for stride in (1, 2):
      got = ocnn.octree_conv(gu.data_cuda(golden['b_x']), w, octree, 4, 5, ks, stride)
      want = golden['b_conv%s_s%d' % (name, stride)]
      assert gu.rel_err(gu.to_np(got), want) < FP32_TOL, (ks, stride)


def test_conv_equals_octree2col_mm(ocnn, golden):
  # pytorch/test/test_octree_conv.py:10-82 (forward): OctreeConv vs OctreeConvFast on
  # octree_1 + octree_2, depth 4, 3 -> 5 channels
  octree = ocnn.octree_batch([torch.from_numpy(golden['k64_octree_1']),
                              torch.from_numpy(golden['k64_octree_2'])])
  rng = np.random.default_rng(2)
  data = gu.data_cuda(rng.uniform(-1, 1, size=(3, 152)).astype(np.float32))
  for stride in (1, 2):
    for ks in ([3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]):
      conv1 = ocnn.OctreeConv(4, 3, 5, ks, stride).cuda()
      conv2 = ocnn.OctreeConvFast(4, 3, 5, ks, stride).cuda()
      with torch.no_grad():
        conv2.weights.copy_(conv1.weights)
      out1, out2 = conv1(data, octree), conv2(data, octree)
      # stride 2 is padded to every node of depth 3 by the module (octree_conv.py:111-112)
      h3 = ocnn.octree_property(octree, 'node_num', 3).item()
      assert out1.shape == out2.shape == (1, 5, 152 if stride == 1 else h3, 1)
      assert gu.rel_err(gu.to_np(out1), gu.to_np(out2)) < FP32_TOL, (ks, stride)


@pytest.mark.parametrize('ks', KERNELS)
@pytest.mark.parametrize('stride', [1, 2])
def test_conv_fp32_channel_major(ocnn, batch, ks, stride):
  merged, octree, v = batch
  rng = np.random.default_rng(sum(ks) + 10 * stride)
  for d, cin, cout in ((6, 3, 32), (5, 16, 24), (3, 70, 65)):
    H = int(v.nnum[d])
    x = rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)
    w = rng.normal(scale=0.1, size=(cout, cin * int(np.prod(ks)))).astype(np.float32)
    got = ocnn.octree_conv(gu.data_cuda(x), torch.from_numpy(w).cuda(), octree, d, cout, ks, stride)
    want = oc.octree_conv(x, w, merged, d, cout, ks, stride)
    assert got.shape == (1, cout, want.shape[1], 1)
    assert gu.rel_err(gu.to_np(got), want) < FP32_TOL, (d, cin, cout)


@pytest.mark.parametrize('bf16', [False, True])
def test_conv_node_major(ocnn, batch, bf16):
  merged, octree, v = batch
  rng = np.random.default_rng(77)
  for ks, stride in (([3, 3, 3], 1), ([3, 3, 3], 2), ([2, 2, 2], 2), ([1, 1, 1], 1), ([3, 1, 3], 1)):
    for d, cin, cout in ((6, 8, 16), (5, 32, 64), (4, 3, 7)):
      H = int(v.nnum[d])
      x = rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)
      w = rng.normal(scale=0.1, size=(cout, cin * int(np.prod(ks)))).astype(np.float32)
      if bf16:
        x = gu.bf16_round(x)
      got = ocnn.octree_conv(gu.data_cuda(x, True, bf16), torch.from_numpy(w).cuda(), octree, d,
                             cout, ks, stride)
      assert got.is_contiguous(memory_format=torch.channels_last) or cout == 1
      want = oc.octree_conv(x, w, merged, d, cout, ks, stride)
      tol = BF16_TOL if bf16 else FP32_TOL
      assert gu.rel_err(gu.to_np(got), want) < tol, (ks, stride, d)


def test_conv_fused_epilogue(ocnn, batch):
  merged, octree, v = batch
  rng = np.random.default_rng(5)
  d, cin, cout, ks = 5, 16, 32, [3, 3, 3]
  H = int(v.nnum[d])
  x = rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)
  w = rng.normal(scale=0.1, size=(cout, cin * 27)).astype(np.float32)
  scale = rng.uniform(0.5, 1.5, size=cout).astype(np.float32)
  bias = rng.normal(size=cout).astype(np.float32)
  res = rng.normal(size=(cout, H)).astype(np.float32)
  ref = oc.octree_conv(x, w, merged, d, cout, ks, 1)
  want = np.maximum(ref * scale[:, None] + bias[:, None] + res, 0)
  for nm in (False, True):
    got = ocnn.nn.octree_conv_fused(gu.data_cuda(x, nm), torch.from_numpy(w).cuda(), octree, d, cout,
                                    ks, 1, torch.from_numpy(scale).cuda(),
                                    torch.from_numpy(bias).cuda(), gu.data_cuda(res, nm), True)
    assert gu.rel_err(gu.to_np(got), want) < FP32_TOL


def test_conv_errors(ocnn, batch):
  _, octree, v = batch
  w = torch.zeros(4, 3 * 27, device='cuda')
  with pytest.raises(RuntimeError, match='data height'):
    ocnn.octree_conv(torch.zeros(1, 3, 10, 1, device='cuda'), w, octree, 5, 4, [3], 1)
  with pytest.raises(RuntimeError, match='[Kk]ernel size'):
    ocnn.octree_conv(torch.zeros(1, 3, int(v.nnum[5]), 1, device='cuda'), w, octree, 5, 4, [4], 1)
  with pytest.raises(RuntimeError, match='stride'):
    ocnn.octree_conv(torch.zeros(1, 3, int(v.nnum[5]), 1, device='cuda'), w, octree, 5, 4, [3], 3)
  with pytest.raises(RuntimeError, match='data height'):    # nempty: rows = non-empty nodes
    ocnn.octree_conv(torch.zeros(1, 3, int(v.nnum[5]), 1, device='cuda'), w, octree, 5, 4, [3], 2, True)


# ---- tensor-core (tcgen05) path -----------------------------------------------------------------
TC_CASES = [
    # (depth, cin, cout, kernel, stride)
    (6, 8, 8, [3, 3, 3], 1),       # ResNet d6 bottleneck: Cout padded to the UMMA minimum of 16
    (6, 8, 32, [3, 3, 3], 1),      # conv1 with the 3 normal channels padded to 8
    (5, 16, 16, [3, 3, 3], 1),
    (4, 32, 32, [3, 3, 3], 1),
    (3, 64, 64, [3, 3, 3], 1),
    (2, 128, 128, [3, 3, 3], 1),
    (3, 64, 256, [3, 3, 3], 1),
    (2, 128, 512, [1, 1, 1], 1),   # 512 output channels: two launches of 256
    (2, 16, 512, [3, 3, 3], 1),
    (5, 24, 40, [3, 3, 3], 1),     # K = 27*24 is not a multiple of 64; Cout not a multiple of 16
    (6, 32, 8, [1, 1, 1], 1),      # the 1x1 convolutions of the bottleneck blocks
    (5, 16, 64, [1, 1, 1], 1),
    (3, 256, 64, [1, 1, 1], 1),
    (5, 16, 32, [2, 2, 2], 2),
    (5, 16, 32, [3, 3, 3], 2),
    (4, 32, 16, [3, 1, 3], 1),
    (5, 24, 8, [3, 3, 3], 1),      # sibling-group mode with 3 chunks per neighbour row
    (6, 8, 16, [2, 2, 2], 1),
    (5, 32, 32, [1, 3, 3], 1),
    (3, 192, 64, [3, 3, 3], 1),    # Cin a multiple of 64 but not a power of two
    (4, 64, 32, [3, 3, 3], 2),     # stride 2 with whole-row gathers
    (4, 64, 48, [2, 2, 2], 2),
    (3, 128, 128, [1, 1, 1], 1),
    (4, 320, 16, [1, 1, 1], 1),
    # sibling-product mode (full 3x3x3 kernel, weight set resident in shared memory), every channel
    # family, on levels from a single tile to many tiles per CTA
    (6, 8, 16, [3, 3, 3], 1),
    (2, 8, 32, [3, 3, 3], 1),
    (6, 16, 32, [3, 3, 3], 1),
    (3, 16, 16, [3, 3, 3], 1),
    (6, 16, 64, [3, 3, 3], 1),
    (6, 32, 32, [3, 3, 3], 1),
    (5, 32, 64, [3, 3, 3], 1),
    (6, 64, 32, [3, 3, 3], 1),
    (4, 64, 16, [3, 3, 3], 1),
    (6, 8, 64, [3, 3, 3], 1),
]


@pytest.mark.parametrize('case', TC_CASES, ids=lambda c: 'd%d_%dto%d_k%s_s%d' % (
    c[0], c[1], c[2], ''.join(map(str, c[3])), c[4]))
def test_conv_tensor_core(ocnn, batch, case):
  merged, octree, v = batch
  d, cin, cout, ks, stride = case
  rng = np.random.default_rng(cin * 1000 + cout + stride)
  H = int(v.nnum[d])
  x = gu.bf16_round(rng.uniform(-1, 1, size=(cin, H)).astype(np.float32))
  w = rng.normal(scale=0.1, size=(cout, cin * int(np.prod(ks)))).astype(np.float32)
  wt = torch.from_numpy(w).cuda()
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights(wt, cin, cout, ks, stride)
  got = ocnn.nn.octree_conv_tc(gu.data_cuda(x, True, True), packed, octree, d, cout, ks, stride,
                               None, None, None, False, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0, 'kernel gave up on a wait (code %d)' % int(status.item())
  want = oc.octree_conv(x, w, merged, d, cout, ks, stride)
  assert got.shape == (1, cout, want.shape[1], 1)
  assert gu.rel_err(gu.to_np(got), want) < BF16_TOL
  # against bf16-rounded weights only the accumulation order and the output rounding differ
  tight = oc.octree_conv(x, gu.bf16_round(w), merged, d, cout, ks, stride)
  assert gu.rel_err(gu.to_np(got), tight) < 6e-3


def test_conv_tensor_core_epilogue(ocnn, batch):
  merged, octree, v = batch
  rng = np.random.default_rng(12)
  d, cin, cout, ks = 5, 16, 32, [3, 3, 3]
  H = int(v.nnum[d])
  x = gu.bf16_round(rng.uniform(-1, 1, size=(cin, H)).astype(np.float32))
  w = rng.normal(scale=0.1, size=(cout, cin * 27)).astype(np.float32)
  scale = rng.uniform(0.5, 1.5, size=cout).astype(np.float32)
  bias = rng.normal(size=cout).astype(np.float32)
  res = gu.bf16_round(rng.normal(size=(cout, H)).astype(np.float32))
  ref = oc.octree_conv(x, gu.bf16_round(w), merged, d, cout, ks, 1)
  want = np.maximum(ref * scale[:, None] + bias[:, None] + res, 0)
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights(torch.from_numpy(w).cuda(), cin, cout, ks)
  got = ocnn.nn.octree_conv_tc(gu.data_cuda(x, True, True), packed, octree, d, cout, ks, 1,
                               torch.from_numpy(scale).cuda(), torch.from_numpy(bias).cuda(),
                               gu.data_cuda(res, True, True), True, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  assert gu.rel_err(gu.to_np(got), want) < 8e-3


@pytest.mark.parametrize('half', [False, True], ids=['bf16', 'fp16'])
@pytest.mark.parametrize('shape', [(1001, 8, 32), (1003, 16, 64), (77, 32, 8), (5, 8, 8), (2048, 32, 16),
                                   (300007, 8, 32), (300001, 32, 8)])
def test_pointwise_tensor_core_any_height(ocnn, shape, half):
  """1x1x1 layers with fewer than 64 input channels run on rows of 64/Cin nodes; a node count that
  does not fill the last row (data on non-empty nodes) is finished by a separate small launch."""
  H, cin, cout = shape
  rng = np.random.default_rng(H + cin)
  rnd = gu.half_round if half else gu.bf16_round
  x = rnd(rng.uniform(-1, 1, size=(cin, H)).astype(np.float32))
  w = rng.normal(scale=0.2, size=(cout, cin)).astype(np.float32)
  scale = rng.uniform(0.5, 1.5, size=cout).astype(np.float32)
  bias = rng.normal(size=cout).astype(np.float32)
  res = rnd(rng.normal(size=(cout, H)).astype(np.float32))
  want = np.maximum((rnd(w) @ x) * scale[:, None] + bias[:, None] + res, 0)
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights_general(torch.from_numpy(w).cuda(), cin, cout, [1, 1, 1], 1, False,
                                             False, half)
  got = ocnn.nn.pointwise_conv_tc(gu.data_cuda(x, True, not half, half), packed, cout,
                                  torch.from_numpy(scale).cuda(), torch.from_numpy(bias).cuda(),
                                  gu.data_cuda(res, True, not half, half), True, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  assert got.shape == (1, cout, H, 1)
  assert gu.rel_err(gu.to_np(got), want) < (3e-3 if half else 8e-3)


@pytest.mark.parametrize('half', [False, True], ids=['bf16', 'fp16'])
@pytest.mark.parametrize('shape', [(1001, 16, 32, 64), (50003, 32, 64, 128), (4099, 64, 128, 256),
                                   (2048, 128, 256, 512), (37, 8, 40, 24), (260000, 16, 32, 64),
                                   (130001, 64, 128, 256)])
def test_pointwise_pair_is_the_sum_of_two_layers(ocnn, shape, half):
  """conv1x1b(y) + conv1x1c(x) of a residual block as one layer over the concatenated channels
  (pytorch/ocnn/modules.py OctreeResBlock.forward computes the two and adds them)."""
  H, ca, cb, cout = shape
  rng = np.random.default_rng(H + ca)
  rnd = gu.half_round if half else gu.bf16_round
  xa = rnd(rng.uniform(-1, 1, size=(ca, H)).astype(np.float32))
  xb = rnd(rng.uniform(-1, 1, size=(cb, H)).astype(np.float32))
  wa = rng.normal(scale=0.2, size=(cout, ca)).astype(np.float32)
  wb = rng.normal(scale=0.2, size=(cout, cb)).astype(np.float32)
  bias = rng.normal(size=cout).astype(np.float32)
  want = np.maximum(rnd(wa) @ xa + rnd(wb) @ xb + bias[:, None], 0)
  w = np.ascontiguousarray(np.concatenate([wa, wb], axis=1))
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights_general(torch.from_numpy(w).cuda(), ca + cb, cout, [1, 1, 1], 1,
                                             False, False, half)
  got = ocnn.nn.pointwise_conv_tc_pair(gu.data_cuda(xa, True, not half, half),
                                       gu.data_cuda(xb, True, not half, half), packed, cout, None,
                                       torch.from_numpy(bias).cuda(), None, True, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  assert got.shape == (1, cout, H, 1)
  assert gu.rel_err(gu.to_np(got), want) < (3e-3 if half else 8e-3)


def test_pointwise_pair_rejects_what_it_cannot_run(ocnn):
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  xa = gu.data_cuda(np.zeros((8, 64), np.float32), True, True)
  xb = gu.data_cuda(np.zeros((8, 64), np.float32), True, True)
  w = torch.zeros(16, 16, device='cuda')
  packed = ocnn.nn.conv_pack_weights(w, 16, 16, [1, 1, 1])
  with pytest.raises(RuntimeError, match='two inputs only'):      # 8 + 8 channels: a folded layer
    ocnn.nn.pointwise_conv_tc_pair(xa, xb, packed, 16, None, None, None, False, status)
  xc = gu.data_cuda(np.zeros((40, 63), np.float32), True, True)
  w = torch.zeros(16, 48, device='cuda')
  packed = ocnn.nn.conv_pack_weights(w, 48, 16, [1, 1, 1])
  with pytest.raises(RuntimeError, match='rows'):
    ocnn.nn.pointwise_conv_tc_pair(xa, xc, packed, 16, None, None, None, False, status)


@pytest.mark.parametrize('half', [False, True], ids=['bf16', 'fp16'])
@pytest.mark.parametrize('shape', [(6, 8, 32), (5, 16, 64), (4, 32, 8), (6, 64, 16), (3, 16, 16)])
def test_conv1x1_max_pool_pad_is_the_two_operators(ocnn, batch, shape, half):
  """A 1x1x1 layer + OctreeMaxPool (pytorch/ocnn/octree_pool.py: octree_max_pool, octree_pad) in one
  pass against the two operators run one after the other on the same 16-bit data."""
  merged, octree, v = batch
  d, cin, cout = shape
  H = int(v.nnum[d])
  rng = np.random.default_rng(d * 100 + cin)
  rnd = gu.half_round if half else gu.bf16_round
  x = gu.data_cuda(rnd(rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)), True, not half, half)
  res = gu.data_cuda(rnd(rng.normal(size=(cout, H)).astype(np.float32)), True, not half, half)
  w = torch.from_numpy(rng.normal(scale=0.3, size=(cout, cin)).astype(np.float32)).cuda()
  scale = torch.from_numpy(rng.uniform(0.5, 1.5, size=cout).astype(np.float32)).cuda()
  bias = torch.from_numpy(rng.normal(size=cout).astype(np.float32)).cuda()
  for relu, r in ((True, res), (False, None)):
    got = ocnn.nn.conv1x1_max_pool_pad(x, w, octree, d, scale, bias, r, relu)
    y = ocnn.nn.octree_conv_fused(x, w, octree, d, cout, [1, 1, 1], 1, scale, bias, r, relu)
    want = ocnn.nn.octree_max_pool_pad(y, octree, d)
    assert got.shape == want.shape == (1, cout, int(v.nnum[d - 1]), 1)
    assert torch.equal(got, want)
  with pytest.raises(RuntimeError, match='channels'):
    ocnn.nn.conv1x1_max_pool_pad(gu.data_cuda(np.zeros((24, H), np.float32), True, True),
                                 torch.zeros(8, 24, device='cuda'), octree, d)


def test_bounded_wait_runs_out_and_reports(ocnn, batch):
  """A wait that nothing completes ends by itself: the waiter writes its code to the status word
  and raises the abort flag, a second waiter is told to stop, the kernel returns, and the next
  convolution on the same context works."""
  merged, octree, v = batch
  st = ocnn.nn.conv_tc_wait_selftest()
  torch.cuda.synchronize()
  code, stopped = st.cpu().tolist()
  assert code in (1, 2) and stopped == 1
  d, cin, cout, ks = 4, 32, 32, [3, 3, 3]
  rng = np.random.default_rng(5)
  x = gu.bf16_round(rng.uniform(-1, 1, size=(cin, int(v.nnum[d]))).astype(np.float32))
  w = rng.normal(scale=0.1, size=(cout, cin * 27)).astype(np.float32)
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights(torch.from_numpy(w).cuda(), cin, cout, ks)
  got = ocnn.nn.octree_conv_tc(gu.data_cuda(x, True, True), packed, octree, d, cout, ks, 1,
                               None, None, None, False, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  assert gu.rel_err(gu.to_np(got), oc.octree_conv(x, w, merged, d, cout, ks, 1)) < BF16_TOL


def test_conv_tensor_core_rejects_unsupported_shapes(ocnn, batch):
  _, octree, v = batch
  w = torch.zeros(16, 3 * 27, device='cuda')
  with pytest.raises(RuntimeError, match='multiple of 8'):
    ocnn.nn.conv_pack_weights(w, 3, 16, [3, 3, 3])
  with pytest.raises(RuntimeError, match='multiple of 256'):
    ocnn.nn.conv_pack_weights(torch.zeros(264, 8, device='cuda'), 8, 264, [1, 1, 1])


# ---- few-channel pointwise (1x1x1) kernel behind octree_conv ---------------------------------------
@pytest.mark.parametrize('shape', [(6, 32, 8), (6, 8, 32), (5, 64, 16), (5, 16, 64), (4, 24, 16),
                                   (3, 128, 32), (6, 256, 64), (5, 8, 8), (5, 16, 16), (5, 32, 16),
                                   (5, 64, 8), (4, 8, 64), (3, 16, 8)])
def test_conv_pointwise_bf16(ocnn, batch, shape):
  merged, octree, v = batch
  d, cin, cout = shape
  rng = np.random.default_rng(cin + 7 * cout)
  H = int(v.nnum[d])
  x = gu.bf16_round(rng.uniform(-1, 1, size=(cin, H)).astype(np.float32))
  w = rng.normal(scale=0.2, size=(cout, cin)).astype(np.float32)
  scale = rng.uniform(0.5, 1.5, size=cout).astype(np.float32)
  bias = rng.normal(size=cout).astype(np.float32)
  res = gu.bf16_round(rng.normal(size=(cout, H)).astype(np.float32))
  got = ocnn.octree_conv(gu.data_cuda(x, True, True), torch.from_numpy(w).cuda(), octree, d, cout,
                         [1], 1)
  ref = w @ x
  assert gu.rel_err(gu.to_np(got), ref) < 6e-3            # only the bf16 rounding of the output
  got = ocnn.nn.octree_conv_fused(gu.data_cuda(x, True, True), torch.from_numpy(w).cuda(), octree,
                                  d, cout, [1, 1, 1], 1, torch.from_numpy(scale).cuda(),
                                  torch.from_numpy(bias).cuda(), gu.data_cuda(res, True, True), True)
  want = np.maximum(ref * scale[:, None] + bias[:, None] + res, 0)
  assert gu.rel_err(gu.to_np(got), want) < 6e-3


# ---- convolution on the non-empty nodes only (nempty=True) ----------------------------------------
@pytest.mark.parametrize('ks', [[3, 3, 3], [3, 1, 1], [2, 2, 2], [1, 1, 1]])
@pytest.mark.parametrize('nm,bf16', [(False, False), (True, False), (True, True)])
def test_conv_nempty(ocnn, batch, ks, nm, bf16):
  """OctreeConv(nempty=True), stride 1, against the oracle's octree2colP-based convolution, and the
  identity the reference's own test relies on (pytorch/test/test_octree_conv.py): it equals the
  dense convolution of the zero-padded data read back at the non-empty nodes."""
  merged, octree, v = batch
  rng = np.random.default_rng(31)
  for d in (5, 3):
    nne = int(v.nnum_nempty[d])
    cin, cout = 6, 10
    x = rng.uniform(-1, 1, size=(cin, nne)).astype(np.float32)
    if bf16:
      x = gu.bf16_round(x)
    w = rng.normal(scale=0.2, size=(cout, cin * int(np.prod(ks)))).astype(np.float32)
    want = oc.octree_conv_nempty(x, w, merged, d, cout, ks)
    wt = torch.from_numpy(w).cuda()
    got = ocnn.octree_conv(gu.data_cuda(x, nm, bf16), wt, octree, d, cout, ks, 1, True)
    assert got.shape == (1, cout, nne, 1)
    assert gu.rel_err(gu.to_np(got), want) < (BF16_TOL if bf16 else 1e-5)
    if not bf16:
      dense = ocnn.octree_conv(ocnn.octree_pad(gu.data_cuda(x, nm, False), octree, d, 0.0), wt,
                               octree, d, cout, ks, 1, False)
      assert np.array_equal(gu.to_np(ocnn.octree_depad(dense, octree, d)), gu.to_np(got))
    mod = ocnn.OctreeConv(d, cin, cout, ks, 1, nempty=True).cuda()
    with torch.no_grad():
      mod.weights.copy_(wt.view_as(mod.weights))
    assert np.array_equal(gu.to_np(mod(gu.data_cuda(x, nm, bf16), octree)), gu.to_np(got))


def test_conv_nempty_errors(ocnn, batch):
  _, octree, v = batch
  w = torch.zeros(4, 3 * 8, device='cuda')
  out = ocnn.octree_conv(torch.zeros(1, 3, int(v.nnum_nempty[4]), 1, device='cuda'), w, octree, 4, 4,
                         [2], 2, True)                      # stride 2 on non-empty nodes
  assert out.shape == (1, 4, int(v.nnum_nempty[3]), 1)
  with pytest.raises(RuntimeError, match='non-empty node number'):
    ocnn.octree_conv(torch.zeros(1, 3, int(v.nnum[4]), 1, device='cuda'),
                     torch.zeros(4, 81, device='cuda'), octree, 4, 4, [3], 1, True)


@pytest.mark.parametrize('case', [(5, 16, 16, [3, 3, 3]), (5, 8, 32, [3, 3, 3]), (4, 64, 64, [3, 3, 3]),
                                  (3, 128, 128, [3, 3, 3]), (4, 24, 40, [3, 3, 3]), (5, 32, 64, [1, 1, 1]),
                                  (4, 32, 16, [3, 1, 3])],
                         ids=lambda c: 'd%d_%dto%d_k%s' % (c[0], c[1], c[2], ''.join(map(str, c[3]))))
def test_conv_tensor_core_nempty(ocnn, batch, case):
  """The tensor-core kernel on the non-empty nodes only, with the fused epilogue, against the
  oracle's octree2colP-based convolution."""
  merged, octree, v = batch
  d, cin, cout, ks = case
  rng = np.random.default_rng(41 + cin + cout)
  nne = int(v.nnum_nempty[d])
  x = gu.bf16_round(rng.uniform(-1, 1, size=(cin, nne)).astype(np.float32))
  w = rng.normal(scale=0.1, size=(cout, cin * int(np.prod(ks)))).astype(np.float32)
  scale = rng.uniform(0.5, 1.5, size=cout).astype(np.float32)
  bias = rng.normal(size=cout).astype(np.float32)
  res = gu.bf16_round(rng.normal(size=(cout, nne)).astype(np.float32))
  wt = torch.from_numpy(w).cuda()
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  packed = ocnn.nn.conv_pack_weights_nempty(wt, cin, cout, ks)
  got = ocnn.nn.octree_conv_tc_nempty(gu.data_cuda(x, True, True), packed, octree, d, cout, ks,
                                      None, None, None, False, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  want = oc.octree_conv_nempty(x, w, merged, d, cout, ks)
  assert got.shape == (1, cout, nne, 1)
  assert gu.rel_err(gu.to_np(got), want) < BF16_TOL
  got = ocnn.nn.octree_conv_tc_nempty(gu.data_cuda(x, True, True), packed, octree, d, cout, ks,
                                      torch.from_numpy(scale).cuda(), torch.from_numpy(bias).cuda(),
                                      gu.data_cuda(res, True, True), True, status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  full = np.maximum(want * scale[:, None] + bias[:, None] + res, 0)
  assert gu.rel_err(gu.to_np(got), full) < BF16_TOL


@pytest.mark.parametrize('half', [False, True], ids=['bf16', 'fp16'])
@pytest.mark.parametrize('triple', [(8, 32, 8), (16, 64, 16), (16, 32, 8), (8, 16, 8)])
def test_conv1x1_chain_is_the_two_layers(ocnn, batch, triple, half):
  """conv1x1b (+ shortcut, ReLU) of one block and conv1x1a of the next in one pass (two consecutive
  OctreeResBlock.forward calls of pytorch/ocnn/modules.py) against the two layers run separately."""
  merged, octree, v = batch
  cin, cmid, cout2 = triple
  d = 6
  H = int(v.nnum[d])
  rng = np.random.default_rng(cin * 7 + cmid)
  rnd = gu.half_round if half else gu.bf16_round
  x = gu.data_cuda(rnd(rng.uniform(-1, 1, size=(cin, H)).astype(np.float32)), True, not half, half)
  res = gu.data_cuda(rnd(rng.normal(size=(cmid, H)).astype(np.float32)), True, not half, half)
  w1 = torch.from_numpy(rng.normal(scale=0.3, size=(cmid, cin)).astype(np.float32)).cuda()
  w2 = torch.from_numpy(rng.normal(scale=0.3, size=(cout2, cmid)).astype(np.float32)).cuda()
  s1 = torch.from_numpy(rng.uniform(0.5, 1.5, size=cmid).astype(np.float32)).cuda()
  b1 = torch.from_numpy(rng.normal(size=cmid).astype(np.float32)).cuda()
  s2 = torch.from_numpy(rng.uniform(0.5, 1.5, size=cout2).astype(np.float32)).cuda()
  b2 = torch.from_numpy(rng.normal(size=cout2).astype(np.float32)).cuda()
  y1, y2 = ocnn.nn.conv1x1_chain(x, w1, s1, b1, res, True, w2, s2, b2, True)
  want1 = ocnn.nn.octree_conv_fused(x, w1, octree, d, cmid, [1, 1, 1], 1, s1, b1, res, True)
  want2 = ocnn.nn.octree_conv_fused(want1, w2, octree, d, cout2, [1, 1, 1], 1, s2, b2, None, True)
  assert torch.equal(y1, want1)
  # the same products summed in another order: equal to fp32 rounding, i.e. at most one 16-bit ulp
  err = float((y2.float() - want2.float()).abs().max()) / max(1.0, float(want2.float().abs().max()))
  assert err < (1e-3 if half else 8e-3)
