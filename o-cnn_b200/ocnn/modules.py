"""Building blocks of the reference's networks (pytorch/ocnn/modules.py:1-345), forward only:
convolution + BatchNorm (+ ReLU) blocks, 1x1 blocks, the two residual blocks, nearest /
trilinear interpolation at points, and `octree_feature`.  Class names, constructor arguments and
parameter names follow the reference, so its state_dicts load.

In eval mode a block folds its BatchNorm (running statistics) and ReLU into the convolution
kernel's epilogue — one launch per block instead of three; set `FUSE_EVAL_BN = False` to run the
torch BatchNorm / ReLU modules after the convolution instead.  In training mode the torch modules
always run (the convolution itself has no backward here).
"""
import torch
from torch import nn as _nn

from . import nn
from .octree_conv import OctreeConv, OctreeDeconv, tc_status, _tensor_core_ready
from .octree_pool import OctreeMaxPool
from .octree_pad import OctreeTile  # noqa: F401  (re-exported: the reference defines it here)

bn_momentum, bn_eps = 0.01, 0.001       # pytorch/ocnn/modules.py:5
FUSE_EVAL_BN = True


def _folded(bn):
  """(scale, bias) float32 vectors equal to an eval-mode BatchNorm."""
  with torch.no_grad():
    scale = bn.weight.float() / torch.sqrt(bn.running_var.float() + bn.eps)
    bias = bn.bias.float() - bn.running_mean.float() * scale
  return scale.contiguous(), bias.contiguous()


class _OctreeBlock(_nn.Module):
  """An octree (de)convolution followed by BatchNorm2d and optionally ReLU."""
  layer, attr, with_relu = OctreeConv, 'conv', True

  def __init__(self, depth, channel_in, channel_out, kernel_size=[3], stride=1, nempty=False):
    super().__init__()
    setattr(self, self.attr, self.layer(depth, channel_in, channel_out, kernel_size, stride, nempty))
    self.bn = _nn.BatchNorm2d(channel_out, bn_eps, bn_momentum)
    if self.with_relu:
      self.relu = _nn.ReLU(inplace=True)

  def forward(self, data_in, octree, residual=None, relu=None):
    op = getattr(self, self.attr)
    relu = self.with_relu if relu is None else relu
    # a stride-2 convolution on all nodes is padded AFTER the kernel, and BatchNorm must see the
    # padded zeros: it cannot be folded into the kernel there
    foldable = not (op.is_conv_layer() and op.stride == 2 and not op.nempty)
    if FUSE_EVAL_BN and foldable and not self.training:
      assert data_in.size(1) == op.channel_in
      if not op.is_conv_layer() and op.stride == 2 and not op.nempty:
        data_in = nn.octree_depad(data_in, octree, op.depth)
      scale, bias = _folded(self.bn)
      return op._run(data_in, octree, (scale, bias, residual, relu))
    out = self.bn(op(data_in, octree))
    if residual is not None:
      out = out + residual
    return torch.relu_(out) if relu else out


class OctreeConvBn(_OctreeBlock):
  with_relu = False


class OctreeConvBnRelu(_OctreeBlock):
  pass


class OctreeDeConvBnRelu(_OctreeBlock):
  layer, attr = OctreeDeconv, 'deconv'


class FcBnRelu(_nn.Module):
  def __init__(self, channel_in, channel_out):
    super().__init__()
    self.flatten = _nn.Flatten(start_dim=1)
    self.fc = _nn.Linear(channel_in, channel_out, bias=False)
    self.bn = _nn.BatchNorm1d(channel_out, bn_eps, bn_momentum)
    self.relu = _nn.ReLU(inplace=True)

  def forward(self, data_in):
    return self.relu(self.bn(self.fc(self.flatten(data_in))))


class OctreeConv1x1(_nn.Module):
  """A per-node linear map.  The parameters live in a torch Conv1d (as in the reference, so the
  state_dict keys match); the product runs on this library's pointwise kernels."""

  def __init__(self, channel_in, channel_out, use_bias=False):
    super().__init__()
    self.conv1x1 = _nn.Conv1d(channel_in, channel_out, kernel_size=1, bias=use_bias)
    self._packed = {}

  def run(self, data_in, scale=None, bias=None, residual=None, relu=False):
    if torch.is_grad_enabled() and (data_in.requires_grad or
                                    (self.training and self.conv1x1.weight.requires_grad)):
      # training: torch's own 1x1 convolution (as the reference), which autograd differentiates
      out = self.conv1x1(data_in.squeeze(-1)).unsqueeze(-1)
      if scale is not None:
        out = out * scale.view(1, -1, 1, 1)
      if bias is not None and self.conv1x1.bias is None:
        out = out + bias.view(1, -1, 1, 1)
      if residual is not None:
        out = out + residual
      return torch.relu(out) if relu else out
    w = self.conv1x1.weight.detach()
    cout, cin = w.shape[0], w.shape[1]
    w2 = w.reshape(cout, cin).float()
    if self.conv1x1.bias is not None:
      b = self.conv1x1.bias.detach().float()
      bias = b if bias is None else bias + (b * scale if scale is not None else b)
    with torch.no_grad():
      if _tensor_core_ready(data_in) and cout % 8 == 0 and (cout <= 256 or cout % 256 == 0):
        half = data_in.dtype == torch.float16
        key = (w.data_ptr(), w._version, half)
        if key not in self._packed:
          self._packed.clear()
          self._packed[key] = nn.conv_pack_weights_general(w2.contiguous(), cin, cout, [1, 1, 1], 1,
                                                           False, False, half)
        return nn.pointwise_conv_tc(data_in, self._packed[key], cout, scale, bias, residual, relu,
                                    tc_status(data_in.device))
      return nn.pointwise_conv(data_in, w2.contiguous(), scale, bias, residual, relu)

  def forward(self, data_in):
    return self.run(data_in)


class _Conv1x1Block(_nn.Module):
  with_relu = True

  def __init__(self, channel_in, channel_out, use_bias=False):
    super().__init__()
    self.conv1x1 = OctreeConv1x1(channel_in, channel_out, use_bias)
    self.bn = _nn.BatchNorm2d(channel_out, bn_eps, bn_momentum)
    if self.with_relu:
      self.relu = _nn.ReLU(inplace=True)

  def forward(self, data_in, residual=None, relu=None):
    relu = self.with_relu if relu is None else relu
    if FUSE_EVAL_BN and not self.training:
      scale, bias = _folded(self.bn)
      return self.conv1x1.run(data_in, scale, bias, residual, relu)
    out = self.bn(self.conv1x1(data_in))
    if residual is not None:
      out = out + residual
    return torch.relu_(out) if relu else out


class OctreeConv1x1Bn(_Conv1x1Block):
  with_relu = False


class OctreeConv1x1BnRelu(_Conv1x1Block):
  pass


class _ResBlockBase(_nn.Module):
  def __init__(self, depth, channel_in, channel_out, stride, nempty):
    super().__init__()
    self.channel_in, self.channel_out = channel_in, channel_out
    self.stride, self.depth = stride, depth
    if stride == 2:
      self.maxpool = OctreeMaxPool(depth)
      self.depth = depth - 1
    self.relu = _nn.ReLU(inplace=True)

  def _finish(self, last, branch, skip_proj, data_in, *octree):
    """relu(last(branch) + skip): in eval mode the sum and the ReLU ride in `last`'s epilogue."""
    skip = data_in if skip_proj is None else skip_proj(data_in)
    return last(branch, *octree, residual=skip, relu=True)


class OctreeResBlock(_ResBlockBase):
  """Bottleneck: 1x1 -> 3x3x3 at channel_out / bottleneck -> 1x1, plus the (projected) input."""

  def __init__(self, depth, channel_in, channel_out, stride=1, bottleneck=4, nempty=False):
    super().__init__(depth, channel_in, channel_out, stride, nempty)
    self.bottleneck = bottleneck
    channelb = int(channel_out / bottleneck)
    self.conv1x1a = OctreeConv1x1BnRelu(channel_in, channelb)
    self.conv3x3 = OctreeConvBnRelu(self.depth, channelb, channelb, nempty=nempty)
    self.conv1x1b = OctreeConv1x1Bn(channelb, channel_out)
    if channel_in != channel_out:
      self.conv1x1c = OctreeConv1x1Bn(channel_in, channel_out)

  def forward(self, data_in, octree):
    if self.stride == 2:
      data_in = self.maxpool(data_in, octree)
    mid = self.conv3x3(self.conv1x1a(data_in), octree)
    proj = self.conv1x1c if self.channel_in != self.channel_out else None
    return self._finish(self.conv1x1b, mid, proj, data_in)


class OctreeResBlock2(_ResBlockBase):
  """Two 3x3x3 convolutions, plus the (projected) input."""

  def __init__(self, depth, channel_in, channel_out, stride=1, bottleneck=1, nempty=False):
    super().__init__(depth, channel_in, channel_out, stride, nempty)
    channelb = int(channel_out / bottleneck)
    self.conv3x3a = OctreeConvBnRelu(self.depth, channel_in, channelb, nempty=nempty)
    self.conv3x3b = OctreeConvBn(self.depth, channelb, channel_out, nempty=nempty)
    if channel_in != channel_out:
      self.conv1x1 = OctreeConv1x1Bn(channel_in, channel_out)

  def forward(self, data_in, octree):
    if self.stride == 2:
      data_in = self.maxpool(data_in, octree)
    mid = self.conv3x3a(data_in, octree)
    proj = self.conv1x1 if self.channel_in != self.channel_out else None
    return self._finish(self.conv3x3b, mid, proj, data_in, octree)


class OctreeResBlocks(_nn.Module):
  def __init__(self, depth, channel_in, channel_out, resblk_num, bottleneck=4, nempty=False,
               resblk=OctreeResBlock, use_checkpoint=False):
    super().__init__()
    self.resblk_num = resblk_num
    self.use_checkpoint = use_checkpoint       # training-time memory saving: no effect here
    widths = [channel_in] + [channel_out] * resblk_num
    self.resblks = _nn.ModuleList(
        resblk(depth, widths[i], widths[i + 1], 1, bottleneck, nempty) for i in range(resblk_num))

  def forward(self, data, octree):
    for blk in self.resblks:
      data = blk(data, octree)
    return data


def create_full_octree(depth, channel, batch_size=1, node_dis=True):
  """A full octree of the given depth, grown level by level from octree_new
  (pytorch/ocnn/modules.py:325-330)."""
  assert depth > 1
  octree = nn.octree_new(batch_size, channel, node_dis)
  for target_depth in range(1, depth + 1):
    octree = nn.octree_grow(octree, target_depth, full_octree=True)
  return octree


def octree_feature(octree, depth, nempty=False):
  """The octree's stored signal at `depth` as [1,C,H,1] (on the non-empty nodes when nempty)."""
  out = nn.octree_property(octree, 'feature', depth)
  return nn.octree_depad(out, octree, depth) if nempty else out


# ---- interpolation of node data at points (pytorch/ocnn/modules.py:209-316) -------------------------
def octree_nearest_pts(data, octree, depth, pts, nempty=False):
  """Rows of the cells holding the points.  pts: [N, 4] = (x, y, z) scaled to [0, 2^depth] and the
  batch id; returns [1, C, N, 1] (zeros for points in no cell)."""
  with torch.no_grad():
    return nn.octree_interp(data, octree, depth, pts, 'nearest', nempty)


def octree_trilinear_pts(data, octree, depth, pts, nempty=False):
  """Trilinear interpolation over the 8 cells around each point, renormalised over the cells that
  exist.  One kernel: key arithmetic, search and the weighted sum (the reference builds a sparse
  matrix and multiplies twice)."""
  with torch.no_grad():
    return nn.octree_interp(data, octree, depth, pts, 'linear', nempty)


def octree_trilinear(data, octree, depth, target_depth):
  """Interpolate data from level `depth` at the cell centres of level `target_depth`."""
  xyz = nn.octree_property(octree, 'xyz', target_depth)
  xyz = nn.octree_decode_key(xyz).float()
  scale = 2.0 ** (depth - target_depth)
  xyz = (xyz + xyz.new_tensor([0.5, 0.5, 0.5, 0.0])) * xyz.new_tensor([scale, scale, scale, 1.0])
  return octree_trilinear_pts(data, octree, depth, xyz)


class OctreeTrilinear(_nn.Module):
  def __init__(self, depth):
    super().__init__()
    self.depth = depth

  def forward(self, data, octree):
    return octree_trilinear(data, octree, self.depth, self.depth + 1)


class OctreeInterp(_nn.Module):
  def __init__(self, depth, method='linear', nempty=False):
    super().__init__()
    self.depth, self.method, self.nempty = depth, method, nempty

  def forward(self, data, octree, pts):
    # pts in [-1, 1] -> [0, 2^depth]
    xyz = (pts[:, :3] + 1.0) * (2 ** (self.depth - 1))
    pts = torch.cat([xyz, pts[:, 3:]], dim=1)
    if self.method == 'nearest':
      return octree_nearest_pts(data, octree, self.depth, pts, self.nempty)
    if self.method == 'linear':
      return octree_trilinear_pts(data, octree, self.depth, pts, self.nempty)
    raise ValueError(self.method)

  def extra_repr(self) -> str:
    return 'depth={}, method={}, nempty={}'.format(self.depth, self.method, self.nempty)
