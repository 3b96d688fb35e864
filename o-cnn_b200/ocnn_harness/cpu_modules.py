"""fp32 CPU forward of the `ocnn` networks (ResNet, LeNet, UNet) over a CPU operator module — the
checker for the module route.  It reads the parameters straight out of the torch modules and
walks the same structure with numpy and the operator module it is handed (the oracle, or an
adapter around the compiled reference): `ops` must provide octree_conv_general, max_pool, pad,
depad, octree_interp and an OctreeView-like reader.  Nothing here imports from oracle/ itself."""
import numpy as np


def _np(t):
  return t.detach().float().cpu().numpy()


def _bn(bn):
  scale = _np(bn.weight) / np.sqrt(_np(bn.running_var) + bn.eps)
  return scale.astype(np.float32), (_np(bn.bias) - _np(bn.running_mean) * scale).astype(np.float32)


class CpuModules:
  def __init__(self, ops, view, round_fn=None):
    """round_fn, if given, is applied to every layer's input (e.g. rounding to bf16) so that a
    per-layer comparison with a 16-bit GPU run sees the same operands."""
    self.ops, self.view = ops, view
    self.round = round_fn or (lambda x: x)
    self.trace = None        # set to a list to record (name, output) of every block

  # ---- blocks --------------------------------------------------------------------------------------
  def conv_block(self, blk, x, octree, residual=None, relu=None):
    op = getattr(blk, blk.attr)
    relu = blk.with_relu if relu is None else relu
    v = self.view(octree)
    transposed = not op.is_conv_layer()
    if transposed and op.stride == 2 and not op.nempty:
      x = self.ops.depad(x, v.prop('child', op.depth), int(v.nnum_nempty[op.depth]))
    y = self.ops.octree_conv_general(self.round(x), _np(op.weights), octree, op.depth, op.channel_out,
                                     op.kernel_size, op.stride, op.nempty, transposed)
    if not transposed and op.stride == 2 and not op.nempty:
      y = self.ops.pad(y, v.prop('child', op.depth - 1), 0.0)
    scale, bias = _bn(blk.bn)
    y = y * scale[:, None] + bias[:, None]
    if residual is not None:
      y = y + residual
    return np.maximum(y, 0) if relu else y

  def conv1x1(self, m, x):
    w = _np(m.conv1x1.weight)[:, :, 0]
    y = w @ self.round(x)
    if m.conv1x1.bias is not None:
      y = y + _np(m.conv1x1.bias)[:, None]
    return y

  def conv1x1_block(self, blk, x, residual=None, relu=None):
    relu = blk.with_relu if relu is None else relu
    y = self.conv1x1(blk.conv1x1, x)
    scale, bias = _bn(blk.bn)
    y = y * scale[:, None] + bias[:, None]
    if residual is not None:
      y = y + residual
    return np.maximum(y, 0) if relu else y

  def pool(self, x, octree, depth):
    top, _ = self.ops.max_pool(x)
    return self.ops.pad(top, self.view(octree).prop('child', depth - 1), 0.0)

  def resblock(self, blk, x, octree):
    if blk.stride == 2:
      x = self.pool(x, octree, blk.depth + 1)
    if hasattr(blk, 'conv1x1a'):          # bottleneck block
      mid = self.conv_block(blk.conv3x3, self.conv1x1_block(blk.conv1x1a, x), octree)
      skip = self.conv1x1_block(blk.conv1x1c, x) if blk.channel_in != blk.channel_out else x
      return self.conv1x1_block(blk.conv1x1b, mid, residual=skip, relu=True)
    mid = self.conv_block(blk.conv3x3a, x, octree)
    skip = self.conv1x1_block(blk.conv1x1, x) if blk.channel_in != blk.channel_out else x
    return self.conv_block(blk.conv3x3b, mid, octree, residual=skip, relu=True)

  def resblocks(self, blocks, x, octree):
    for blk in blocks.resblks:
      x = self.resblock(blk, x, octree)
    return x

  def _note(self, name, x):
    if self.trace is not None:
      self.trace.append((name, x))
    return x

  # ---- networks ------------------------------------------------------------------------------------
  def feature(self, octree, depth, nempty=False, channel_in=None):
    v = self.view(octree)
    x = np.ascontiguousarray(v.prop('feature', depth))
    if nempty:
      x = self.ops.depad(x, v.prop('child', depth), int(v.nnum_nempty[depth]))
    if channel_in is not None and channel_in > x.shape[0]:      # zero-padded input channels
      x = np.concatenate([x, np.zeros((channel_in - x.shape[0], x.shape[1]), np.float32)])
    return x

  def resnet(self, net, octree):
    x = self.feature(octree, net.depth, False, net.channel_in)
    x = self._note('conv1', self.conv_block(net.conv1, x, octree))
    for blocks, pool in zip(net.resblocks, net.pools):
      x = self._note('blocks%d' % pool.depth, self.resblocks(blocks, x, octree))
      x = self.pool(x, octree, pool.depth)
    pooled = x.reshape(x.shape[0], -1, 64).mean(axis=2).T             # FullOctreeGlobalPool(2)
    fc = net.header[1]
    return pooled @ _np(fc.weight).T + _np(fc.bias)

  def unet(self, net, octree, pts=None):
    depth = net.depth
    x = self.feature(octree, depth, net.nempty, net.channel_in)
    level = {depth: self._note('conv1', self.conv_block(net.conv1, x, octree))}
    for i in range(net.stages):
      d = depth - i - 1
      down = self._note('down%d' % d, self.conv_block(net.downsample[i], level[d + 1], octree))
      level[d] = self._note('enc%d' % d, self.resblocks(net.encoder[i], down, octree))
    d = depth - net.stages
    x = level[d]
    for i in range(net.stages):
      d += 1
      up = self._note('up%d' % d, self.conv_block(net.upsample[i], x, octree))
      x = np.concatenate([level[d], up], axis=0)
      x = self._note('dec%d' % d, self.resblocks(net.decoder[i], x, octree))
    if pts is not None:
      p = np.asarray(pts, np.float32).copy()
      p[:, :3] = (p[:, :3] + np.float32(1.0)) * np.float32(2 ** (depth - 1))
      x = self.ops.octree_interp(x, octree, depth, p, net.octree_interp.method, net.nempty)
    hidden = self.conv1x1_block(net.header[0], x)
    return self.conv1x1(net.header[1], hidden).T
