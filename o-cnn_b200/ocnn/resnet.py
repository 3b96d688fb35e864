"""The reference's classification ResNet (pytorch/ocnn/resnet.py:5-31): a 3x3x3 stem at `depth`,
then per level d = depth .. 3 `resblk_num` bottleneck blocks and a max-pool, channels
2^max(11 - d, 2), a global average over the full level 2 and one linear layer."""
import torch
from torch import nn as _nn

from . import nn
from .modules import OctreeConvBnRelu, OctreeResBlocks
from .octree_pool import OctreeMaxPool, FullOctreeGlobalPool


class ResNet(_nn.Module):
  def __init__(self, depth, channel_in, nout, resblk_num):
    super().__init__()
    self.depth, self.channel_in = depth, channel_in
    width = lambda d: 2 ** max(11 - d, 2)
    self.conv1 = OctreeConvBnRelu(depth, channel_in, width(depth))
    levels = range(depth, 2, -1)
    self.resblocks = _nn.ModuleList(
        OctreeResBlocks(d, width(min(d + 1, depth)), width(d), resblk_num) for d in levels)
    self.pools = _nn.ModuleList(OctreeMaxPool(d) for d in levels)
    self.header = _nn.Sequential(FullOctreeGlobalPool(depth=2), _nn.Linear(width(3), nout))

  def forward(self, octree, data=None):
    """`data` overrides the octree's stored signal (e.g. a bfloat16 channels_last copy of it)."""
    if data is None:
      data = nn.octree_property(octree, 'feature', self.depth)
    assert data.size(1) == self.channel_in
    data = self.conv1(data, octree)
    for blocks, pool in zip(self.resblocks, self.pools):
      data = pool(blocks(data, octree), octree)
    return self.header(data.float() if data.dtype != torch.float32 else data)
