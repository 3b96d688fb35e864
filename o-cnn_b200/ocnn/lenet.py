"""The reference's LeNet-style classifier (pytorch/ocnn/lenet.py:5-32): per level d = depth .. 3 a
3x3x3 convolution + BatchNorm + ReLU and a max-pool, channels 2^max(9 - d, 2), then the full
level 2 as voxels through two fully connected layers."""
import torch
from torch import nn as _nn

from . import nn
from .modules import OctreeConvBnRelu, FcBnRelu
from .octree_pool import OctreeMaxPool
from .octree2voxel import FullOctree2Voxel


class LeNet(_nn.Module):
  def __init__(self, depth, channel_in, nout):
    super().__init__()
    self.depth, self.channel_in = depth, channel_in
    width = lambda d: 2 ** max(9 - d, 2)
    levels = list(range(depth, 2, -1))
    self.convs = _nn.ModuleList(
        OctreeConvBnRelu(d, channel_in if d == depth else width(d + 1), width(d)) for d in levels)
    self.pools = _nn.ModuleList(OctreeMaxPool(d) for d in levels)
    self.octree2voxel = FullOctree2Voxel(2)
    self.header = _nn.Sequential(_nn.Dropout(p=0.5), FcBnRelu(width(3) * 64, width(2)),
                                 _nn.Dropout(p=0.5), _nn.Linear(width(2), nout))

  def forward(self, octree, data=None):
    if data is None:
      data = nn.octree_property(octree, 'feature', self.depth)
    assert data.size(1) == self.channel_in
    for conv, pool in zip(self.convs, self.pools):
      data = pool(conv(data, octree), octree)
    data = self.octree2voxel(data.float() if data.dtype != torch.float32 else data)
    return self.header(data)
