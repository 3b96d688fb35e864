"""Octree pooling modules (pytorch/ocnn/octree_pool.py:79-115 of the reference), forward only."""
import torch
from torch import nn as _nn

from . import nn
from .octree_pad import octree_pad
from .octree2voxel import FullOctree2Voxel


def octree_max_pool(data_in, octree, depth):
  """Max over each sibling group: returns (pooled [1,C,nnum[depth]/8,1], mask int32)."""
  with torch.no_grad():
    out, mask = nn.octree_max_pool(data_in, octree, depth)
  return out, mask


class OctreePoolBase(_nn.Module):
  def __init__(self, depth):
    super().__init__()
    self.depth = depth

  def extra_repr(self) -> str:
    return 'depth={}'.format(self.depth)


class OctreeMaxPool(OctreePoolBase):
  """Pool level `depth` and pad the result to every node of level `depth - 1`."""

  def __init__(self, depth, return_indices=False):
    super().__init__(depth)
    self.return_indices = return_indices

  def forward(self, data, octree):
    if (not self.return_indices and data.dtype == torch.bfloat16 and data.shape[1] % 8 == 0 and
        data.is_contiguous(memory_format=torch.channels_last)):
      with torch.no_grad():      # both steps in one kernel
        return nn.octree_max_pool_pad(data, octree, self.depth)
    pool, mask = octree_max_pool(data, octree, self.depth)
    output = octree_pad(pool, octree, self.depth - 1)
    return output if not self.return_indices else (output, mask)


class OctreeAvgPool(OctreePoolBase):
  def forward(self, data, octree):
    channel = data.shape[1]
    pool = data.reshape(1, channel, -1, 8).mean(dim=3, keepdim=True)
    return octree_pad(pool.contiguous(), octree, self.depth - 1)


class FullOctreeGlobalPool(OctreePoolBase):
  """Mean over the nodes of a full level, per octree of the batch: [1,C,B*8^d,1] -> [B,C]."""

  def __init__(self, depth):
    super().__init__(depth)
    self.octree2voxel = FullOctree2Voxel(depth)

  def forward(self, data):
    return self.octree2voxel(data).mean(dim=2)
