"""octree_pad / octree_depad as functions and modules (pytorch/ocnn/octree_pad.py:7-71 of the
reference).  Forward only: this package serves inference."""
import torch
from torch import nn as _nn

from . import nn


def octree_pad(data_in, octree, depth, val=0.0):
  """[1,C,nnum_nempty[depth],1] -> [1,C,nnum[depth],1]; rows of empty nodes get `val`."""
  with torch.no_grad():
    return nn.octree_pad(data_in, octree, depth, val)


def octree_depad(data_in, octree, depth):
  """[1,C,nnum[depth],1] -> [1,C,nnum_nempty[depth],1]: keep the rows of non-empty nodes."""
  with torch.no_grad():
    return nn.octree_depad(data_in, octree, depth)


class OctreePad(_nn.Module):
  def __init__(self, depth, val=0.0):
    super().__init__()
    self.depth = depth
    self.val = val

  def forward(self, data_in, octree):
    return octree_pad(data_in, octree, self.depth, self.val)

  def extra_repr(self) -> str:
    return 'depth={}, val={}'.format(self.depth, self.val)


class OctreeDepad(_nn.Module):
  def __init__(self, depth):
    super().__init__()
    self.depth = depth

  def forward(self, data_in, octree):
    return octree_depad(data_in, octree, self.depth)

  def extra_repr(self) -> str:
    return 'depth={}'.format(self.depth)


def octree_tile(data_in, octree, depth):
  """Nearest-neighbour upsampling from level `depth` to `depth + 1`: octree_depad, then every row
  repeated for its eight children (one kernel)."""
  with torch.no_grad():
    return nn.octree_tile(data_in, octree, depth)


class OctreeTile(_nn.Module):
  """pytorch/ocnn/modules.py:193-207 of the reference."""

  def __init__(self, depth):
    super().__init__()
    self.depth = depth

  def forward(self, data_in, octree):
    return octree_tile(data_in, octree, self.depth)

  def extra_repr(self) -> str:
    return 'depth={}'.format(self.depth)
