"""octree_pad / octree_depad as functions and modules (pytorch/ocnn/octree_pad.py:7-71 of the
reference).  Each is the other's backward."""
import torch
from torch import nn as _nn

from . import nn


class _PadFunction(torch.autograd.Function):
  @staticmethod
  def forward(ctx, data_in, octree, depth, val, pad):
    ctx.save_for_backward(octree)
    ctx.depth, ctx.pad = depth, pad
    if pad:
      return nn.octree_pad(data_in, octree, depth, val)
    return nn.octree_depad(data_in, octree, depth)

  @staticmethod
  def backward(ctx, grad_in):
    octree, = ctx.saved_tensors
    if ctx.pad:
      return nn.octree_depad(grad_in.contiguous(), octree, ctx.depth), None, None, None, None
    return nn.octree_pad(grad_in.contiguous(), octree, ctx.depth, 0.0), None, None, None, None


def octree_pad(data_in, octree, depth, val=0.0):
  """[1,C,nnum_nempty[depth],1] -> [1,C,nnum[depth],1]; rows of empty nodes get `val`."""
  if torch.is_grad_enabled() and data_in.requires_grad:
    return _PadFunction.apply(data_in, octree, depth, val, True)
  with torch.no_grad():
    return nn.octree_pad(data_in, octree, depth, val)


def octree_depad(data_in, octree, depth):
  """[1,C,nnum[depth],1] -> [1,C,nnum_nempty[depth],1]: keep the rows of non-empty nodes."""
  if torch.is_grad_enabled() and data_in.requires_grad:
    return _PadFunction.apply(data_in, octree, depth, 0.0, False)
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
