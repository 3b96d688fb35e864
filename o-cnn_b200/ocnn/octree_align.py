"""octree_align (pytorch/ocnn/octree_align.py:7-40 of the reference): carry node data from one
octree to another at a given depth by matching node keys."""
import torch
from torch import nn as _nn

from . import nn


def octree_align(src_data, src_octree, des_octree, depth):
  """Returns (des_data [1,C,nnum_des[depth],1], index int32 [nnum_src[depth]]): des_data holds the
  source row of every node both octrees have, zeros elsewhere; index[h] = destination row of source
  node h or -1."""
  if torch.is_grad_enabled() and src_data.requires_grad:
    return _AlignFunction.apply(src_data, src_octree, des_octree, depth)
  with torch.no_grad():
    des, index = nn.octree_align(src_data, src_octree, des_octree, depth)
  return des, index


class _AlignFunction(torch.autograd.Function):
  @staticmethod
  def forward(ctx, src_data, src_octree, des_octree, depth):
    des, index = nn.octree_align(src_data.contiguous(), src_octree, des_octree, depth)
    ctx.save_for_backward(index)
    ctx.mark_non_differentiable(index)
    return des, index

  @staticmethod
  def backward(ctx, des_grad, index_grad):
    index, = ctx.saved_tensors
    return nn.octree_align_grad(des_grad.contiguous(), index), None, None, None


class OctreeAlign(_nn.Module):
  def __init__(self, depth, return_index=False):
    super().__init__()
    self.depth = depth
    self.return_index = return_index

  def forward(self, src_data, src_octree, des_octree):
    output = octree_align(src_data, src_octree, des_octree, self.depth)
    return output if self.return_index else output[0]

  def extra_repr(self) -> str:
    return 'depth={}'.format(self.depth)
