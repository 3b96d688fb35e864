"""octree2col / col2octree as functions and modules (pytorch/ocnn/octree2col.py:7-81 of the
reference)."""
import torch
from torch import nn as _nn

from . import nn


class _ColFunction(torch.autograd.Function):
  """octree2col and col2octree are each other's transposes, hence each other's backward."""

  @staticmethod
  def forward(ctx, data_in, octree, depth, kernel_size, stride, nempty, to_col):
    ctx.save_for_backward(octree)
    ctx.args = (depth, list(kernel_size), stride, nempty)
    ctx.to_col = to_col
    op = nn.octree2col if to_col else nn.col2octree
    return op(data_in.contiguous(), octree, *ctx.args)

  @staticmethod
  def backward(ctx, grad_in):
    octree, = ctx.saved_tensors
    op = nn.col2octree if ctx.to_col else nn.octree2col
    return (op(grad_in.contiguous(), octree, *ctx.args),) + (None,) * 6


def octree2col(data_in, octree, depth, kernel_size, stride, nempty=False):
  """[1,C,H,1] float32 -> [C, K, H_out]: the neighbourhood of every node, K taps per channel."""
  if torch.is_grad_enabled() and data_in.requires_grad:
    return _ColFunction.apply(data_in, octree, depth, kernel_size, stride, nempty, True)
  with torch.no_grad():
    return nn.octree2col(data_in, octree, depth, list(kernel_size), stride, nempty)


def col2octree(data_in, octree, depth, kernel_size, stride, nempty=False):
  """The transpose of octree2col: [C, K, H_col] float32 -> [1,C,H,1], every column entry added to
  the node it would have been gathered from."""
  if torch.is_grad_enabled() and data_in.requires_grad:
    return _ColFunction.apply(data_in, octree, depth, kernel_size, stride, nempty, False)
  with torch.no_grad():
    return nn.col2octree(data_in, octree, depth, list(kernel_size), stride, nempty)


class Octree2Col(_nn.Module):
  def __init__(self, depth, kernel_size, stride, nempty=False):
    super().__init__()
    self.depth = depth
    self.kernel_size = kernel_size
    self.stride = stride
    self.nempty = nempty

  def forward(self, data_in, octree):
    return octree2col(data_in, octree, self.depth, self.kernel_size, self.stride, self.nempty)

  def extra_repr(self) -> str:
    return 'depth={}, kernel_size={}, stride={}, nempty={}'.format(
        self.depth, self.kernel_size, self.stride, self.nempty)


class Col2Octree(Octree2Col):
  def forward(self, data_in, octree):
    return col2octree(data_in, octree, self.depth, self.kernel_size, self.stride, self.nempty)
