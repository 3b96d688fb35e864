"""OctreeConv (pytorch/ocnn/octree_conv.py:8-127 of the reference), forward only.

`OctreeConv` holds its weights exactly as the reference module does — float32
[channel_out, channel_in * K] with column index cin*K + tap — so a reference state_dict loads
unchanged.  The convolution itself is one implicit-GEMM CUDA kernel; no column buffer is built.
"""
import torch
from torch import nn as _nn

from . import nn
from .octree_pad import octree_pad
from .octree2col import octree2col


def resize_with_last_val(list_in, num=3):
  assert (type(list_in) is list and len(list_in) < num + 1)
  out = list(list_in)
  for _ in range(len(out), num):
    out.append(out[-1])
  return out


def octree_conv(data_in, weights, octree, depth, channel_out, kernel_size, stride=1, nempty=False):
  with torch.no_grad():
    return nn.octree_conv(data_in, weights, octree, depth, channel_out,
                          resize_with_last_val(list(kernel_size)), stride, nempty)


class OctreeConvBase(_nn.Module):
  def __init__(self, depth, channel_in, channel_out, kernel_size=[3], stride=1, nempty=False):
    super().__init__()
    self.depth = depth
    self.channel_in = channel_in
    self.channel_out = channel_out
    self.kernel_size = resize_with_last_val(kernel_size)
    self.stride = stride
    self.nempty = nempty
    self.kdim = self.kernel_size[0] * self.kernel_size[1] * self.kernel_size[2]
    self.cdim = channel_in * self.kdim
    self.weights = _nn.Parameter(torch.Tensor(channel_out, self.cdim))
    _nn.init.xavier_uniform_(self.weights)

  def extra_repr(self) -> str:
    return ('depth={}, channel_in={}, channel_out={}, kernel_size={}, stride={}, '
            'nempty={}').format(self.depth, self.channel_in, self.channel_out, self.kernel_size,
                                self.stride, self.nempty)


class OctreeConv(OctreeConvBase):
  def forward(self, data, octree):
    assert data.size(1) == self.channel_in
    conv = octree_conv(data, self.weights, octree, self.depth, self.channel_out,
                       self.kernel_size, self.stride, self.nempty)
    if self.stride == 2 and not self.nempty:
      conv = octree_pad(conv, octree, self.depth - 1)
    return conv


class OctreeConvFast(OctreeConvBase):
  """octree2col followed by a dense matrix product — the reference's memory-hungry variant, kept
  because the reference's own test compares OctreeConv against it."""

  def forward(self, data, octree):
    col = octree2col(data, octree, self.depth, self.kernel_size, self.stride, False)
    col = col.view([self.cdim, -1])
    conv = torch.mm(self.weights.detach(), col)
    conv = torch.unsqueeze(torch.unsqueeze(conv, 0), -1)
    if self.stride == 2:
      conv = octree_pad(conv, octree, self.depth - 1)
    return conv
