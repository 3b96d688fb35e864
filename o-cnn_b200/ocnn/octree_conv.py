"""OctreeConv / OctreeDeconv (pytorch/ocnn/octree_conv.py:8-158 of the reference).

The modules hold their weights exactly as the reference's do — float32 [channel_out,
channel_in * K] for the convolution, [channel_in, channel_out * K] for the deconvolution, column
index c * K + tap — so a reference state_dict loads unchanged.  Every variant (stride 1 or 2, all
nodes or non-empty nodes only) is one implicit-GEMM CUDA kernel; no column buffer is built.

Data in bfloat16 / float16 with torch's channels_last memory format runs on the tensor-core
kernel (weights are packed once per module and dtype and cached); float32 data, or the
reference's contiguous [1,C,H,1] layout, runs on the CUDA-core kernel.  float32 data that takes
part in autograd (training) goes through `OctreeConvFunction` / `OctreeDeconvFunction`, whose
backward is the transposed operator for the data and a node-reduction kernel for the weights.
"""
import torch
from torch import nn as _nn

from . import nn
from .octree_pad import octree_pad, octree_depad
from .octree2col import octree2col, col2octree

_STATUS = {}


def tc_status(device):
  """The int32 status word the tensor-core kernels write on a bounded wait that ran out (one per
  device; 0 = no kernel ever gave up)."""
  key = torch.device(device)
  if key not in _STATUS:
    _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=key)
  return _STATUS[key]


def resize_with_last_val(list_in, num=3):
  assert (type(list_in) is list and len(list_in) < num + 1)
  out = list(list_in)
  for _ in range(len(out), num):
    out.append(out[-1])
  return out


def _tensor_core_ready(data):
  return (data.is_cuda and data.dtype in (torch.bfloat16, torch.float16) and data.dim() == 4 and
          data.shape[1] % 8 == 0 and data.is_contiguous(memory_format=torch.channels_last))


class _ConvFunctionBase(torch.autograd.Function):
  deconv = False

  @classmethod
  def _forward(cls, ctx, data_in, weights, octree, depth, channel_out, kernel_size, stride, nempty):
    ctx.save_for_backward(data_in, weights, octree)     # (either memory layout is taken as it is)
    ctx.args = (depth, channel_out, resize_with_last_val(list(kernel_size)), stride, nempty)
    op = nn.octree_deconv if cls.deconv else nn.octree_conv
    return op(data_in, weights, octree, *ctx.args)

  @classmethod
  def _backward(cls, ctx, grad_in):
    data_in, weights, octree = ctx.saved_tensors
    op = nn.octree_deconv_grad if cls.deconv else nn.octree_conv_grad
    grad_out, grad_w = op(data_in, weights, octree, grad_in.contiguous(), *ctx.args)
    return (grad_out, grad_w) + (None,) * 6


class OctreeConvFunction(_ConvFunctionBase):
  @staticmethod
  def forward(ctx, *args):
    return OctreeConvFunction._forward(ctx, *args)

  @staticmethod
  def backward(ctx, grad_in):
    return OctreeConvFunction._backward(ctx, grad_in)


class OctreeDeconvFunction(_ConvFunctionBase):
  deconv = True

  @staticmethod
  def forward(ctx, *args):
    return OctreeDeconvFunction._forward(ctx, *args)

  @staticmethod
  def backward(ctx, grad_in):
    return OctreeDeconvFunction._backward(ctx, grad_in)


def _wants_grad(*tensors):
  return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


def octree_conv(data_in, weights, octree, depth, channel_out, kernel_size, stride=1, nempty=False):
  if _wants_grad(data_in, weights):
    return OctreeConvFunction.apply(data_in, weights, octree, depth, channel_out, kernel_size, stride,
                                    nempty)
  with torch.no_grad():
    return nn.octree_conv(data_in, weights, octree, depth, channel_out,
                          resize_with_last_val(list(kernel_size)), stride, nempty)


def octree_deconv(data_in, weights, octree, depth, channel_out, kernel_size, stride=1,
                  nempty=False):
  if _wants_grad(data_in, weights):
    return OctreeDeconvFunction.apply(data_in, weights, octree, depth, channel_out, kernel_size,
                                      stride, nempty)
  with torch.no_grad():
    return nn.octree_deconv(data_in, weights, octree, depth, channel_out,
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
    self.conv_in = channel_in if self.is_conv_layer() else channel_out
    self.conv_out = channel_out if self.is_conv_layer() else channel_in
    self.cdim = self.conv_in * self.kdim
    self.weights = _nn.Parameter(torch.Tensor(self.conv_out, self.cdim))
    _nn.init.xavier_uniform_(self.weights)
    self._packed = {}

  def is_conv_layer(self):
    raise NotImplementedError

  def _run(self, data, octree, fused=None):
    """One kernel for the layer; `fused` = (scale, bias, residual, relu) applied in its epilogue."""
    scale, bias, residual, relu = fused if fused is not None else (None, None, None, False)
    transposed = not self.is_conv_layer()
    if (fused is None and data.dtype == torch.float32 and torch.is_grad_enabled() and
        (data.requires_grad or (self.training and self.weights.requires_grad))):
      fn = OctreeDeconvFunction if transposed else OctreeConvFunction
      return fn.apply(data, self.weights, octree, self.depth, self.channel_out, self.kernel_size,
                      self.stride, self.nempty)
    w = self.weights.detach()
    with torch.no_grad():
      if _tensor_core_ready(data) and self.channel_out % 8 == 0:
        half = data.dtype == torch.float16
        key = (w.data_ptr(), w._version, half)
        if key not in self._packed:
          self._packed.clear()
          try:
            self._packed[key] = nn.conv_pack_weights_general(
                w, self.channel_in, self.channel_out, self.kernel_size, self.stride, transposed,
                self.nempty, half)
          except RuntimeError:
            self._packed[key] = None          # a shape the tensor-core kernel does not take
        packed = self._packed[key]
        if packed is not None:
          return nn.octree_conv_tc_general(
              data, packed, octree, self.depth, self.channel_out, self.kernel_size, self.stride,
              self.nempty, transposed, scale, bias, residual, relu, tc_status(data.device))
      return nn.octree_conv_general(data, w, octree, self.depth, self.channel_out, self.kernel_size,
                                    self.stride, self.nempty, transposed, scale, bias, residual, relu)

  def extra_repr(self) -> str:
    return ('depth={}, channel_in={}, channel_out={}, kernel_size={}, stride={}, '
            'nempty={}').format(self.depth, self.channel_in, self.channel_out, self.kernel_size,
                                self.stride, self.nempty)


class OctreeConv(OctreeConvBase):
  def is_conv_layer(self):
    return True

  def forward(self, data, octree):
    assert data.size(1) == self.channel_in
    conv = self._run(data, octree)
    if self.stride == 2 and not self.nempty:
      conv = octree_pad(conv, octree, self.depth - 1)
    return conv


class OctreeDeconv(OctreeConvBase):
  def is_conv_layer(self):
    return False

  def forward(self, data, octree):
    assert data.size(1) == self.channel_in
    if self.stride == 2 and not self.nempty:
      data = octree_depad(data, octree, self.depth)
    return self._run(data, octree)


class OctreeConvFast(OctreeConvBase):
  """octree2col followed by a dense matrix product — the reference's memory-hungry variant, kept
  because the reference's own test compares OctreeConv against it."""

  def is_conv_layer(self):
    return True

  def forward(self, data, octree):
    col = octree2col(data, octree, self.depth, self.kernel_size, self.stride, False)
    col = col.view([self.cdim, -1])
    conv = torch.mm(self.weights, col)
    conv = torch.unsqueeze(torch.unsqueeze(conv, 0), -1)
    if self.stride == 2:
      conv = octree_pad(conv, octree, self.depth - 1)
    return conv


class OctreeDeconvFast(OctreeConvBase):
  """Dense product followed by col2octree (the scatter-add transpose of octree2col)."""

  def is_conv_layer(self):
    return False

  def forward(self, data, octree):
    if self.stride == 2:
      data = octree_depad(data, octree, self.depth)
    data = data.contiguous().view(self.channel_in, -1)
    col = torch.mm(self.weights.t(), data)
    col = col.view(self.channel_out, self.kdim, -1)
    depth = self.depth + 1 if self.stride == 2 else self.depth
    return col2octree(col, octree, depth, self.kernel_size, self.stride, False)
