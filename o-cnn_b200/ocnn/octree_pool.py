"""Octree pooling functions and modules (pytorch/ocnn/octree_pool.py:7-115 of the reference)."""
import torch
from torch import nn as _nn

from . import nn
from .octree_pad import octree_pad
from .octree2voxel import FullOctree2Voxel


class _PoolFunction(torch.autograd.Function):
  """kind 0: max-pool (backward: unpool through the mask); 1: max-unpool (backward: mask-pool);
  2: mask-pool (backward: unpool)."""

  @staticmethod
  def forward(ctx, data_in, mask, octree, depth, kind):
    ctx.depth, ctx.kind = depth, kind
    data_in = data_in.contiguous()
    if kind == 0:
      out, mask = nn.octree_max_pool(data_in, octree, depth)
      ctx.save_for_backward(mask, octree)
      ctx.mark_non_differentiable(mask)
      return out, mask
    ctx.save_for_backward(mask, octree)
    if kind == 1:
      return nn.octree_max_unpool(data_in, mask, octree, depth)
    return nn.octree_mask_pool(data_in, mask, octree, depth)

  @staticmethod
  def backward(ctx, grad_in, *unused):
    mask, octree = ctx.saved_tensors
    grad_in = grad_in.contiguous()
    if ctx.kind == 1:
      grad = nn.octree_mask_pool(grad_in, mask, octree, ctx.depth)
    else:
      grad = nn.octree_max_unpool(grad_in, mask, octree, ctx.depth)
    return grad, None, None, None, None


def octree_max_pool(data_in, octree, depth):
  """Max over each sibling group: returns (pooled [1,C,nnum[depth]/8,1], mask int32)."""
  if torch.is_grad_enabled() and data_in.requires_grad:
    return _PoolFunction.apply(data_in, None, octree, depth, 0)
  with torch.no_grad():
    out, mask = nn.octree_max_pool(data_in, octree, depth)
  return out, mask


def octree_max_unpool(data_in, mask, octree, depth):
  """Scatter [1,C,nnum_nempty[depth-1],1] back to the rows its maxima came from: [1,C,nnum[depth],1]."""
  if torch.is_grad_enabled() and data_in.requires_grad:
    return _PoolFunction.apply(data_in, mask, octree, depth, 1)
  with torch.no_grad():
    return nn.octree_max_unpool(data_in, mask, octree, depth)


def octree_mask_pool(data_in, mask, octree, depth):
  """Gather the rows a max-pool mask points at: [1,C,nnum[depth],1] -> [1,C,nnum[depth]/8,1]."""
  if torch.is_grad_enabled() and data_in.requires_grad:
    return _PoolFunction.apply(data_in, mask, octree, depth, 2)
  with torch.no_grad():
    return nn.octree_mask_pool(data_in, mask, octree, depth)


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
    if (not self.return_indices and data.dtype in (torch.bfloat16, torch.float16) and
        data.shape[1] % 8 == 0 and data.is_contiguous(memory_format=torch.channels_last) and
        not (torch.is_grad_enabled() and data.requires_grad)):
      with torch.no_grad():      # both steps in one kernel
        return nn.octree_max_pool_pad(data, octree, self.depth)
    pool, mask = octree_max_pool(data, octree, self.depth)
    output = octree_pad(pool, octree, self.depth - 1)
    return output if not self.return_indices else (output, mask)


class OctreeMaxUnpool(OctreePoolBase):
  def forward(self, data, mask, octree):
    from .octree_pad import octree_depad
    pool = octree_depad(data, octree, self.depth)
    return octree_max_unpool(pool, mask, octree, self.depth + 1)


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
