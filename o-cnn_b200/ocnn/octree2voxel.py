"""FullOctree2Voxel (pytorch/ocnn/octree2voxel.py:5-15 of the reference)."""
import torch


class FullOctree2Voxel(torch.nn.Module):
  """[1,C,B*8^depth,1] on a full octree level -> [B,C,8^depth]."""

  def __init__(self, depth):
    super().__init__()
    self.depth = depth

  def forward(self, data):
    height = 2 ** (3 * self.depth)
    channel = data.size(1)
    out = data.reshape(channel, -1, height)
    return out.permute(1, 0, 2)

  def extra_repr(self) -> str:
    return 'depth={}'.format(self.depth)
