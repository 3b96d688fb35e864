"""Points2Octree and collate_octrees (pytorch/ocnn/transforms.py:7-32,127-148 of the reference).

Both run on the GPU here.  `collate_octrees` accepts what the reference's DataLoader pipeline
hands it — a list of per-sample dicts whose 'octree' entries are octree tensors — and also
per-sample 'points' entries alone, in which case the batch octree is built from the point clouds
in a single pass (`points2octree_batch`) without building per-sample octrees first.
"""
import torch

from . import nn


class Points2Octree:
  """Convert a point cloud (a uint8 points tensor) into an octree tensor on the GPU."""

  def __init__(self, depth, full_depth=2, node_dis=False, node_feature=False, split_label=False,
               adaptive=False, adp_depth=4, th_normal=0.1, th_distance=2.0, extrapolate=False,
               save_pts=False, key2xyz=False, **kwargs):
    self.depth = depth
    self.full_depth = full_depth
    self.node_dis = node_dis
    self.node_feature = node_feature
    self.split_label = split_label
    self.adaptive = adaptive
    self.adp_depth = adp_depth
    self.th_normal = th_normal
    self.th_distance = th_distance
    self.extrapolate = extrapolate
    self.save_pts = save_pts
    self.key2xyz = key2xyz

  def _args(self):
    return (self.depth, self.full_depth, self.node_dis, self.node_feature, self.split_label,
            self.adaptive, self.adp_depth, self.th_normal, self.th_distance, self.extrapolate,
            self.save_pts, self.key2xyz)

  def __call__(self, points):
    return nn.points2octree(points, *self._args())

  def batch(self, points_list):
    """Merged batch octree of a list of point clouds, built in one pass."""
    return nn.points2octree_batch(list(points_list), *self._args())


def collate_octrees(batch):
  assert type(batch) == list
  outputs = {}
  for key in batch[0].keys():
    outputs[key] = [b[key] for b in batch]
    if 'octree' in key:
      outputs[key] = nn.octree_batch(outputs[key])
    if 'label' in key:
      outputs['label'] = torch.tensor(outputs[key])
  return outputs
