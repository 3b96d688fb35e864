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


class NormalizePoints:
  """Centre a cloud and scale it into the unit ball (pytorch/ocnn/transforms.py:35-57).  bsphere:
  'box' (centre and half diagonal of the bounding box; computed on the GPU) — the reference's
  'sphere' needs its external Miniball code and is rejected; or give radius / center yourself."""

  def __init__(self, bsphere='box', radius=-1.0, center=(-1.0,), **kwargs):
    self.bsphere, self.radius, self.center = bsphere, radius, center

  def __call__(self, points):
    if self.radius < 0:
      sphere = nn.bounding_sphere(points, self.bsphere)
      radius, center = sphere[0], sphere[1:]
    else:
      radius, center = self.radius, list(self.center)
    return nn.normalize_points(points, radius, center)


class TransformPoints:
  """Random rotation / scaling / jitter (when `distort`), displacement along the normals and
  normal orientation, then a clip to (-1, 1)^3 (pytorch/ocnn/transforms.py:60-104).  Returns
  (points, inbox_mask); both live on the GPU."""

  def __init__(self, distort, angle=[0, 180, 0], scale=0.25, jitter=0.25, offset=0.0,
               angle_interval=[1, 1, 1], uniform_scale=False, normal_axis='', **kwargs):
    self.distort, self.angle, self.scale, self.jitter = distort, angle, scale, jitter
    self.offset, self.angle_interval = offset, angle_interval
    self.uniform_scale, self.normal_axis = uniform_scale, normal_axis

  def draw(self):
    """The random (angle, scale, jitter) of one call."""
    import numpy as np
    angle, scale, jitter = [0.0] * 3, [1.0] * 3, [0.0] * 3
    if self.distort:
      for i in range(3):
        steps = self.angle[i] // self.angle_interval[i]
        pick = np.random.randint(low=-steps, high=steps + 1, dtype=np.int32)
        angle[i] = pick * self.angle_interval[i] * (3.14159265 / 180.0)
      scale = np.random.uniform(1 - self.scale, 1 + self.scale, size=3).tolist()
      if self.uniform_scale:
        scale = [scale[0]] * 3
      jitter = np.random.uniform(-self.jitter, self.jitter, size=3).tolist()
    return angle, scale, jitter

  def __call__(self, points):
    angle, scale, jitter = self.draw()
    points = nn.transform_points(points, angle, scale, jitter, self.offset, self.normal_axis)
    points, inbox_mask = nn.clip_points(points, [-1.0] * 3, [1.0] * 3)
    return points, inbox_mask


class TransformCompose:
  """normalize -> transform + clip -> octree, as the reference's dataset transform
  (pytorch/ocnn/transforms.py:107-124)."""

  def __init__(self, flags):
    self.flags = flags
    self.normalize_points = NormalizePoints(**flags)
    self.transform_points = TransformPoints(**flags)
    self.points2octree = Points2Octree(**flags)

  def __call__(self, points, idx=None):
    points = self.normalize_points(points)
    points, inbox_mask = self.transform_points(points)
    return {'octree': self.points2octree(points), 'points': points, 'inbox_mask': inbox_mask}
