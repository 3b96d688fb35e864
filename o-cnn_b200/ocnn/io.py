"""`.points` and `.octree` files: both are the flat buffers themselves, written byte for byte
(Points::read_points / write_points, octree/octree/points.cpp:9-42; Octree::read_octree /
write_octree, octree/octree/octree.cpp:41-72).  Reading validates the header and returns a uint8
tensor that `points2octree` / `octree_batch` / the operators take as it is."""
import numpy as np
import torch

from . import nn


def _read(filename, magic, min_bytes, what):
  data = np.fromfile(filename, dtype=np.uint8)
  if data.size < min_bytes:
    raise ValueError('%s: %d bytes is shorter than a %s header' % (filename, data.size, what))
  if bytes(data[:len(magic)]) != magic:
    raise ValueError('%s: not a %s file (magic %r)' % (filename, what, bytes(data[:12])))
  return torch.from_numpy(data)


def read_points(filename, device=None):
  t = _read(filename, b'_POINTS_1.0_', 88, 'points')
  size = int(np.frombuffer(t.numpy()[56:88].tobytes(), np.int32)[4])       # ptr_dis[4] = total bytes
  if size > t.numel():
    raise ValueError('%s: truncated (header says %d bytes, file has %d)' % (filename, size, t.numel()))
  return t if device is None else t.to(device)


def read_octree(filename, device=None):
  t = _read(filename, b'_OCTREE_', 716, 'octree')
  nn.octree_info(t)            # parses and validates the header (raises on a malformed one)
  return t if device is None else t.to(device)


def _write(tensor, filename):
  tensor.detach().cpu().contiguous().numpy().astype(np.uint8, copy=False).tofile(filename)


def write_points(points, filename):
  _write(points, filename)


def write_octree(octree, filename):
  _write(octree, filename)


_SAMPLES = {}


def octree_samples(names):
  """The small octrees the reference library carries for its own tests (`octree_1` .. `octree_6`,
  octree/octree/octree_samples.cpp; binding pytorch/cpp/octree_samples.cpp:5-22), as CPU uint8
  tensors in the current key width (`ocnn.set_key_bits`)."""
  import os
  if not _SAMPLES:
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'data', 'octree_samples.npz')
    _SAMPLES.update(np.load(path))
  out = []
  for name in names:
    key = 'k%d_%s' % (nn.get_key_bits(), name)
    if key not in _SAMPLES:
      raise ValueError('unknown octree sample %r' % (name,))
    out.append(torch.from_numpy(_SAMPLES[key].copy()))
  return out
