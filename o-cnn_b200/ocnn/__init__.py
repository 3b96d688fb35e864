"""ocnn — the operator API of O-CNN's PyTorch package (pytorch/ocnn/__init__.py of the reference),
served by the B200 CUDA library `libocnn_b200.so` through the `ocnn.nn` extension.

Only the inference hot path is provided: octree construction (`points2octree`, `octree_batch`),
`octree_property`, `OctreeConv`, `OctreeMaxPool`, `OctreePad` / `OctreeDepad`, `octree2col` and
the small layout helpers the reference networks use around them.  Everything computes on the GPU;
importing this package fails if the compiled extension is missing — there is no fallback.
"""
import os as _os

try:
  from . import nn
except ImportError as _err:  # pragma: no cover - exercised only on a broken install
  raise ImportError(
      'ocnn.nn (the compiled CUDA extension) is missing or cannot be loaded: %s. '
      'Build it with `python o-cnn_b200/build.py`; there is no CPU or PyTorch fallback.' % _err)

from .nn import (octree_batch, octree_property, points2octree, points2octree_batch, points_new,
                 points_pack, points2octree_packed, octree_info, set_key_bits, get_key_bits)
from .transforms import Points2Octree, collate_octrees
from .octree2voxel import FullOctree2Voxel
from .octree2col import octree2col, Octree2Col
from .octree_pad import (octree_pad, OctreePad, octree_depad, OctreeDepad, octree_tile,
                         OctreeTile)
from .octree_conv import octree_conv, OctreeConv, OctreeConvFast
from .octree_pool import octree_max_pool, OctreeMaxPool, OctreeAvgPool, FullOctreeGlobalPool

LIBRARY = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
                        'libocnn_b200.so')
