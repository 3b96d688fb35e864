"""ocnn — the operator API of O-CNN's PyTorch package (pytorch/ocnn/__init__.py of the reference),
served by the B200 CUDA library `libocnn_b200.so` through the `ocnn.nn` extension.

The inference path is provided: octree construction (`points2octree`, `octree_batch`),
`octree_property`, `OctreeConv` / `OctreeDeconv` (stride 1 or 2, on all or on the non-empty nodes),
`OctreeMaxPool`, `OctreePad` / `OctreeDepad`, `octree2col` / `col2octree`, key conversion and
search, `OctreeInterp`, `octree_align`, the reference's building blocks (`modules`) and its
`LeNet`, `ResNet` and `UNet`.  Everything computes on the GPU;
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
                 points_pack, points2octree_packed, octree_info, set_key_bits, get_key_bits,
                 octree_encode_key, octree_decode_key, octree_search_key, octree_xyz2key,
                 octree_key2xyz)
from .nn import (transform_points, clip_points, normalize_points, bounding_sphere, points_property,
                 points_batch_property, points_set_property)
from .nn import octree_new, octree_grow, octree_update
from .transforms import (Points2Octree, collate_octrees, NormalizePoints, TransformPoints,
                         TransformCompose)
from .io import read_points, write_points, read_octree, write_octree, octree_samples
from .octree2voxel import FullOctree2Voxel
from .octree2col import octree2col, Octree2Col, col2octree, Col2Octree
from .octree_align import octree_align, OctreeAlign
from .octree_pad import (octree_pad, OctreePad, octree_depad, OctreeDepad, octree_tile,
                         OctreeTile)
from .octree_conv import (octree_conv, OctreeConv, OctreeConvFast, octree_deconv, OctreeDeconv,
                          OctreeDeconvFast, tc_status)
from .octree_pool import (octree_max_pool, OctreeMaxPool, octree_max_unpool, OctreeMaxUnpool,
                          octree_mask_pool, OctreeAvgPool, FullOctreeGlobalPool)

from .modules import (OctreeConvBn, OctreeConvBnRelu, OctreeDeConvBnRelu, FcBnRelu, OctreeConv1x1,
                      OctreeConv1x1Bn, OctreeConv1x1BnRelu, OctreeResBlock, OctreeResBlock2,
                      OctreeResBlocks, octree_trilinear_pts, octree_trilinear, octree_nearest_pts,
                      OctreeTrilinear, OctreeInterp, octree_feature, create_full_octree)
from .lenet import LeNet
from .resnet import ResNet
from .unet import UNet

nn.octree_samples = octree_samples      # the reference exposes it on the extension module too

LIBRARY = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
                        'libocnn_b200.so')
