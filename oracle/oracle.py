"""TEST INFRASTRUCTURE ONLY: ctypes driver for the C oracle (``oracle/ocnn_oracle.c``).

The oracle restates the reference's CPU algorithms for the octree hot path.  Only tests, the
smoke check and the benchmark's CPU-baseline leg import this module; the shipped CUDA library
never does.  ``OctreeView`` is a small numpy reader of the octree wire format used by the tests to
slice properties out of a buffer, whichever implementation produced it.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

c_float_p = ctypes.POINTER(ctypes.c_float)
c_int_p = ctypes.POINTER(ctypes.c_int32)
c_u8_p = ctypes.POINTER(ctypes.c_uint8)

PROPS = ['key', 'child', 'neigh', 'feature', 'label', 'split']


def build():
  """Compile the C oracle in place (gcc only; a second or so)."""
  subprocess.check_call(['make', '-s', '-C', _HERE, 'port'])


def lib():
  global _LIB
  if _LIB is None:
    path = os.path.join(_HERE, 'libocnn_oracle.so')
    src = os.path.join(_HERE, 'ocnn_oracle.c')
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
      build()
    L = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    L.oc_points2octree.restype = ctypes.c_long
    L.oc_points2octree.argtypes = [ctypes.c_char_p] + [ctypes.c_int] * 7 + [
        ctypes.c_float, ctypes.c_float, c_float_p, c_u8_p, ctypes.c_long]
    L.oc_octree_batch.restype = ctypes.c_long
    L.oc_octree_batch.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.c_int, c_u8_p,
                                  ctypes.c_long]
    L.oc_morton.restype = ctypes.c_uint64
    L.oc_morton.argtypes = [ctypes.c_uint64] * 3 + [ctypes.c_int]
    L.oc_ni_table.restype = ctypes.c_int
    L.oc_ni_table.argtypes = [c_int_p, c_int_p]
    L.oc_calc_neigh_full.argtypes = [c_int_p, ctypes.c_int, ctypes.c_int]
    L.oc_calc_neigh_split.argtypes = [c_int_p, c_int_p, c_int_p, ctypes.c_int]
    L.oc_octree2col.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 4 + [c_int_p, c_int_p]
    L.oc_octree2col_p.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 4 + [c_int_p] * 4
    L.oc_ichild.argtypes = [c_int_p, c_int_p, ctypes.c_int]
    L.oc_octree_conv_nempty.restype = ctypes.c_long
    L.oc_octree_conv_nempty.argtypes = [c_float_p, ctypes.c_long, c_float_p, c_float_p,
                                        ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        c_int_p]
    L.oc_octree_conv.restype = ctypes.c_long
    L.oc_octree_conv.argtypes = [c_float_p, ctypes.c_long, c_float_p, c_float_p, ctypes.c_char_p,
                                 ctypes.c_int, ctypes.c_int, ctypes.c_int, c_int_p, ctypes.c_int]
    L.oc_octree_conv_general.restype = ctypes.c_long
    L.oc_octree_conv_general.argtypes = [c_float_p, ctypes.c_long, c_float_p, c_float_p,
                                         ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                         c_int_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    L.oc_col2octree.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 4 + [c_int_p, c_int_p]
    L.oc_octree2col_p2.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 5 + [c_int_p] * 4
    L.oc_col2octree_p.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 5 + [c_int_p] * 4
    L.oc_xyz2key.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_int]
    L.oc_key2xyz.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_int]
    L.oc_search_key.argtypes = [c_int_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_long]
    L.oc_max_pool.argtypes = [c_float_p, ctypes.c_int, c_int_p, c_float_p, ctypes.c_int,
                              ctypes.c_int]
    L.oc_pad.argtypes = [c_float_p, ctypes.c_int, ctypes.c_int, c_float_p, ctypes.c_int, c_int_p,
                         ctypes.c_float]
    L.oc_depad.argtypes = [c_float_p, ctypes.c_int, ctypes.c_int, c_float_p, ctypes.c_int,
                           c_int_p]
    _LIB = L
  return _LIB


def _fp(a):
  return None if a is None else a.ctypes.data_as(c_float_p)


def _ip(a):
  return None if a is None else a.ctypes.data_as(c_int_p)


def _f32(a):
  return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
  return np.ascontiguousarray(a, dtype=np.int32)


def _bytes(a):
  return np.ascontiguousarray(a, dtype=np.uint8).tobytes()


# -- wire formats --------------------------------------------------------------------------
def points_new(pts, normals=None, feats=None, labels=None):
  """Points buffer: 88-byte PointsInfo header then xyz / normal / feature / label arrays,
  point-major float32 (octree/octree/points_info.h:8-40, points.cpp:96-150)."""
  pts = _f32(pts).reshape(-1, 3)
  n = pts.shape[0]
  blocks = [pts]
  channels = [3, 0, 0, 0]
  flags = 1
  for i, arr in enumerate((normals, feats, labels), start=1):
    if arr is None:
      blocks.append(None)
      continue
    arr = _f32(arr).reshape(n, -1)
    channels[i] = arr.shape[1]
    flags |= 1 << i
    blocks.append(arr)
  hdr = np.zeros(88, dtype=np.uint8)
  hdr[:12] = np.frombuffer(b'_POINTS_1.0_', dtype=np.uint8)
  ints = hdr[16:].view(np.int32)
  ints[0] = n
  ints[1] = flags
  ints[2:6] = channels
  dis = 88
  for i in range(5):
    ints[10 + i] = dis
    if i < 4:
      dis += 4 * n * channels[i]
  payload = b''.join(b.tobytes() for b in blocks if b is not None)
  return np.concatenate([hdr, np.frombuffer(payload, dtype=np.uint8)])


class OctreeView:
  """Read-only numpy view of an octree buffer (single or merged batch)."""

  def __init__(self, buf):
    self.buf = np.ascontiguousarray(buf, dtype=np.uint8)
    b = self.buf
    self.magic = bytes(b[:12])
    self.key_bits = 64 if self.magic == b'_OCTREE_2.0_' else 32
    i32 = lambda off, n=1: b[off:off + 4 * n].view(np.int32)
    self.batch_size = int(i32(16)[0])
    self.depth = int(i32(20)[0])
    self.full_depth = int(i32(24)[0])
    self.nnum = i32(48, 16).copy()
    self.nnum_cum = i32(112, 16).copy()
    self.nnum_nempty = i32(176, 16).copy()
    self.content_flags = int(i32(240)[0])
    self.channels = i32(244, 16).copy()
    self.locations = i32(308, 16).copy()
    self.ptr_dis = i32(652, 16).copy()
    self.sizeof_octree = int(self.ptr_dis[6])

  def has(self, prop):
    return self.channels[PROPS.index(prop)] != 0

  def prop(self, prop, d):
    """Array of property `prop` at level d: key uint32/uint64 [n], child int32 [n],
    neigh int32 [n/8, 64], feature float32 [C, n], label/split float32 [n]."""
    p = PROPS.index(prop)
    ch = int(self.channels[p])
    assert ch != 0, prop
    esz = self.key_bits // 8 if prop == 'key' else 4
    off = int(self.ptr_dis[p])
    if self.locations[p] == -1:
      off += int(self.nnum_cum[d]) * ch * esz
    else:
      assert d == self.locations[p]
    n = int(self.nnum[d])
    raw = self.buf[off:off + n * ch * esz]
    if prop == 'key':
      return raw.view(np.uint64 if esz == 8 else np.uint32)
    if prop in ('child',):
      return raw.view(np.int32)
    if prop == 'neigh':
      return raw.view(np.int32).reshape(-1, 64)
    if prop == 'feature':
      return raw.view(np.float32).reshape(ch, n)
    return raw.view(np.float32)


# -- oracle calls --------------------------------------------------------------------------
def _sized(call):
  n = call(None, 0)
  if n < 0:
    raise ValueError('oracle call failed (%d)' % n)
  out = np.zeros(n, dtype=np.uint8)
  m = call(out.ctypes.data_as(c_u8_p), n)
  assert m == n
  return out


def points2octree(points, depth, full_depth=2, node_dis=False, split_label=False,
                  save_pts=False, key_bits=32, bbox=None, adp_depth=4, th_normal=0.1,
                  th_distance=2.0):
  pbuf = _bytes(points)
  bb = None if bbox is None else _f32(bbox)
  return _sized(lambda o, c: lib().oc_points2octree(
      pbuf, depth, full_depth, int(node_dis), int(split_label), int(save_pts), key_bits,
      adp_depth, th_normal, th_distance, _fp(bb), o, c))


def octree_batch(octrees):
  bufs = [_bytes(o) for o in octrees]
  arr = (ctypes.c_char_p * len(bufs))(*bufs)
  return _sized(lambda o, c: lib().oc_octree_batch(arr, len(bufs), o, c))


def morton(x, y, z, depth):
  return int(lib().oc_morton(int(x), int(y), int(z), depth))


def ni_table(ksize):
  ks = _i32(ksize)
  n = lib().oc_ni_table(_ip(ks), None)
  if n < 0:
    raise ValueError('unsupported kernel size %s' % (list(ksize),))
  out = np.empty(n, np.int32)
  lib().oc_ni_table(_ip(ks), _ip(out))
  return out


def calc_neigh_full(depth, batch_size):
  out = np.empty(batch_size * (8 ** depth) * 8, dtype=np.int32)
  lib().oc_calc_neigh_full(_ip(out), depth, batch_size)
  return out


def calc_neigh_split(neigh, child, nnum_child, fill=-7):
  neigh, child = _i32(neigh), _i32(child)
  out = np.full(nnum_child * 8, fill, dtype=np.int32)
  lib().oc_calc_neigh_split(_ip(out), _ip(neigh), _ip(child), child.size)
  return out


def octree2col(data, neigh, ksize, stride, height):
  data, neigh = _f32(data), _i32(neigh)
  channel = data.shape[0]
  ni = ni_table(ksize)
  kdim = int(np.prod(ksize))
  col = np.empty((channel, kdim, height), np.float32)
  lib().oc_octree2col(_fp(col), _fp(data), channel, height, kdim, stride, _ip(neigh), _ip(ni))
  return col


def octree_conv(data, weights, octree, depth, num_output, ksize, stride):
  data, weights = _f32(data), _f32(weights)
  ks = _i32(ksize)
  obuf = _bytes(octree)
  cin = data.shape[0]
  n = lib().oc_octree_conv(None, 0, _fp(data), _fp(weights), obuf, depth, cin, num_output,
                           _ip(ks), stride)
  if n < 0:
    raise ValueError('unsupported convolution')
  top = np.zeros((num_output, n // num_output), np.float32)
  lib().oc_octree_conv(_fp(top), n, _fp(data), _fp(weights), obuf, depth, cin, num_output,
                       _ip(ks), stride)
  return top


def octree2col_p(data, neigh, child, ksize):
  """octree2colP (nempty, stride 1): data [C, nne] over the non-empty nodes -> [C, K, nne]."""
  data, neigh, child = _f32(data), _i32(neigh), _i32(child)
  channel, nne = data.shape
  ni = ni_table(ksize)
  kdim = int(np.prod(ksize))
  ichild = np.zeros(max(nne, 1), np.int32)
  lib().oc_ichild(_ip(ichild), _ip(child), child.shape[0])
  col = np.empty((channel, kdim, nne), np.float32)
  lib().oc_octree2col_p(_fp(col), _fp(data), channel, nne, nne, kdim, _ip(neigh), _ip(ni),
                        _ip(child), _ip(ichild))
  return col


def octree_conv_nempty(data, weights, octree, depth, num_output, ksize):
  """OctreeConv(nempty=True), stride 1: data [Cin, nne[depth]] -> [Cout, nne[depth]]."""
  data, weights = _f32(data), _f32(weights)
  ks = _i32(ksize)
  obuf = _bytes(octree)
  cin = data.shape[0]
  n = lib().oc_octree_conv_nempty(None, 0, _fp(data), _fp(weights), obuf, depth, cin, num_output,
                                  _ip(ks))
  if n < 0:
    raise ValueError('unsupported convolution')
  top = np.zeros((num_output, n // num_output), np.float32)
  lib().oc_octree_conv_nempty(_fp(top), n, _fp(data), _fp(weights), obuf, depth, cin, num_output,
                              _ip(ks))
  return top


def octree_conv_general(data, weights, octree, depth, num_output, ksize, stride=1, nempty=False,
                        deconv=False):
  """OctreeConv / OctreeDeconv forward for any stride / nempty combination.  data: [Cin, H] with
  H = nnum[depth], or nnum_nempty[depth] when nempty or for a stride-2 deconvolution."""
  data, weights = _f32(data), _f32(weights)
  ks = _i32(ksize)
  obuf = _bytes(octree)
  cin = data.shape[0]
  args = (_fp(data), _fp(weights), obuf, depth, cin, num_output, _ip(ks), stride, int(nempty),
          int(deconv))
  n = lib().oc_octree_conv_general(None, 0, *args)
  if n < 0:
    raise ValueError('unsupported convolution')
  top = np.zeros((num_output, n // num_output), np.float32)
  lib().oc_octree_conv_general(_fp(top), n, *args)
  return top


def ichild_of(child, nne):
  child = _i32(child)
  ichild = np.zeros(max(nne, 1), np.int32)
  lib().oc_ichild(_ip(ichild), _ip(child), child.shape[0])
  return ichild


def octree2col_general(data, neigh, ksize, stride, height, child=None):
  """octree2col (child is None) or octree2colP (child given: data holds the non-empty nodes
  only).  height = rows of the column matrix (nodes at stride 1, sibling groups at stride 2)."""
  if child is None:
    return octree2col(data, neigh, ksize, stride, height)
  data, neigh, child = _f32(data), _i32(neigh), _i32(child)
  channel, octree_h = data.shape
  ni = ni_table(ksize)
  kdim = int(np.prod(ksize))
  ichild = ichild_of(child, max(octree_h, height))
  col = np.empty((channel, kdim, height), np.float32)
  lib().oc_octree2col_p2(_fp(col), _fp(data), channel, height, octree_h, kdim, stride, _ip(neigh),
                         _ip(ni), _ip(child), _ip(ichild))
  return col


def col2octree_general(col, neigh, ksize, stride, octree_h, child=None):
  """col2octree / col2octreeP: col [C, K, height] scattered back to data [C, octree_h]."""
  col, neigh = _f32(col), _i32(neigh)
  channel, kdim, height = col.shape
  ni = ni_table(ksize)
  data = np.zeros((channel, octree_h), np.float32)
  if child is None:
    assert octree_h == height << (3 * (stride - 1))
    lib().oc_col2octree(_fp(col), _fp(data), channel, height, kdim, stride, _ip(neigh), _ip(ni))
  else:
    child = _i32(child)
    ichild = ichild_of(child, max(octree_h, height))
    lib().oc_col2octree_p(_fp(col), _fp(data), channel, height, octree_h, kdim, stride,
                          _ip(neigh), _ip(ni), _ip(child), _ip(ichild))
  return data


def _u64(a):
  return np.ascontiguousarray(np.asarray(a).astype(np.uint64, copy=False), dtype=np.uint64)


def xyz2key(xyz, depth, key_bits=64):
  """Packed (x, y, z, id) lanes -> Morton key with the id lane kept; uint64 arrays either width."""
  xyz = _u64(xyz)
  out = np.empty_like(xyz)
  lib().oc_xyz2key(out.ctypes.data_as(ctypes.c_void_p), xyz.ctypes.data_as(ctypes.c_void_p), xyz.size,
                   depth, key_bits)
  return out


def key2xyz(key, depth, key_bits=64):
  key = _u64(key)
  out = np.empty_like(key)
  lib().oc_key2xyz(out.ctypes.data_as(ctypes.c_void_p), key.ctypes.data_as(ctypes.c_void_p), key.size,
                   depth, key_bits)
  return out


def search_key(keys, query):
  keys, query = _u64(keys), _u64(query)
  idx = np.empty(query.size, np.int32)
  lib().oc_search_key(_ip(idx), keys.ctypes.data_as(ctypes.c_void_p), keys.size,
                      query.ctypes.data_as(ctypes.c_void_p), query.size)
  return idx


def level_keys(octree, depth, nempty=False):
  """Ascending Morton keys (batch id in the top lane) of a level, as uint64; of its non-empty nodes
  only when nempty (pytorch/cpp/octree_key.cpp:96-108)."""
  v = OctreeView(octree)
  keys = v.prop('key', depth).astype(np.uint64)
  if nempty:
    child = v.prop('child', depth)
    keys = keys[child >= 0]
  return keys


def octree_interp(data, octree, depth, pts, method='linear', nempty=False):
  """The reference's octree_nearest_pts / octree_trilinear_pts (pytorch/ocnn/modules.py:209-275)
  restated in numpy over xyz2key / search_key.  data: [C, H]; pts: [N, 4] float32 with xyz already
  scaled to [0, 2^depth]; returns [C, N] float32.  64-bit keys."""
  data = _f32(data)
  pts = _f32(pts)
  keys = level_keys(octree, depth, nempty)
  n = pts.shape[0]
  if method == 'nearest':
    lanes = pts.astype(np.int16).astype(np.uint16).astype(np.uint64)       # Tensor.short()
    word = lanes[:, 0] | (lanes[:, 1] << 16) | (lanes[:, 2] << 32) | (lanes[:, 3] << 48)
    idx = search_key(keys, xyz2key(word, depth))
    ok = idx > -1
    out = data[:, idx * ok] * ok.astype(np.float32)
    return np.ascontiguousarray(out, np.float32)
  xyzf = pts[:, :3] - np.float32(0.5)
  xyzi = np.floor(xyzf)
  frac = xyzf - xyzi
  lanes = np.concatenate([xyzi, pts[:, 3:4]], axis=1).astype(np.int16).astype(np.uint16).astype(np.uint64)
  word = lanes[:, 0] | (lanes[:, 1] << 16) | (lanes[:, 2] << 32) | (lanes[:, 3] << 48)
  mask = np.array([[0, 0, 0], [0, 0, 1], [0, 1, 0], [0, 1, 1], [1, 0, 0], [1, 0, 1], [1, 1, 0], [1, 1, 1]],
                  np.float32)
  masku = np.array([0, 4294967296, 65536, 4295032832, 1, 4294967297, 65537, 4295032833], np.uint64)
  word8 = (word[:, None] + masku[None, :]).reshape(-1)           # packed addition: lanes may carry
  idx = search_key(keys, xyz2key(word8, depth)).reshape(n, 8)
  w = np.abs(np.prod((1 - mask)[None, :, :] - frac[:, None, :], axis=2)).astype(np.float32)
  ok = idx > -1
  w = w * ok
  out = np.zeros((data.shape[0], n), np.float32)
  for j in range(8):
    out += data[:, idx[:, j] * ok[:, j]] * w[:, j][None, :]
  norm = w.sum(axis=1)
  return (out / (norm + np.float32(1e-10))[None, :]).astype(np.float32)


# ---- point-cloud preparation (octree/octree/points_parser.cpp:42-259) -------------------------------
def _points_blocks(buf):
  """Views (xyz, normal, feature, label) into a points buffer, None where absent; and pt_num."""
  npt = int(buf[16:20].view(np.int32)[0])
  channels = buf[24:56].view(np.int32)
  ptr_dis = buf[56:88].view(np.int32)
  out = []
  for t in range(4):
    c = int(channels[t])
    out.append(None if c == 0 else buf[ptr_dis[t]:ptr_dis[t] + 4 * npt * c].view(np.float32).reshape(npt, c))
  return out, npt


def _matrix_prod3(A, B):
  """matrix_prod of two column-major 3x3 matrices, math_functions.cpp:185-196, in fp32."""
  C = np.zeros(9, np.float32)
  for n in range(3):
    for m in range(3):
      acc = np.float32(0)
      for k in range(3):
        acc = np.float32(acc + np.float32(A[k * 3 + m] * B[n * 3 + k]))
      C[n * 3 + m] = acc
  return C


def rotation_matrix(angle):
  """rotation_matrix(rot, angles), math_functions.cpp:148-158 (cos / sin evaluated in double)."""
  c = [np.float32(np.cos(np.float64(np.float32(a)))) for a in angle]
  s = [np.float32(np.sin(np.float64(np.float32(a)))) for a in angle]
  z, o = np.float32(0), np.float32(1)
  rx = np.array([o, z, z, z, c[0], s[0], z, -s[0], c[0]], np.float32)
  ry = np.array([c[1], z, -s[1], z, o, z, s[1], z, c[1]], np.float32)
  rz = np.array([c[2], s[2], z, -s[2], c[2], z, z, z, o], np.float32)
  return _matrix_prod3(_matrix_prod3(rx, ry), rz)


def _apply3(rot, v):
  out = np.zeros_like(v)
  for m in range(3):
    acc = np.zeros(v.shape[0], np.float32)
    for k in range(3):
      acc = acc + rot[k * 3 + m] * v[:, k]
    out[:, m] = acc
  return out


def transform_points(points, angle, scale, jitter, offset, normal_axis=''):
  """transform_points, pytorch/cpp/transform_points.cpp:71-108, on a copy of the buffer."""
  buf = np.array(points, dtype=np.uint8, copy=True)
  (xyz, nrm, _, _), npt = _points_blocks(buf)
  eps = np.float32(1.0e-10)
  angle, scale, jitter = _f32(angle), _f32(scale), _f32(jitter)
  offset = np.float32(offset)
  if offset > eps and nrm is not None:
    xyz += nrm * offset
  if np.any(np.abs(angle) > eps):
    rot = rotation_matrix(angle)
    xyz[:] = _apply3(rot, xyz)
    if nrm is not None:
      nrm[:] = _apply3(rot, nrm)
  if np.any(np.abs(jitter) > eps):
    xyz += jitter[None, :]
  if np.any(scale != 1) and not np.any(scale == 0):
    xyz *= scale[None, :]
    if not (scale[0] == scale[1] == scale[2]) and nrm is not None:
      nrm *= (np.float32(1.0) / scale)[None, :]
      length = np.zeros(npt, np.float32)
      for m in range(3):
        length = length + nrm[:, m] * nrm[:, m]
      inv = np.float32(1.0) / (np.sqrt(length) + np.float32(1.0e-15))
      nrm *= inv[:, None]
  if nrm is not None and normal_axis in ('x', 'y', 'z'):
    j = 'xyz'.index(normal_axis)
    nrm[nrm[:, j] < 0] *= np.float32(-1)
  elif nrm is not None and normal_axis == 'xyz':
    nrm[:] = np.where(nrm < 0, -nrm, nrm)
  return buf


def clip_points(points, bbmin, bbmax):
  """clip_points, transform_points.cpp:110-125 / PointsParser::clip: (buffer, in-box mask)."""
  buf = np.array(points, dtype=np.uint8, copy=True)
  blocks, npt = _points_blocks(buf)
  xyz = blocks[0]
  lo, hi = _f32(bbmin), _f32(bbmax)
  inside = np.all((lo[None, :] < xyz) & (xyz < hi[None, :]), axis=1)
  mask = inside.astype(np.int32)
  if inside.all():
    return buf, mask
  if not inside.any():
    mask[0] = 1
    inside = mask.astype(bool)
    xyz[0] = lo
  kept = int(inside.sum())
  for b in blocks:
    if b is not None:
      b[:kept] = b[inside]
  buf[16:20].view(np.int32)[0] = kept
  return buf, mask


def bounding_box(xyz):
  xyz = _f32(xyz).reshape(-1, 3)
  return np.concatenate([xyz.min(axis=0), xyz.max(axis=0)]).astype(np.float32)


def max_pool(btm):
  btm = _f32(btm)
  channel, btm_h = btm.shape
  top_h = btm_h // 8
  top = np.empty((channel, top_h), np.float32)
  mask = np.empty((channel, top_h), np.int32)
  lib().oc_max_pool(_fp(top), top_h, _ip(mask), _fp(btm), btm_h, channel)
  return top, mask


def pad(x, child, val=0.0):
  x, child = _f32(x), _i32(child)
  channel, hx = x.shape
  y = np.empty((channel, child.size), np.float32)
  lib().oc_pad(_fp(y), child.size, channel, _fp(x), hx, _ip(child), val)
  return y


def depad(y, child, hx):
  y, child = _f32(y), _i32(child)
  channel = y.shape[0]
  x = np.zeros((channel, hx), np.float32)
  lib().oc_depad(_fp(x), hx, channel, _fp(y), child.size, _ip(child))
  return x


# -- the generative path's octree editing ----------------------------------------------------------
# Restated from pytorch/cpp/octree_grow.cpp and the OctreeInfo setters it calls
# (octree/octree/octree_info.cpp:188-268).  Header field offsets: octree_info.h:93-116.
_OFF = dict(batch=16, depth=20, full=24, adp_layer=28, is_adaptive=32, key2xyz=44, node_dis=45,
            nnum=48, nnum_cum=112, nnum_nempty=176, flags=240, channels=244, locations=308,
            bbmin=372, bbmax=384, ptr_dis=652)


def _hdr_i32(hdr, name, n=1):
  off = _OFF[name]
  return hdr[off:off + 4 * n].view(np.int32)


def _finish_header(hdr, key_bits):
  """set_nnum_cum() (capacity 0) and set_ptr_dis() (octree_info.cpp:216-223, 254-268)."""
  depth = int(_hdr_i32(hdr, 'depth')[0])
  nnum, cum = _hdr_i32(hdr, 'nnum', 16), _hdr_i32(hdr, 'nnum_cum', 16)
  cum[0] = 0
  for d in range(1, depth + 2):
    cum[d] = cum[d - 1] + nnum[d - 1]
  cum[depth + 2] = cum[depth + 1]
  ch, lc, dis = _hdr_i32(hdr, 'channels', 6), _hdr_i32(hdr, 'locations', 6), _hdr_i32(hdr, 'ptr_dis', 7)
  dis[0] = 720
  for p in range(6):
    n = int(cum[depth + 2]) if lc[p] == -1 else int(nnum[lc[p]])
    esz = key_bits // 8 if p == 0 else 4
    dis[p + 1] = dis[p] + esz * n * ch[p]


def octree_new(batch_size, channel, node_dis=False, adaptive_layer=0, key_bits=64):
  """octree_new (octree_grow.cpp:108-148): `batch_size` root nodes, depth 0 (full_layer clamps to
  1, octree_info.cpp:192-194), xyz keys, Key/Child/Neigh(8)/Feature(channel) on every level, box
  [0,2]^3; key and child of level 0 are 0..batch-1, neigh and feature stay zero."""
  hdr = np.zeros(720, np.uint8)
  hdr[:12] = np.frombuffer(b'_OCTREE_2.0_' if key_bits == 64 else b'_OCTREE_1.0_', np.uint8)
  _hdr_i32(hdr, 'batch')[0] = batch_size
  _hdr_i32(hdr, 'depth')[0] = 0
  _hdr_i32(hdr, 'full')[0] = 1
  hdr[_OFF['node_dis']] = 1 if node_dis else 0
  if adaptive_layer > 1:
    hdr[_OFF['is_adaptive']] = 1
    _hdr_i32(hdr, 'adp_layer')[0] = adaptive_layer
  hdr[_OFF['key2xyz']] = 1
  ch, lc = _hdr_i32(hdr, 'channels', 6), _hdr_i32(hdr, 'locations', 6)
  flags = 0
  for p, c in enumerate((1, 1, 8, channel)):
    ch[p] = c
    lc[p] = -1
    # set_channel records the property in content_flags when it has channels (octree_info.cpp:232-243)
    if c != 0:
      flags |= 1 << p
  _hdr_i32(hdr, 'flags')[0] = flags
  hdr[_OFF['bbmax']:_OFF['bbmax'] + 12].view(np.float32)[:] = 2.0
  _hdr_i32(hdr, 'nnum', 16)[0] = batch_size
  _hdr_i32(hdr, 'nnum_nempty', 16)[0] = batch_size
  _finish_header(hdr, key_bits)
  size = int(_hdr_i32(hdr, 'ptr_dis', 7)[6])
  out = np.zeros(size, np.uint8)
  out[:720] = hdr
  v = OctreeView(out)
  kdt = np.uint64 if key_bits == 64 else np.uint32
  out[v.ptr_dis[0]:v.ptr_dis[0] + batch_size * (key_bits // 8)].view(kdt)[:] = np.arange(batch_size)
  out[v.ptr_dis[1]:v.ptr_dis[1] + 4 * batch_size].view(np.int32)[:] = np.arange(batch_size)
  return out


def _lanes(keys, key_bits):
  """[n, 4] view of the four lanes of xyz keys (uint8 lanes for 32-bit keys, uint16 for 64-bit)."""
  return keys.view(np.uint16 if key_bits == 64 else np.uint8).reshape(-1, 4)


def octree_grow(octree, target_depth, full_octree):
  """octree_grow (octree_grow.cpp:8-104): a copy of the octree with level `target_depth` added —
  eight children under every non-empty node of the level above (all nodes when full_octree).
  New keys are xyz keys: child j of a node doubles the parent's x,y,z lanes and appends the bits of
  j (generate_key_cpu, octree_nn.cpp:428-444), or, for a full level, de-interleaves the node's
  index (:446-464) with the batch index in lane 3; child = 0..n-1; neigh from the level above
  (calc_neigh_cpu)."""
  vin = OctreeView(octree)
  kb = vin.key_bits
  hdr = np.array(vin.buf[:720], copy=True)
  node_num = int(vin.nnum_nempty[target_depth - 1]) << 3
  full_old = int(_hdr_i32(hdr, 'full')[0])
  _hdr_i32(hdr, 'depth')[0] = max(full_old, target_depth)          # set_depth, octree_info.cpp:188-190
  if full_octree:
    _hdr_i32(hdr, 'full')[0] = max(1, target_depth)
  hdr[_OFF['bbmin']:_OFF['bbmin'] + 12].view(np.float32)[:] = 0.0
  hdr[_OFF['bbmax']:_OFF['bbmax'] + 12].view(np.float32)[:] = float(1 << target_depth)
  _hdr_i32(hdr, 'nnum', 16)[target_depth] = node_num
  _hdr_i32(hdr, 'nnum_nempty', 16)[target_depth] = node_num
  _finish_header(hdr, kb)
  size = int(_hdr_i32(hdr, 'ptr_dis', 7)[6])
  out = np.zeros(size, np.uint8)
  out[:720] = hdr
  vo = OctreeView(out)
  cum = int(vin.nnum_cum[target_depth])
  for p, esz in ((0, kb // 8), (1, 4), (2, 4), (3, 4)):
    nbytes = cum * int(vin.channels[p]) * esz
    out[vo.ptr_dis[p]:vo.ptr_dis[p] + nbytes] = vin.buf[vin.ptr_dis[p]:vin.ptr_dis[p] + nbytes]
  vo = OctreeView(out)
  kdt = np.uint64 if kb == 64 else np.uint32
  key_off = int(vo.ptr_dis[0]) + int(vo.nnum_cum[target_depth]) * (kb // 8)
  child_off = int(vo.ptr_dis[1]) + int(vo.nnum_cum[target_depth]) * 4
  neigh_off = int(vo.ptr_dis[2]) + int(vo.nnum_cum[target_depth]) * 8 * 4
  new_keys = np.zeros(node_num, kdt)
  if full_octree:
    per = 1 << (3 * target_depth)
    k = np.arange(node_num, dtype=np.uint64) % per
    lanes = np.zeros((node_num, 4), np.uint64)
    for d in range(target_depth):
      lanes[:, 0] |= (k & np.uint64(1 << (3 * d + 2))) >> np.uint64(2 * d + 2)
      lanes[:, 1] |= (k & np.uint64(1 << (3 * d + 1))) >> np.uint64(2 * d + 1)
      lanes[:, 2] |= (k & np.uint64(1 << (3 * d + 0))) >> np.uint64(2 * d + 0)
    lanes[:, 3] = np.arange(node_num, dtype=np.uint64) // per
    _lanes(new_keys, kb)[:] = lanes
    neigh = calc_neigh_full(target_depth, vo.batch_size)
  else:
    parent_keys = np.array(vo.prop('key', target_depth - 1), copy=True)
    child = vo.prop('child', target_depth - 1)
    pl = _lanes(parent_keys, kb).astype(np.uint64)
    nl = np.zeros((node_num, 4), np.uint64)
    for i in np.nonzero(child >= 0)[0]:
      for j in range(8):
        r = 8 * int(child[i]) + j
        nl[r, 0] = (pl[i, 0] << 1) | ((j & 4) >> 2)
        nl[r, 1] = (pl[i, 1] << 1) | ((j & 2) >> 1)
        nl[r, 2] = (pl[i, 2] << 1) | (j & 1)
        nl[r, 3] = pl[i, 3]
    _lanes(new_keys, kb)[:] = nl      # (lanes wrap to their width, as the reference's typed stores do)
    neigh = calc_neigh_split(vo.prop('neigh', target_depth - 1).reshape(-1), child, node_num, fill=0)
  out[key_off:key_off + node_num * (kb // 8)] = new_keys.view(np.uint8)
  out[child_off:child_off + 4 * node_num].view(np.int32)[:] = np.arange(node_num)
  out[neigh_off:neigh_off + 4 * neigh.size] = neigh.view(np.uint8)
  return out


def octree_update(octree, label, depth, split):
  """octree_update (octree_grow.cpp:150-177): child[depth][i] = rank among the nodes whose label
  equals `split`, -1 for the others (generate_label, octree_nn.cpp:466-473); their number becomes
  nnum_nempty[depth] (1, with child[0] = 0, when there is none)."""
  out = np.array(octree, dtype=np.uint8, copy=True)
  v = OctreeView(out)
  label = _i32(label)
  n = int(v.nnum[depth])
  assert label.size == n
  hit = label == split
  child = np.where(hit, np.cumsum(hit) - 1, -1).astype(np.int32)
  split_num = int(hit.sum())
  if split_num == 0:
    split_num = 1
    child[0] = 0
  off = int(v.ptr_dis[1]) + int(v.nnum_cum[depth]) * 4
  out[off:off + 4 * n].view(np.int32)[:] = child
  _hdr_i32(out, 'nnum_nempty', 16)[depth] = split_num
  return out
