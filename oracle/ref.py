"""TEST INFRASTRUCTURE ONLY: ctypes driver for the reference's own CPU code.

Loads ``oracle/_ref/libocnn_ref{32,64}.so`` (built by ``oracle/Makefile`` from the unmodified
reference sources behind ``oracle/ref_shim.cpp``).  Only tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import this module; the
shipped library never does.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS = {}

c_float_p = ctypes.POINTER(ctypes.c_float)
c_int_p = ctypes.POINTER(ctypes.c_int)
GEMM_CB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                           c_float_p, c_float_p, c_float_p)


def available(key_bits=32):
  return os.path.exists(os.path.join(_HERE, '_ref', 'libocnn_ref%d.so' % key_bits))


def _fp(a):
  return None if a is None else a.ctypes.data_as(c_float_p)


def _ip(a):
  return None if a is None else a.ctypes.data_as(c_int_p)


def _f32(a):
  return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
  return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


class Ref:
  """One instance per key width (the reference fixes ``uintk`` at compile time,
  octree/octree/types.h:16-24)."""

  def __init__(self, key_bits):
    path = os.path.join(_HERE, '_ref', 'libocnn_ref%d.so' % key_bits)
    self.lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    L = self.lib
    L.ref_key_bits.restype = ctypes.c_int
    assert L.ref_key_bits() == key_bits
    self.key_bits = key_bits
    for name in ('ref_points_new', 'ref_points2octree', 'ref_octree_batch', 'ref_octree_sample',
                 'ref_octree_conv', 'ref_octree_conv_general'):
      getattr(L, name).restype = ctypes.c_long
    L.ref_points_new.argtypes = [c_float_p, c_float_p, c_float_p, c_float_p, ctypes.c_int,
                                 ctypes.c_int, ctypes.c_char_p, ctypes.c_long]
    L.ref_points2octree.argtypes = [ctypes.c_char_p] + [ctypes.c_int] * 7 + [
        ctypes.c_float, ctypes.c_float] + [ctypes.c_int] * 3 + [
        c_float_p, ctypes.c_char_p, ctypes.c_long]
    L.ref_octree_batch.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.c_int,
                                   ctypes.c_char_p, ctypes.c_long]
    L.ref_octree_sample.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_long]
    L.ref_octree_info.argtypes = [ctypes.c_char_p, c_int_p]
    L.ref_calc_neigh_full.argtypes = [c_int_p, ctypes.c_int, ctypes.c_int]
    L.ref_calc_neigh_split.argtypes = [c_int_p, c_int_p, c_int_p, ctypes.c_int]
    L.ref_ni_table.argtypes = [c_int_p, c_int_p]
    L.ref_ni_table.restype = ctypes.c_int
    L.ref_neigh_tables.argtypes = [c_int_p, c_int_p]
    L.ref_octree2col.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 4 + [
        c_int_p, c_int_p, ctypes.c_int, ctypes.c_int]
    L.ref_octree2colP.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 5 + [
        c_int_p, c_int_p, c_int_p, c_int_p, ctypes.c_int, ctypes.c_int]
    L.ref_max_pool.argtypes = [c_float_p, ctypes.c_int, c_int_p, c_float_p, ctypes.c_int,
                               ctypes.c_int]
    L.ref_pad_forward.argtypes = [c_float_p, ctypes.c_int, ctypes.c_int, c_float_p,
                                  ctypes.c_int, c_int_p, ctypes.c_float]
    L.ref_pad_backward.argtypes = [c_float_p, ctypes.c_int, ctypes.c_int, c_float_p,
                                   ctypes.c_int, c_int_p]
    L.ref_octree_conv.argtypes = [c_float_p, ctypes.c_long, c_float_p, c_float_p,
                                  ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                  c_int_p, ctypes.c_int]
    L.ref_octree_conv_general.argtypes = [c_float_p, ctypes.c_long, c_float_p, c_float_p,
                                          ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                          c_int_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    L.ref_col2octree.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 4 + [
        c_int_p, c_int_p, ctypes.c_int, ctypes.c_int]
    L.ref_col2octreeP.argtypes = [c_float_p, c_float_p] + [ctypes.c_int] * 5 + [
        c_int_p, c_int_p, c_int_p, c_int_p, ctypes.c_int, ctypes.c_int]
    L.ref_xyz2key.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    L.ref_key2xyz.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    L.ref_search_key.argtypes = [c_int_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    L.ref_transform_points.argtypes = [ctypes.c_char_p, c_float_p, c_float_p, c_float_p,
                                       ctypes.c_float, ctypes.c_char_p]
    L.ref_clip_points.argtypes = [ctypes.c_char_p, c_float_p, c_float_p, c_int_p]
    L.ref_bounding_box.argtypes = [c_float_p, ctypes.c_int, c_float_p]
    L.ref_set_gemm.argtypes = [ctypes.c_void_p]
    L.ref_octree_new.restype = ctypes.c_long
    L.ref_octree_new.argtypes = [ctypes.c_int] * 4 + [ctypes.c_char_p, ctypes.c_long]
    L.ref_octree_grow.restype = ctypes.c_long
    L.ref_octree_grow.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_long]
    L.ref_octree_update.argtypes = [ctypes.c_char_p, c_int_p, ctypes.c_int, ctypes.c_int]
    self._gemm_cb = None

  # -- buffers ---------------------------------------------------------------------------
  def _sized(self, call):
    n = call(None, 0)
    if n < 0:
      raise ValueError('reference call failed')
    buf = ctypes.create_string_buffer(n)
    m = call(buf, n)
    assert m == n
    return np.frombuffer(buf.raw, dtype=np.uint8).copy()

  def points_new(self, pts, normals=None, feats=None, labels=None):
    pts = _f32(pts)
    normals, feats, labels = _f32(normals), _f32(feats), _f32(labels)
    n = pts.size // 3
    cf = 0 if feats is None else feats.size // n
    return self._sized(lambda o, c: self.lib.ref_points_new(
        _fp(pts), _fp(normals), _fp(feats), _fp(labels), n, cf, o, c))

  def points2octree(self, points, depth, full_depth=2, node_dis=False, node_feature=False,
                    split_label=False, adaptive=False, adp_depth=4, th_normal=0.1,
                    th_distance=2.0, extrapolate=False, save_pts=False, key2xyz=False,
                    bbox=None):
    pbuf = np.ascontiguousarray(points, dtype=np.uint8).tobytes()
    bb = None if bbox is None else _f32(bbox)
    return self._sized(lambda o, c: self.lib.ref_points2octree(
        pbuf, depth, full_depth, int(node_dis), int(node_feature), int(split_label),
        int(adaptive), adp_depth, th_normal, th_distance, int(extrapolate), int(save_pts),
        int(key2xyz), _fp(bb), o, c))

  def octree_batch(self, octrees):
    bufs = [np.ascontiguousarray(o, dtype=np.uint8).tobytes() for o in octrees]
    arr = (ctypes.c_char_p * len(bufs))(*bufs)
    return self._sized(lambda o, c: self.lib.ref_octree_batch(arr, len(bufs), o, c))

  # -- the generative path's octree editing (pytorch/cpp/octree_grow.cpp) ----------------------
  def octree_new(self, batch_size, channel, node_dis=False, adaptive_layer=0):
    return self._sized(lambda o, c: self.lib.ref_octree_new(batch_size, channel, int(node_dis),
                                                            adaptive_layer, o, c))

  def octree_grow(self, octree, target_depth, full_octree):
    buf = np.ascontiguousarray(octree, dtype=np.uint8).tobytes()
    return self._sized(lambda o, c: self.lib.ref_octree_grow(buf, target_depth, int(full_octree), o, c))

  def octree_update(self, octree, label, depth, split):
    buf = ctypes.create_string_buffer(np.ascontiguousarray(octree, dtype=np.uint8).tobytes(),
                                      len(octree))
    label = _i32(label)
    self.lib.ref_octree_update(buf, _ip(label), depth, split)
    return np.frombuffer(buf.raw, dtype=np.uint8).copy()

  def octree_sample(self, name):
    return self._sized(lambda o, c: self.lib.ref_octree_sample(name.encode(), o, c))

  def octree_info(self, octree):
    out = np.zeros(80, dtype=np.int32)
    self.lib.ref_octree_info(np.ascontiguousarray(octree, dtype=np.uint8).tobytes(), _ip(out))
    props = ['key', 'child', 'neigh', 'feature', 'label', 'split']
    return {
        'batch_size': int(out[0]), 'depth': int(out[1]), 'full_depth': int(out[2]),
        'sizeof_octree': int(out[3]), 'content_flags': int(out[4]), 'total_nnum': int(out[5]),
        'sizeof_octinfo': int(out[6]), 'key_bits': int(out[7]),
        'nnum': out[8:24].copy(), 'nnum_cum': out[24:40].copy(), 'nnum_nempty': out[40:56].copy(),
        'channel': {p: int(out[56 + 3 * i]) for i, p in enumerate(props)},
        'location': {p: int(out[57 + 3 * i]) for i, p in enumerate(props)},
        'ptr_dis': {p: int(out[58 + 3 * i]) for i, p in enumerate(props)},
    }

  # -- ops -------------------------------------------------------------------------------
  def calc_neigh_full(self, depth, batch_size):
    out = np.empty(batch_size * (8 ** depth) * 8, dtype=np.int32)
    self.lib.ref_calc_neigh_full(_ip(out), depth, batch_size)
    return out

  def calc_neigh_split(self, neigh, child, nnum_child):
    neigh, child = _i32(neigh), _i32(child)
    # the reference leaves blocks of empty parents untouched; start from a known fill
    out = np.full(nnum_child * 8, -7, dtype=np.int32)
    self.lib.ref_calc_neigh_split(_ip(out), _ip(neigh), _ip(child), child.size)
    return out

  def ni_table(self, ksize):
    ks = _i32(ksize)
    n = self.lib.ref_ni_table(_ip(ks), None)
    out = np.empty(n, dtype=np.int32)
    self.lib.ref_ni_table(_ip(ks), _ip(out))
    return out

  def neigh_tables(self):
    parent, dis = np.empty(512, np.int32), np.empty(64, np.int32)
    self.lib.ref_neigh_tables(_ip(parent), _ip(dis))
    return parent, dis

  def octree2col(self, data, neigh, ksize, stride, height):
    data, neigh = _f32(data), _i32(neigh)
    channel = data.shape[0]
    ni = self.ni_table(ksize)
    kdim = int(np.prod(ksize))
    col = np.empty((channel, kdim, height), dtype=np.float32)
    self.lib.ref_octree2col(_fp(col), _fp(data), channel, height, kdim, stride, _ip(neigh),
                            _ip(ni), height, 0)
    return col

  def octree2col_p(self, data, neigh, child, ksize):
    """octree2colP_cpu with ichild built as the PyTorch binding does (pad_backward of 0..nnum-1)."""
    data, neigh, child = _f32(data), _i32(neigh), _i32(child)
    channel, nne = data.shape
    ni = self.ni_table(ksize)
    kdim = int(np.prod(ksize))
    nnum = child.shape[0]
    ichild = np.zeros((1, max(nne, 1)), dtype=np.float32)
    self.lib.ref_pad_backward(_fp(ichild), nne, 1, _fp(np.arange(nnum, dtype=np.float32)), nnum,
                              _ip(child))
    ichild = ichild.reshape(-1).astype(np.int32)
    col = np.empty((channel, kdim, nne), dtype=np.float32)
    self.lib.ref_octree2colP(_fp(col), _fp(data), channel, nne, nne, kdim, 1, _ip(neigh), _ip(ni),
                             _ip(child), _ip(ichild), nne, 0)
    return col

  def max_pool(self, btm):
    btm = _f32(btm)
    channel, btm_h = btm.shape
    top_h = btm_h // 8
    top = np.empty((channel, top_h), np.float32)
    mask = np.empty((channel, top_h), np.int32)
    self.lib.ref_max_pool(_fp(top), top_h, _ip(mask), _fp(btm), btm_h, channel)
    return top, mask

  def pad_forward(self, x, child, val=0.0):
    x, child = _f32(x), _i32(child)
    channel, hx = x.shape
    y = np.empty((channel, child.size), np.float32)
    self.lib.ref_pad_forward(_fp(y), child.size, channel, _fp(x), hx, _ip(child), val)
    return y

  def pad_backward(self, y, child, hx):
    y, child = _f32(y), _i32(child)
    channel = y.shape[0]
    x = np.zeros((channel, hx), np.float32)
    self.lib.ref_pad_backward(_fp(x), hx, channel, _fp(y), child.size, _ip(child))
    return x

  def set_gemm(self, fn):
    """fn(M, N, K, A, B, C) on raw float pointers, or None for the shim's plain loop."""
    self._gemm_cb = None if fn is None else GEMM_CB(fn)
    self.lib.ref_set_gemm(ctypes.cast(self._gemm_cb, ctypes.c_void_p) if fn else None)

  def octree_conv(self, data, weights, octree, depth, num_output, ksize, stride):
    data, weights = _f32(data), _f32(weights)
    ks = _i32(ksize)
    obuf = np.ascontiguousarray(octree, dtype=np.uint8).tobytes()
    cin = data.shape[0]
    n = self.lib.ref_octree_conv(None, 0, _fp(data), _fp(weights), obuf, depth, cin,
                                 num_output, _ip(ks), stride)
    top = np.zeros((num_output, n // num_output), np.float32)
    self.lib.ref_octree_conv(_fp(top), n, _fp(data), _fp(weights), obuf, depth, cin,
                             num_output, _ip(ks), stride)
    return top


def _general_methods():
  def octree_conv_general(self, data, weights, octree, depth, num_output, ksize, stride=1,
                          nempty=False, deconv=False):
    data, weights = _f32(data), _f32(weights)
    ks = _i32(ksize)
    obuf = np.ascontiguousarray(octree, dtype=np.uint8).tobytes()
    cin = data.shape[0]
    args = (_fp(data), _fp(weights), obuf, depth, cin, num_output, _ip(ks), stride, int(nempty),
            int(deconv))
    n = self.lib.ref_octree_conv_general(None, 0, *args)
    top = np.zeros((num_output, n // num_output), np.float32)
    self.lib.ref_octree_conv_general(_fp(top), n, *args)
    return top

  def _ichild(self, child, n):
    ichild = np.zeros(max(n, 1), np.int32)
    pos = child >= 0
    ichild[child[pos]] = np.nonzero(pos)[0].astype(np.int32)
    return ichild

  def octree2col_general(self, data, neigh, ksize, stride, height, child=None):
    if child is None:
      return self.octree2col(data, neigh, ksize, stride, height)
    data, neigh, child = _f32(data), _i32(neigh), _i32(child)
    channel, octree_h = data.shape
    ni = self.ni_table(ksize)
    kdim = int(np.prod(ksize))
    ichild = self._ichild(child, max(octree_h, height))
    col = np.empty((channel, kdim, height), dtype=np.float32)
    self.lib.ref_octree2colP(_fp(col), _fp(data), channel, height, octree_h, kdim, stride,
                             _ip(neigh), _ip(ni), _ip(child), _ip(ichild), height, 0)
    return col

  def col2octree_general(self, col, neigh, ksize, stride, octree_h, child=None):
    col, neigh = _f32(col), _i32(neigh)
    channel, kdim, height = col.shape
    ni = self.ni_table(ksize)
    data = np.full((channel, octree_h), 7.0, np.float32)     # the call must clear it (n == 0)
    if child is None:
      self.lib.ref_col2octree(_fp(col), _fp(data), channel, height, kdim, stride, _ip(neigh),
                              _ip(ni), height, 0)
    else:
      child = _i32(child)
      ichild = self._ichild(child, max(octree_h, height))
      self.lib.ref_col2octreeP(_fp(col), _fp(data), channel, height, octree_h, kdim, stride,
                               _ip(neigh), _ip(ni), _ip(child), _ip(ichild), height, 0)
    return data

  def _keys(self, a):
    return np.ascontiguousarray(a, dtype=np.uint64 if self.key_bits == 64 else np.uint32)

  def xyz2key(self, xyz, depth):
    xyz = self._keys(xyz)
    out = np.empty_like(xyz)
    self.lib.ref_xyz2key(out.ctypes.data_as(ctypes.c_void_p), xyz.ctypes.data_as(ctypes.c_void_p),
                         xyz.size, depth)
    return out

  def key2xyz(self, key, depth):
    key = self._keys(key)
    out = np.empty_like(key)
    self.lib.ref_key2xyz(out.ctypes.data_as(ctypes.c_void_p), key.ctypes.data_as(ctypes.c_void_p),
                         key.size, depth)
    return out

  def search_key(self, keys, query):
    keys, query = self._keys(keys), self._keys(query)
    idx = np.empty(query.size, np.int32)
    self.lib.ref_search_key(_ip(idx), keys.ctypes.data_as(ctypes.c_void_p), keys.size,
                            query.ctypes.data_as(ctypes.c_void_p), query.size)
    return idx

  def transform_points(self, points, angle, scale, jitter, offset, normal_axis=''):
    buf = ctypes.create_string_buffer(np.ascontiguousarray(points, np.uint8).tobytes())
    a, sc, j = _f32(angle), _f32(scale), _f32(jitter)
    self.lib.ref_transform_points(buf, _fp(a), _fp(sc), _fp(j), ctypes.c_float(offset),
                                  normal_axis.encode())
    return np.frombuffer(buf.raw[:len(points)], np.uint8).copy()

  def clip_points(self, points, bbmin, bbmax):
    buf = ctypes.create_string_buffer(np.ascontiguousarray(points, np.uint8).tobytes())
    npt = int(np.frombuffer(buf.raw[16:20], np.int32)[0])
    mask = np.zeros(npt, np.int32)
    lo, hi = _f32(bbmin), _f32(bbmax)
    self.lib.ref_clip_points(buf, _fp(lo), _fp(hi), _ip(mask))
    return np.frombuffer(buf.raw[:len(points)], np.uint8).copy(), mask

  def bounding_box(self, xyz):
    xyz = _f32(xyz)
    out = np.zeros(6, np.float32)
    self.lib.ref_bounding_box(_fp(xyz), xyz.size // 3, _fp(out))
    return out

  Ref.transform_points, Ref.clip_points, Ref.bounding_box = transform_points, clip_points, bounding_box
  Ref._keys, Ref.xyz2key, Ref.key2xyz, Ref.search_key = _keys, xyz2key, key2xyz, search_key
  Ref.octree_conv_general = octree_conv_general
  Ref._ichild = _ichild
  Ref.octree2col_general = octree2col_general
  Ref.col2octree_general = col2octree_general


_general_methods()


def get(key_bits=32):
  if key_bits not in _LIBS:
    _LIBS[key_bits] = Ref(key_bits)
  return _LIBS[key_bits]
