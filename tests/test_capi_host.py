"""CPU-only checks of the C-ABI library: it loads, exports every symbol the public header declares,
and its host-side logic (header parsing, block offsets, merged-header arithmetic, argument
validation) agrees with the oracle.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import oracle as oc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, 'o-cnn_b200', 'libocnn_b200.so')
HEADER = os.path.join(ROOT, 'include', 'ocnn_b200.h')


class Meta(ctypes.Structure):
  _fields_ = [('key_bits', ctypes.c_int32), ('batch_size', ctypes.c_int32),
              ('depth', ctypes.c_int32), ('full_depth', ctypes.c_int32),
              ('is_adaptive', ctypes.c_int32), ('key2xyz', ctypes.c_int32),
              ('has_node_dis', ctypes.c_int32), ('save_pts', ctypes.c_int32),
              ('nnum', ctypes.c_int32 * 16), ('nnum_cum', ctypes.c_int32 * 18),
              ('nnum_nempty', ctypes.c_int32 * 16), ('channels', ctypes.c_int32 * 6),
              ('locations', ctypes.c_int32 * 6), ('ptr_dis', ctypes.c_int64 * 7)]


@pytest.fixture(scope='module')
def lib():
  assert os.path.exists(LIB), 'build the library first: python o-cnn_b200/build.py'
  L = ctypes.CDLL(LIB)
  L.ocnn_last_error.restype = ctypes.c_char_p
  L.ocnn_prop_offset.restype = ctypes.c_int64
  L.ocnn_prop_offset.argtypes = [ctypes.POINTER(Meta), ctypes.c_int, ctypes.c_int]
  L.ocnn_parse_header.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(Meta)]
  L.ocnn_octree_batch_meta.argtypes = [ctypes.POINTER(Meta), ctypes.c_int, ctypes.POINTER(Meta)]
  L.ocnn_octree_build_workspace_bytes.restype = ctypes.c_size_t
  L.ocnn_octree_build_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                  ctypes.c_int]
  return L


def test_exports_every_declared_symbol(lib):
  text = open(HEADER).read()
  text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
  names = sorted(set(re.findall(r'\b(ocnn_[a-z0-9_]+)\s*\(', text)))
  assert len(names) >= 20
  missing = [n for n in names if not hasattr(lib, n)]
  assert not missing, missing
  assert lib.ocnn_compiled_arch() == 100


def parse(lib, buf):
  m = Meta()
  raw = np.ascontiguousarray(buf, np.uint8).tobytes()
  status = lib.ocnn_parse_header(raw, len(raw), ctypes.byref(m))
  return status, m


@pytest.mark.parametrize('name', ['k32_b_merged', 'k64_b_merged', 'k32_a_octree_flags',
                                  'k64_a_octree_nonormal', 'k64_octree_2'])
def test_parse_header_matches_wire_format(lib, golden, name):
  buf = golden[name]
  status, m = parse(lib, buf)
  assert status == 0, lib.ocnn_last_error()
  v = oc.OctreeView(buf)
  assert (m.key_bits, m.batch_size, m.depth, m.full_depth) == (v.key_bits, v.batch_size, v.depth,
                                                                v.full_depth)
  assert list(m.nnum) == list(v.nnum) and list(m.nnum_nempty) == list(v.nnum_nempty)
  assert list(m.nnum_cum)[:16] == list(v.nnum_cum)
  assert list(m.channels) == list(v.channels[:6])
  assert list(m.ptr_dis) == list(v.ptr_dis[:7]) and m.ptr_dis[6] == buf.size
  for p, pname in enumerate(oc.PROPS):
    for d in range(v.depth + 1):
      want = -1
      if v.has(pname) and (v.locations[p] == -1 or v.locations[p] == d):
        esz = v.key_bits // 8 if pname == 'key' else 4
        want = int(v.ptr_dis[p]) + (int(v.nnum_cum[d]) * int(v.channels[p]) * esz
                                    if v.locations[p] == -1 else 0)
      got = lib.ocnn_prop_offset(ctypes.byref(m), p, d)
      if want >= 0:
        assert got == want, (pname, d)
      elif not v.has(pname):
        assert got == -1


def test_parse_header_rejects_garbage(lib, golden):
  good = golden['k32_b_merged'].copy()
  bad = good.copy()
  bad[:4] = 0
  status, _ = parse(lib, bad)
  assert status == 1 and b'magic' in lib.ocnn_last_error()
  status, _ = parse(lib, good[:100])
  assert status == 1 and b'shorter' in lib.ocnn_last_error()
  bad = good.copy()
  bad[20:24] = np.frombuffer(np.int32(40).tobytes(), np.uint8)   # depth 40
  status, _ = parse(lib, bad)
  assert status == 1 and b'depth' in lib.ocnn_last_error()
  bad = good.copy()
  bad[240:244] = 0                                               # content flags vs channels
  status, _ = parse(lib, bad)
  assert status == 1 and b'content flags' in lib.ocnn_last_error()


@pytest.mark.parametrize('kb', [32, 64])
def test_batch_meta_matches_oracle_merge(lib, golden, kb):
  tag = 'k%d_' % kb
  singles = [golden[tag + 'b%d_octree' % i] for i in range(3)]
  metas = (Meta * 3)()
  for i, s in enumerate(singles):
    status, m = parse(lib, s)
    assert status == 0
    metas[i] = m
  merged = Meta()
  assert lib.ocnn_octree_batch_meta(metas, 3, ctypes.byref(merged)) == 0, lib.ocnn_last_error()
  _, want = parse(lib, golden[tag + 'b_merged'])
  for f, _t in Meta._fields_:
    a, b = getattr(merged, f), getattr(want, f)
    assert (list(a) == list(b)) if hasattr(a, '__len__') else (a == b), f
  # inconsistent inputs are refused, as merge_octrees does (merge_octrees.cpp:27-37)
  _, other = parse(lib, golden[tag + 'a_octree'])
  metas[1] = other
  assert lib.ocnn_octree_batch_meta(metas, 3, ctypes.byref(merged)) == 1
  assert b'not consistent' in lib.ocnn_last_error()


def test_argument_validation_without_gpu(lib):
  ks = (ctypes.c_int * 3)(4, 3, 3)
  one = ctypes.c_void_p(16)
  assert lib.ocnn_octree_conv(one, one, one, one, 8, 8, 3, 5, ks, 1, 0, 0, None, None) == 2
  assert b'unsupported kernel size' in lib.ocnn_last_error()
  ks = (ctypes.c_int * 3)(3, 3, 3)
  assert lib.ocnn_octree_conv(one, one, one, one, 8, 8, 3, 5, ks, 3, 0, 0, None, None) == 1
  assert lib.ocnn_octree_conv(one, one, one, one, 8, 9, 3, 5, ks, 1, 0, 0, None, None) == 1
  assert lib.ocnn_octree_pad(one, one, one, 0, 8, 16, ctypes.c_float(0), 0, 0, None) == 1
  assert lib.ocnn_octree_pad(one, one, one, 3, 17, 16, ctypes.c_float(0), 0, 0, None) == 1
  assert lib.ocnn_calc_neigh_split(one, one, one, 12, None) == 1
  assert lib.ocnn_octree_build_workspace_bytes(0, 1, 5, 2) == 0
  assert lib.ocnn_octree_build_workspace_bytes(10000, 1, 5, 2) > 10000 * 16


def test_extension_loads_and_fails_loudly_without_gpu():
  import torch
  import ocnn
  assert os.path.samefile(ocnn.LIBRARY, LIB)
  if torch.cuda.is_available():
    pytest.skip('CPU-only check')
  pts = ocnn.points_new(torch.rand(10, 3) - 0.5, torch.rand(10, 3), torch.zeros(0), torch.zeros(0))
  assert pts.numel() == 88 + 10 * 24
  with pytest.raises(RuntimeError):
    ocnn.points2octree(pts, 4, 2, False, False, False, False, 4, 0.1, 2.0, False, False, False)
  with pytest.raises(RuntimeError):
    ocnn.nn.octree_pad(torch.zeros(1, 2, 8, 1), torch.zeros(2000, dtype=torch.uint8), 1, 0.0)


@pytest.mark.parametrize('kb', [32, 64])
def test_octree_new_and_grow_header_on_the_host(lib, kb):
  """ocnn_octree_new and ocnn_octree_grow_header are host code: bytes equal to the oracle's
  (itself pinned on the compiled reference), incl. the depth-0 / full-layer-1 header and a
  Feature block without channels."""
  lib.ocnn_octree_new_bytes.restype = ctypes.c_size_t
  for batch, channel, node_dis, adp in ((1, 3, 0, 0), (2, 4, 1, 0), (3, 0, 0, 4)):
    want = oc.octree_new(batch, channel, bool(node_dis), adp, kb)
    n = lib.ocnn_octree_new_bytes(batch, channel, kb)
    assert n == want.size
    buf = ctypes.create_string_buffer(n)
    assert lib.ocnn_octree_new(batch, channel, node_dis, adp, kb, buf, ctypes.c_size_t(n)) == 0, \
        lib.ocnn_last_error()
    assert np.array_equal(np.frombuffer(buf.raw, np.uint8), want)
    cur = want
    for d in (1, 2, 3):
      grown = oc.octree_grow(cur, d, True)
      hdr = ctypes.create_string_buffer(720)
      assert lib.ocnn_octree_grow_header(cur[:720].tobytes(), d, 1, hdr) == 0, lib.ocnn_last_error()
      assert np.array_equal(np.frombuffer(hdr.raw, np.uint8), grown[:720]), d
      cur = grown
    # a partly split level, then a label-driven level
    label = (np.arange(int(oc.OctreeView(cur).nnum[3])) % 3 == 0).astype(np.int32)
    cur = oc.octree_update(cur, label, 3, 1)
    grown = oc.octree_grow(cur, 4, False)
    hdr = ctypes.create_string_buffer(720)
    assert lib.ocnn_octree_grow_header(cur[:720].tobytes(), 4, 0, hdr) == 0, lib.ocnn_last_error()
    assert np.array_equal(np.frombuffer(hdr.raw, np.uint8), grown[:720])
  # a full level cannot follow a level with empty nodes
  assert lib.ocnn_octree_grow_header(cur[:720].tobytes(), 4, 1, hdr) != 0
  assert b'non-empty' in lib.ocnn_last_error()
