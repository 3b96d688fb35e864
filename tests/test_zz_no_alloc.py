"""ocnn_octree_batch_noalloc — the merge entry point that keeps its scratch table inside the
library instead of taking a workspace — must produce exactly what ocnn_octree_batch produces.

Some users of the library cannot obtain device memory at the moment they need to merge octrees
(their framework's allocator already owns the GPU, or they are inside a region where cudaMalloc is
not permitted); for them the library carries a fixed 144 KiB table.  This test drives both entry
points through the C ABI with ctypes (torch only supplies device buffers), twice in a row with
different batches, so that the second call runs over the first call's leftovers.

It lives in a file that pytest collects last: a failure here cannot hide the other tests from a
run that stops at the first failure.
"""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle as oc
from ocnn_harness import synth

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, 'o-cnn_b200', 'libocnn_b200.so')


class Meta(ctypes.Structure):
  _fields_ = [('key_bits', ctypes.c_int32), ('batch_size', ctypes.c_int32),
              ('depth', ctypes.c_int32), ('full_depth', ctypes.c_int32),
              ('is_adaptive', ctypes.c_int32), ('key2xyz', ctypes.c_int32),
              ('has_node_dis', ctypes.c_int32), ('save_pts', ctypes.c_int32),
              ('nnum', ctypes.c_int32 * 16), ('nnum_cum', ctypes.c_int32 * 18),
              ('nnum_nempty', ctypes.c_int32 * 16), ('channels', ctypes.c_int32 * 6),
              ('locations', ctypes.c_int32 * 6), ('ptr_dis', ctypes.c_int64 * 7)]


def load():
  L = ctypes.CDLL(LIB)
  L.ocnn_last_error.restype = ctypes.c_char_p
  L.ocnn_parse_header.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(Meta)]
  L.ocnn_octree_batch_meta.argtypes = [ctypes.POINTER(Meta), ctypes.c_int, ctypes.POINTER(Meta)]
  L.ocnn_octree_batch_workspace_bytes.restype = ctypes.c_size_t
  L.ocnn_octree_batch_workspace_bytes.argtypes = [ctypes.c_int, ctypes.c_int]
  vp = ctypes.c_void_p
  L.ocnn_octree_batch.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(Meta), ctypes.c_char_p,
                                  ctypes.c_int, ctypes.POINTER(Meta), vp, ctypes.c_size_t, vp, vp, vp]
  L.ocnn_octree_batch_noalloc.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(Meta),
                                          ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(Meta), vp,
                                          vp, vp]
  return L


def merge_both_ways(L, torch, singles):
  """Run the workspace entry point and the built-in-scratch entry point on the same inputs."""
  batch = len(singles)
  dev = [torch.from_numpy(s).cuda() for s in singles]
  metas = (Meta * batch)()
  for i, s in enumerate(singles):
    raw = s.tobytes()
    assert L.ocnn_parse_header(raw, len(raw), ctypes.byref(metas[i])) == 0, L.ocnn_last_error()
  merged = Meta()
  assert L.ocnn_octree_batch_meta(metas, batch, ctypes.byref(merged)) == 0, L.ocnn_last_error()
  ptrs = (ctypes.c_void_p * batch)(*[d.data_ptr() for d in dev])
  first = singles[0][:720].tobytes()
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  size = int(merged.ptr_dis[6])

  ws_bytes = L.ocnn_octree_batch_workspace_bytes(batch, merged.depth)
  ws = torch.empty(ws_bytes, dtype=torch.uint8, device='cuda')
  out_a = torch.empty(size, dtype=torch.uint8, device='cuda')
  status = L.ocnn_octree_batch(ptrs, metas, first, batch, ctypes.byref(merged), ws.data_ptr(),
                               ws_bytes, out_a.data_ptr(), None, stream)
  assert status == 0, L.ocnn_last_error()

  out_b = torch.empty(size, dtype=torch.uint8, device='cuda')
  hdr = ctypes.create_string_buffer(720)
  status = L.ocnn_octree_batch_noalloc(ptrs, metas, first, batch, ctypes.byref(merged),
                                       out_b.data_ptr(), hdr, stream)
  assert status == 0, L.ocnn_last_error()
  torch.cuda.synchronize()
  return out_a.cpu().numpy(), out_b.cpu().numpy(), np.frombuffer(hdr.raw, np.uint8)


def test_noalloc_merge_equals_workspace_merge_twice():
  import torch
  L = load()
  clouds = [synth.primitive_union(2500 + 200 * i, 950 + i) for i in range(5)]
  singles = [oc.points2octree(oc.points_new(p, q), 6, 2, key_bits=64) for p, q in clouds]
  # first call: 5 octrees; second call: 3 other octrees (fewer table entries than the array still
  # holds from the first call), 32-bit keys
  a1, b1, h1 = merge_both_ways(L, torch, singles)
  assert np.array_equal(a1, b1)                      # bit-exact: integer / copy work
  assert np.array_equal(a1, oc.octree_batch(singles))
  assert np.array_equal(h1, b1[:720])
  singles2 = [oc.points2octree(oc.points_new(p, q), 5, 2, key_bits=32) for p, q in clouds[2:]]
  a2, b2, h2 = merge_both_ways(L, torch, singles2)
  assert np.array_equal(a2, b2)
  assert np.array_equal(a2, oc.octree_batch(singles2))
  assert np.array_equal(h2, b2[:720])


def test_noalloc_rejects_requests_beyond_its_table():
  import torch
  L = load()
  p, q = synth.primitive_union(500, 990)
  single = oc.points2octree(oc.points_new(p, q), 7, 2, key_bits=64)
  batch = 300                                         # 300 * (7 + 1) = 2400 > 2048 pairs
  dev = torch.from_numpy(single).cuda()
  metas = (Meta * batch)()
  raw = single.tobytes()
  for i in range(batch):
    assert L.ocnn_parse_header(raw, len(raw), ctypes.byref(metas[i])) == 0
  merged = Meta()
  assert L.ocnn_octree_batch_meta(metas, batch, ctypes.byref(merged)) == 0
  ptrs = (ctypes.c_void_p * batch)(*[dev.data_ptr()] * batch)
  out = torch.empty(int(merged.ptr_dis[6]), dtype=torch.uint8, device='cuda')
  status = L.ocnn_octree_batch_noalloc(ptrs, metas, raw[:720], batch, ctypes.byref(merged),
                                       out.data_ptr(), None, None)
  assert status == 4                                  # OCNN_ERR_CAPACITY
  assert b'exceeds the built-in scratch' in L.ocnn_last_error()
