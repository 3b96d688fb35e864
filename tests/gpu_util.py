"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import oracle as oc
from ocnn_harness import synth


def to_cuda_u8(buf):
  return torch.from_numpy(np.ascontiguousarray(buf, np.uint8)).cuda()


def data_cuda(x, node_major=False, bf16=False, half=False):
  """[C,H] numpy -> [1,C,H,1] CUDA tensor in the requested dtype / memory layout."""
  t = torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda().view(1, x.shape[0], x.shape[1], 1)
  if bf16:
    t = t.to(torch.bfloat16)
  if half:
    t = t.to(torch.float16)
  if node_major:
    t = t.contiguous(memory_format=torch.channels_last)
  return t


def to_np(t):
  """[1,C,H,1] tensor (any layout / dtype) -> [C,H] float32 numpy."""
  return t.detach().float().contiguous().view(t.shape[1], t.shape[2]).cpu().numpy()


def bf16_round(x):
  return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.bfloat16).float().numpy()


def half_round(x):
  return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(torch.float16).float().numpy()


def rel_err(a, b):
  """max |a - b| / max |b| over the tensor (the tolerance definition used for convolutions)."""
  denom = float(np.max(np.abs(b)))
  return float(np.max(np.abs(a - b))) / (denom if denom > 0 else 1.0)


def oracle_batch(clouds, depth, full_depth=2, key_bits=64, feats=None, **flags):
  """(list of single octrees, merged octree, list of points buffers) from the CPU oracle."""
  pts, singles = [], []
  for i, c in enumerate(clouds):
    f = c[2] if len(c) > 2 else None
    if feats is not None:
      f = feats[i]
    p = oc.points_new(c[0], c[1], f)
    pts.append(p)
    singles.append(oc.points2octree(p, depth, full_depth, key_bits=key_bits, **flags))
  return singles, oc.octree_batch(singles), pts


def small_clouds(n=3, npt=4000, seed=100):
  return [synth.primitive_union(npt + 300 * i, seed + i) for i in range(n)]
