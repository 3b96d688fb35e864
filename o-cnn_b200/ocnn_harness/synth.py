"""Seeded synthetic point clouds standing in for the public datasets the reference is evaluated
on (ModelNet40 / ShapeNet-like objects, ScanNet-like indoor scenes).  Only shapes, sizes and value
distributions follow those datasets; no dataset item is reproduced.

All generators return float32 arrays with every coordinate strictly inside (-1, 1): the octree
builder truncates ``(p + 1) * 2^(depth-1)`` to an unsigned cell index, so a coordinate on or
outside the cube has no defined cell (the reference clips its inputs the same way,
pytorch/ocnn/transforms.py:101).
"""
import numpy as np

_INSIDE = 0.999


def _rng(cfg, item):
  return np.random.default_rng(1000 * cfg + item)


def sphere_cloud(npt=10000, seed=1000):
  """Points uniform on the unit sphere with outward normals."""
  rng = np.random.default_rng(seed)
  p = rng.normal(size=(npt, 3))
  p /= np.linalg.norm(p, axis=1, keepdims=True)
  return (p * _INSIDE).astype(np.float32), p.astype(np.float32)


def _sample_sphere(rng, n):
  p = rng.normal(size=(n, 3))
  p /= np.linalg.norm(p, axis=1, keepdims=True)
  return p, p.copy()


def _sample_box(rng, n, half):
  hx, hy, hz = half
  areas = np.array([hy * hz, hy * hz, hx * hz, hx * hz, hx * hy, hx * hy])
  face = rng.choice(6, size=n, p=areas / areas.sum())
  uv = rng.uniform(-1.0, 1.0, size=(n, 3)) * half
  axis = face // 2
  sign = np.where(face % 2 == 0, -1.0, 1.0)
  p = uv
  p[np.arange(n), axis] = sign * np.asarray(half)[axis]
  nrm = np.zeros((n, 3))
  nrm[np.arange(n), axis] = sign
  return p, nrm


def _sample_cylinder(rng, n, radius, half_h):
  side, cap = 2 * np.pi * radius * 2 * half_h, np.pi * radius * radius
  part = rng.choice(3, size=n, p=np.array([side, cap, cap]) / (side + 2 * cap))
  th = rng.uniform(0, 2 * np.pi, size=n)
  r = radius * np.sqrt(rng.uniform(0, 1, size=n))
  z = rng.uniform(-half_h, half_h, size=n)
  on_side = part == 0
  rr = np.where(on_side, radius, r)
  p = np.stack([rr * np.cos(th), rr * np.sin(th),
                np.where(on_side, z, np.where(part == 1, half_h, -half_h))], axis=1)
  nrm = np.stack([np.where(on_side, np.cos(th), 0.0), np.where(on_side, np.sin(th), 0.0),
                  np.where(on_side, 0.0, np.where(part == 1, 1.0, -1.0))], axis=1)
  return p, nrm


def primitive_union(npt, seed, jitter_frac=0.0, jitter_sigma=0.0):
  """Union of 1-4 primitives (sphere / box / cylinder), scale U(0.2, 0.5), random rotation and
  offset, analytic outward normals, normalised to the unit cube.  `jitter_frac` of the points are
  then displaced off the surface by N(0, jitter_sigma^2) per axis."""
  rng = np.random.default_rng(seed)
  nprim = int(rng.integers(1, 5))
  share = rng.dirichlet(np.full(nprim, 4.0))
  counts = np.floor(share * npt).astype(int)
  counts[0] += npt - counts.sum()
  pts, nrms = [], []
  for k in range(nprim):
    kind = int(rng.integers(0, 3))
    s = rng.uniform(0.2, 0.5)
    n = int(counts[k])
    if kind == 0:
      p, q = _sample_sphere(rng, n)
      p = p * s
    elif kind == 1:
      p, q = _sample_box(rng, n, s * rng.uniform(0.5, 1.0, size=3))
    else:
      p, q = _sample_cylinder(rng, n, s * rng.uniform(0.4, 1.0), s)
    rot, _ = np.linalg.qr(rng.normal(size=(3, 3)))
    off = rng.uniform(-0.3, 0.3, size=3)
    pts.append(p @ rot.T + off)
    nrms.append(q @ rot.T)
  p = np.concatenate(pts)
  q = np.concatenate(nrms)
  p -= 0.5 * (p.max(0) + p.min(0))
  p *= _INSIDE / np.abs(p).max()
  if jitter_frac > 0:
    pick = rng.uniform(size=npt) < jitter_frac
    p[pick] += rng.normal(scale=jitter_sigma, size=(int(pick.sum()), 3))
    p = np.clip(p, -_INSIDE, _INSIDE)
  order = rng.permutation(npt)
  return p[order].astype(np.float32), q[order].astype(np.float32)


def indoor_scene(npt, seed):
  """A 10 x 10 x 3 m room: floor, 4 walls, 20-40 axis-aligned boxes, N(0, 0.01^2) m noise;
  returns xyz scaled into (-1,1)^3 by the largest half extent, unit normals and RGB in [0,1]."""
  rng = np.random.default_rng(seed)
  ext = np.array([10.0, 10.0, 3.0])
  nbox = int(rng.integers(20, 41))
  size = rng.uniform(0.3, 1.5, size=(nbox, 3)) * np.array([1.0, 1.0, 0.8])
  cen = np.stack([rng.uniform(0.8, 9.2, nbox), rng.uniform(0.8, 9.2, nbox), 0.5 * size[:, 2]], 1)
  box_area = 2 * (size[:, 0] * size[:, 1] + size[:, 0] * size[:, 2] + size[:, 1] * size[:, 2])
  surf_area = np.concatenate([[100.0], np.full(4, 30.0), box_area])
  which = rng.choice(surf_area.size, size=npt, p=surf_area / surf_area.sum())
  p = np.zeros((npt, 3))
  q = np.zeros((npt, 3))
  col = np.zeros((npt, 3))
  palette = rng.uniform(0.1, 0.9, size=(surf_area.size, 3))
  m = which == 0
  p[m] = np.stack([rng.uniform(0, 10, m.sum()), rng.uniform(0, 10, m.sum()), np.zeros(m.sum())], 1)
  q[m] = [0, 0, 1]
  for w in range(4):
    m = which == 1 + w
    k = int(m.sum())
    a, h = rng.uniform(0, 10, k), rng.uniform(0, 3, k)
    fixed = 0.0 if w % 2 == 0 else 10.0
    if w < 2:
      p[m] = np.stack([np.full(k, fixed), a, h], 1)
      q[m] = [1.0 if w == 0 else -1.0, 0, 0]
    else:
      p[m] = np.stack([a, np.full(k, fixed), h], 1)
      q[m] = [0, 1.0 if w == 2 else -1.0, 0]
  for b in range(nbox):
    m = which == 5 + b
    k = int(m.sum())
    if k == 0:
      continue
    bp, bq = _sample_box(rng, k, 0.5 * size[b])
    p[m] = bp + cen[b]
    q[m] = bq
  col[:] = palette[which] + rng.normal(scale=0.03, size=(npt, 3))
  p += rng.normal(scale=0.01, size=p.shape)
  p = (p - 0.5 * ext) / (0.5 * ext.max())
  p = np.clip(p, -_INSIDE, _INSIDE)
  return (p.astype(np.float32), q.astype(np.float32), np.clip(col, 0, 1).astype(np.float32))


def config_clouds(cfg, count=None):
  """The seeded inputs of benchmark configuration `cfg` (1..5): list of (xyz, normals, features)."""
  out = []
  if cfg == 1:
    p, q = sphere_cloud(10000, 1000)
    return [(p, q, None)]
  if cfg in (2, 3):
    npt = 10000 if cfg == 2 else 20000
    for i in range(count or 32):
      p, q = primitive_union(npt, 1000 * cfg + i)
      out.append((p, q, None))
  elif cfg == 4:
    for i in range(count or 64):
      p, q = primitive_union(100000, 4000 + i, jitter_frac=0.05, jitter_sigma=0.005)
      out.append((p, q, None))
  elif cfg == 5:
    for i in range(count or 8):
      p, q, c = indoor_scene(200000, 5000 + i)
      out.append((p, q, c))
  else:
    raise ValueError('unknown configuration %r' % (cfg,))
  return out
