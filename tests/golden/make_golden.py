"""Generate tests/golden/reference_vectors.npz and reference_vectors_general.npz from the
reference's own CPU code.

Run in a container that has the reference checkout (it is compiled unmodified by
``make -C oracle ref``):

    python tests/golden/make_golden.py            # both files
    python tests/golden/make_golden.py general    # only reference_vectors_general.npz
    python tests/golden/make_golden.py samples    # only o-cnn_b200/ocnn/data/octree_samples.npz

Every array written here is an input fed to, or an output produced by, the reference
(``oracle/_ref/libocnn_ref{32,64}.so``); nothing is computed by this repository's own oracle or
CUDA code.  The fixtures let the oracle be pinned on machines where the reference is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'o-cnn_b200'))

from oracle import ref  # noqa: E402
from ocnn_harness import synth  # noqa: E402

KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [1, 3, 1], [1, 1, 3], [3, 3, 1], [3, 1, 3], [1, 3, 3],
           [1, 1, 1]]


def main():
  out = {}
  rng = np.random.default_rng(20240)
  for kb in (32, 64):
    R = ref.get(kb)
    tag = 'k%d_' % kb
    for name in ('octree_1', 'octree_2'):
      out[tag + name] = R.octree_sample(name)
    out[tag + 'merge_samples_12'] = R.octree_batch([out[tag + 'octree_1'], out[tag + 'octree_2']])
    out[tag + 'merge_samples_11'] = R.octree_batch([out[tag + 'octree_1']] * 2)

    # one cloud with every supported signal, two flag combinations
    if kb == 32:
      p, q = synth.primitive_union(250, 11)
      out['a_xyz'], out['a_normal'] = p, q
      out['a_feat'] = rng.normal(size=(250, 2)).astype(np.float32)
      out['a_label'] = rng.integers(-1, 4, size=250).astype(np.float32)
    pts = R.points_new(out['a_xyz'], out['a_normal'], out['a_feat'], out['a_label'])
    if kb == 32:
      out['a_points'] = pts
    out[tag + 'a_octree'] = R.points2octree(pts, 5, 2)
    out[tag + 'a_octree_flags'] = R.points2octree(pts, 5, 2, node_dis=True, split_label=True,
                                                  save_pts=True)
    pts_nn = R.points_new(out['a_xyz'], None, out['a_feat'])
    out[tag + 'a_octree_nonormal'] = R.points2octree(pts_nn, 4, 1, node_dis=True)

    # a merged batch of three clouds and the operators on it
    singles = []
    for i in range(3):
      if kb == 32:
        p, q = synth.primitive_union(120 + 30 * i, 21 + i)
        out['b%d_xyz' % i], out['b%d_normal' % i] = p, q
      singles.append(R.points2octree(R.points_new(out['b%d_xyz' % i], out['b%d_normal' % i]), 4, 2))
      out[tag + 'b%d_octree' % i] = singles[-1]
    merged = R.octree_batch(singles)
    out[tag + 'b_merged'] = merged
    if kb == 32:
      info = R.octree_info(merged)
      d = 4
      H, Hne = int(info['nnum'][d]), int(info['nnum_nempty'][d])
      out['b_x'] = rng.uniform(-1, 1, size=(3, H)).astype(np.float32)
      out['b_xne'] = rng.uniform(-1, 1, size=(3, Hne)).astype(np.float32)
      for ks in KERNELS:
        kd = int(np.prod(ks))
        name = ''.join(map(str, ks))
        out['b_w' + name] = rng.normal(scale=0.2, size=(5, 3 * kd)).astype(np.float32)
        for stride in (1, 2):
          out['b_conv%s_s%d' % (name, stride)] = R.octree_conv(
              out['b_x'], out['b_w' + name], merged, d, 5, ks, stride)
      neigh = merged[info['ptr_dis']['neigh'] + 32 * int(info['nnum_cum'][d]):][:32 * H].view(np.int32)
      child = merged[info['ptr_dis']['child'] + 4 * int(info['nnum_cum'][d]):][:4 * H].view(np.int32)
      out['b_col311_s1'] = R.octree2col(out['b_x'], neigh, [3, 1, 1], 1, H)
      out['b_col222_s2'] = R.octree2col(out['b_x'], neigh, [2, 2, 2], 2, H // 8)
      top, mask = R.max_pool(out['b_x'])
      out['b_pool'], out['b_pool_mask'] = top, mask
      out['b_pad'] = R.pad_forward(out['b_xne'], child, 0.25)
      out['b_depad'] = R.pad_backward(out['b_x'], child, Hne)
      for dd in (1, 2, 3):
        out['neigh_full_d%d_b2' % dd] = R.calc_neigh_full(dd, 2)
      parent, dis = R.neigh_tables()
      out['tbl_parent'], out['tbl_dis'] = parent, dis
      for ks in KERNELS:
        out['tbl_ni' + ''.join(map(str, ks))] = R.ni_table(ks)

  path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'reference_vectors.npz')
  np.savez_compressed(path, **out)
  print('wrote %s: %d arrays, %d bytes' % (path, len(out), os.path.getsize(path)))


GENERAL_KERNELS = [[3, 3, 3], [2, 2, 2], [3, 1, 1], [3, 3, 1], [1, 1, 1]]


def main_general():
  """Convolution and deconvolution forward for every stride / nempty combination, the column
  operators behind them, and the key / search / interpolation helpers, on the merged batch
  `k32_b_merged` of reference_vectors.npz (kept in a file of its own so that the first file's
  bytes never change)."""
  here = os.path.dirname(os.path.abspath(__file__))
  base = dict(np.load(os.path.join(here, 'reference_vectors.npz')))
  R = ref.get(32)
  merged = base['k32_b_merged']
  info = R.octree_info(merged)
  rng = np.random.default_rng(20241)
  out = {}
  d = 3
  H = {k: int(info['nnum'][k]) for k in range(5)}
  Hne = {k: int(info['nnum_nempty'][k]) for k in range(5)}
  out['g_x_full'] = rng.uniform(-1, 1, size=(3, H[d])).astype(np.float32)
  out['g_x_ne'] = rng.uniform(-1, 1, size=(3, Hne[d])).astype(np.float32)
  for ks in GENERAL_KERNELS:
    kd = int(np.prod(ks))
    name = ''.join(map(str, ks))
    out['g_wc' + name] = rng.normal(scale=0.2, size=(5, 3 * kd)).astype(np.float32)
    out['g_wd' + name] = rng.normal(scale=0.2, size=(3, 5 * kd)).astype(np.float32)
    for stride in (1, 2):
      for nempty in (0, 1):
        for deconv in (0, 1):
          x = out['g_x_ne'] if (nempty or (deconv and stride == 2)) else out['g_x_full']
          w = out['g_wd' + name] if deconv else out['g_wc' + name]
          out['g_y%s_s%d_n%d_t%d' % (name, stride, nempty, deconv)] = R.octree_conv_general(
              x, w, merged, d, 5, ks, stride, bool(nempty), bool(deconv))
  path = os.path.join(here, 'reference_vectors_general.npz')
  np.savez_compressed(path, **out)
  print('wrote %s: %d arrays, %d bytes' % (path, len(out), os.path.getsize(path)))


def main_samples():
  """The six small octrees the reference library embeds for its own tests
  (octree/octree/octree_samples.cpp, read through octree::get_one_octree), in both key widths, as
  the package data behind `ocnn.octree_samples`."""
  out = {}
  for kb in (32, 64):
    R = ref.get(kb)
    for i in range(1, 7):
      out['k%d_octree_%d' % (kb, i)] = R.octree_sample('octree_%d' % i)
  path = os.path.join(ROOT, 'o-cnn_b200', 'ocnn', 'data', 'octree_samples.npz')
  os.makedirs(os.path.dirname(path), exist_ok=True)
  np.savez_compressed(path, **out)
  print('wrote %s: %d arrays, %d bytes' % (path, len(out), os.path.getsize(path)))


def main_grow():
  """octree_new / octree_grow / octree_update (pytorch/cpp/octree_grow.cpp) through the compiled
  reference: two octrees grown full to depth 2, then three label-driven levels."""
  here = os.path.dirname(os.path.abspath(__file__))
  out = {}
  for kb in (32, 64):
    R = ref.get(kb)
    rng = np.random.default_rng(77 + kb)
    cur = R.octree_new(2, 4, True, 0)
    out['k%d_new' % kb] = cur
    for d in range(1, 5):
      cur = R.octree_grow(cur, d, d <= 2)
      out['k%d_grow%d' % (kb, d)] = cur
      if d >= 2:
        n = int(R.octree_info(cur)['nnum'][d])
        label = (rng.random(n) < 0.45).astype(np.int32)
        out['k%d_label%d' % (kb, d)] = label
        cur = R.octree_update(cur, label, d, 1)
        out['k%d_update%d' % (kb, d)] = cur
  path = os.path.join(here, 'reference_vectors_grow.npz')
  np.savez_compressed(path, **out)
  print('wrote %s: %d arrays, %d bytes' % (path, len(out), os.path.getsize(path)))


if __name__ == '__main__':
  what = sys.argv[1] if len(sys.argv) > 1 else 'all'
  if what == 'all':
    main()
  if what in ('all', 'general'):
    main_general()
  if what in ('all', 'samples'):
    main_samples()
  if what in ('all', 'grow'):
    main_grow()
