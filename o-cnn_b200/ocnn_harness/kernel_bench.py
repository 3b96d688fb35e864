"""Per-kernel measurements of the hot path on one GPU: CUDA-event timings of single operators on
seeded synthetic octrees, reported as achieved algorithmic GB/s or TFLOP/s against the measured
peaks.  Profiler captures of single kernels are taken from this program as well.

    python o-cnn_b200/ocnn_harness/kernel_bench.py conv  --depth 6 --shapes 8 --cin 8 --cout 8
    python o-cnn_b200/ocnn_harness/kernel_bench.py conv  --depth 5 --shapes 32 --cin 128 --cout 128
    python o-cnn_b200/ocnn_harness/kernel_bench.py build --config 4 --clouds 64
    python o-cnn_b200/ocnn_harness/kernel_bench.py merge --config 3
    python o-cnn_b200/ocnn_harness/kernel_bench.py net   --config 5
    python o-cnn_b200/ocnn_harness/kernel_bench.py ops   --depth 6 --shapes 32 --channels 32

Algorithmic work per launch (what `achieved` divides by the measured time):
  conv   flops = 2*Cout*Cin*K*H; bytes = (Cin + Cout)*H*s + 32*H (neighbour indices, K > 1)
         + Cout*Cin*K*s
  build  bytes = N*(12 + 4*C_point) read + octree bytes written (whole plan + emit, incl. neigh)
  neigh  level d: nnum[d-1]*(32 + 4) read + nnum[d]*32 written
  pool   C*nnum*s + C*(nnum/8)*(s + 4);  pad: C*nne*s + nnum*4 + C*nnum*s;  depad: mirror of pad
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
for _p in (ROOT, os.path.join(ROOT, 'o-cnn_b200')):
  if _p not in sys.path:
    sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

import ocnn  # noqa: E402
from ocnn_harness import synth  # noqa: E402


def peaks():
  path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  if os.path.exists(path):
    with open(path) as f:
      pk = json.load(f)
    return pk['hbm_gbs'], pk['bf16_tflops'], 'measured'
  return 6650.0, 1590.0, 'fallback'


def time_op(fn, iters, warmup=5, flush=None):
  """Median and best CUDA-event time of fn() in ms; `flush` (a big tensor) is rewritten before
  each timed call so that L2 holds none of the operands."""
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  times = []
  for _ in range(iters):
    if flush is not None:
      flush.zero_()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    times.append(a.elapsed_time(b))
  times.sort()
  return times[len(times) // 2], times[0]


def make_points(cfg_clouds):
  return [ocnn.points_new(torch.from_numpy(c[0]), torch.from_numpy(c[1]),
                          torch.from_numpy(c[2]) if len(c) > 2 and c[2] is not None else torch.zeros(0),
                          torch.zeros(0)) for c in cfg_clouds]


def build_octree(shapes, npt, depth, seed=7000, key_bits=64):
  ocnn.set_key_bits(key_bits)
  clouds = [synth.primitive_union(npt, seed + i) for i in range(shapes)]
  pts = make_points(clouds)
  return ocnn.points2octree_batch(pts, depth, 2, False, False, False, False, 4, 0.1, 2.0, False,
                                  False, False)


def report(name, ms, best, byts, flops, extra=None):
  hbm, tf, src = peaks()
  out = {'kernel': name, 'ms_median': ms, 'ms_best': best, 'algorithmic_bytes': byts,
         'GBps': byts / (ms * 1e-3) / 1e9, 'hbm_frac': byts / (ms * 1e-3) / 1e9 / hbm,
         'peak_source': src}
  if flops:
    out['TFLOPs'] = flops / (ms * 1e-3) / 1e12
    out['tensor_frac'] = out['TFLOPs'] / tf
  if extra:
    out.update(extra)
  print(json.dumps(out))
  return out


def run_conv(args):
  octree = build_octree(args.shapes, args.points, args.depth)
  info = ocnn.octree_info(octree)
  H = int(info[4 + args.depth])
  ks = [args.kernel] * 3
  K = args.kernel ** 3
  rng = np.random.default_rng(0)
  x = torch.from_numpy(rng.uniform(-1, 1, size=(1, args.cin, H, 1)).astype(np.float32)).cuda()
  x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
  w = torch.from_numpy(rng.normal(scale=0.1, size=(args.cout, args.cin * K)).astype(np.float32)).cuda()
  status = torch.zeros(1, dtype=torch.int32, device='cuda')
  flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if args.flush else None
  flops = 2.0 * args.cout * args.cin * K * H
  byts = (args.cin + args.cout) * H * 2 + (32 * H if K > 1 else 0) + args.cout * args.cin * K * 2
  shape = {'cin': args.cin, 'cout': args.cout, 'taps': K, 'nodes': H, 'depth': args.depth}
  if not args.simt_only:
    packed = ocnn.nn.conv_pack_weights(w, args.cin, args.cout, ks)
    fn = lambda: ocnn.nn.octree_conv_tc(x, packed, octree, args.depth, args.cout, ks, 1, None,
                                        None, None, False, status)
    ms, best = time_op(fn, args.iters, flush=flush)
    assert int(status.item()) == 0
    report('conv_tc_kernel', ms, best, byts, flops, shape)
  if args.simt or args.simt_only:
    fn = lambda: ocnn.nn.octree_conv_fused(x, w, octree, args.depth, args.cout, ks, 1)
    ms, best = time_op(fn, max(3, args.iters // 4), flush=flush)
    report('conv_simt_kernel<bf16,node-major>', ms, best, byts, flops, shape)


def run_build(args):
  kb = 32 if args.config == 4 else 64
  depth = {2: 5, 3: 6, 4: 8, 5: 9}[args.config]
  ocnn.set_key_bits(kb)
  clouds = synth.config_clouds(args.config, args.clouds)
  pts = make_points(clouds)
  packed, meta = ocnn.points_pack(pts, True)
  headers = torch.cat([p[:88] for p in pts]).contiguous()
  dev = packed.cuda()
  bargs = (depth, 2, False, False, False, False, 4, 0.1, 2.0, False, False, False, True)
  fn = lambda: ocnn.points2octree_packed(dev, meta, headers, *bargs)
  octree = fn()
  n = sum(c[0].shape[0] for c in clouds)
  cpt = 3 + (clouds[0][2].shape[1] if clouds[0][2] is not None else 0)
  byts = n * (12 + 4 * cpt) + octree.numel()
  flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if args.flush else None
  ms, best = time_op(fn, args.iters, flush=flush)
  info = ocnn.octree_info(octree)
  n0 = ocnn.nn.launch_count()
  fn()
  report('points2octree+neigh (plan + emit, %d kernels)' % (ocnn.nn.launch_count() - n0), ms, best, byts, 0,
         {'clouds': len(clouds), 'points': n, 'depth': depth, 'key_bits': kb,
          'octree_bytes': int(octree.numel()), 'finest_nodes': int(info[4 + depth]),
          'clouds_per_s': len(clouds) / (ms * 1e-3), 'points_per_s': n / (ms * 1e-3)})
  ocnn.set_key_bits(64)


def run_merge(args):
  """octree_batch over octrees built one by one: the route for octrees that were not built by the
  fused batch build (the merged result is the same)."""
  kb = 32 if args.config == 4 else 64
  depth = {2: 5, 3: 6, 4: 8, 5: 9}[args.config]
  ocnn.set_key_bits(kb)
  clouds = synth.config_clouds(args.config, args.clouds)
  pts = make_points(clouds)
  singles = [ocnn.nn.points2octree(p, depth, 2, False, False, False, False, 4, 0.1, 2.0, False,
                                   False, False) for p in pts]
  fn = lambda: ocnn.nn.octree_batch(singles)
  merged = fn()
  byts = sum(int(t.numel()) for t in singles) + int(merged.numel())
  flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if args.flush else None
  ms, best = time_op(fn, args.iters, flush=flush)
  report('octree_batch (merge + neighbour table)', ms, best, byts, 0,
         {'octrees': len(singles), 'depth': depth, 'key_bits': kb, 'merged_bytes': int(merged.numel())})
  ocnn.set_key_bits(64)


def run_net(args):
  """Whole forward of the other named configurations: LeNet (config 2: 32 shapes x 10k points,
  depth 5, fp32) and the scene U-Net (config 5: one 200k-point scene, depth 9, bf16), octree build
  included."""
  from ocnn_harness import models
  ocnn.set_key_bits(64)
  if args.config == 2:
    clouds = synth.config_clouds(2, args.clouds)
    depth, net, mode = 5, models.lenet_params(5, 3, 40, seed=0), 'fp32'
  else:
    clouds = synth.config_clouds(5, args.clouds or 1)
    depth, net, mode = 9, models.unet_params(9, 6, 20, seed=0), 'bf16'
  pts = make_points(clouds)
  packed, meta = ocnn.points_pack(pts, True)
  headers = torch.cat([p[:88] for p in pts]).contiguous()
  dev = packed.cuda()
  bargs = (depth, 2, False, False, False, False, 4, 0.1, 2.0, False, False, False, True)
  gnet = models.GpuNet(net, mode)
  fn = lambda: gnet.forward(ocnn.points2octree_packed(dev, meta, headers, *bargs))
  out = fn()
  flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if args.flush else None
  ms, best = time_op(fn, args.iters, warmup=3, flush=flush)
  assert gnet.error_status() == 0
  flops = sum(2.0 * p['cout'] * p.get('_cin', p['cin']) * int(np.prod(p['ks'])) *
              int(ocnn.octree_info(ocnn.points2octree_packed(dev, meta, headers, *bargs))[4 + d])
              for d, p in models.conv_layers(net))
  print(json.dumps({'network': net['kind'], 'config': args.config, 'mode': mode, 'clouds': len(clouds),
                    'ms_median': ms, 'ms_best': best, 'items_per_s': len(clouds) / (ms * 1e-3),
                    'conv_TFLOPs': flops / (ms * 1e-3) / 1e12, 'output_shape': list(out.shape)}))


def run_ops(args):
  octree = build_octree(args.shapes, args.points, args.depth)
  info = ocnn.octree_info(octree)
  d, C = args.depth, args.channels
  H, Hne, Hp = int(info[4 + d]), int(info[20 + d]), int(info[4 + d - 1])
  flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if args.flush else None
  for bf16, nm in ((False, False), (True, True)):
    s = 2 if bf16 else 4
    tag = 'bf16 node-major' if bf16 else 'fp32 channel-major'
    x = torch.rand(1, C, H, 1, device='cuda')
    xne = torch.rand(1, C, Hne, 1, device='cuda')
    if bf16:
      x, xne = x.to(torch.bfloat16), xne.to(torch.bfloat16)
    if nm:
      x = x.contiguous(memory_format=torch.channels_last)
      xne = xne.contiguous(memory_format=torch.channels_last)
    ms, best = time_op(lambda: ocnn.nn.octree_max_pool(x, octree, d), args.iters, flush=flush)
    report('octree_max_pool ' + tag, ms, best, C * H * s + C * (H // 8) * (s + 4), 0, {'nodes': H, 'C': C})
    ms, best = time_op(lambda: ocnn.nn.octree_pad(xne, octree, d, 0.0), args.iters, flush=flush)
    report('octree_pad ' + tag, ms, best, C * Hne * s + H * 4 + C * H * s, 0, {'nodes': H, 'C': C})
    ms, best = time_op(lambda: ocnn.nn.octree_depad(x, octree, d), args.iters, flush=flush)
    report('octree_depad ' + tag, ms, best, C * H * s + H * 4 + C * Hne * s, 0, {'nodes': H, 'C': C})


def main():
  ap = argparse.ArgumentParser()
  sub = ap.add_subparsers(dest='cmd', required=True)
  c = sub.add_parser('conv')
  c.add_argument('--depth', type=int, default=6)
  c.add_argument('--shapes', type=int, default=8)
  c.add_argument('--points', type=int, default=20000)
  c.add_argument('--cin', type=int, default=8)
  c.add_argument('--cout', type=int, default=8)
  c.add_argument('--kernel', type=int, default=3)
  c.add_argument('--iters', type=int, default=20)
  c.add_argument('--simt', action='store_true')
  c.add_argument('--simt-only', action='store_true')
  c.add_argument('--no-flush', dest='flush', action='store_false')
  b = sub.add_parser('build')
  b.add_argument('--config', type=int, default=4, choices=[2, 3, 4, 5])
  b.add_argument('--clouds', type=int, default=None)
  b.add_argument('--iters', type=int, default=10)
  b.add_argument('--no-flush', dest='flush', action='store_false')
  g = sub.add_parser('merge')
  g.add_argument('--config', type=int, default=3, choices=[2, 3, 4, 5])
  g.add_argument('--clouds', type=int, default=None)
  g.add_argument('--iters', type=int, default=10)
  g.add_argument('--no-flush', dest='flush', action='store_false')
  w = sub.add_parser('net')
  w.add_argument('--config', type=int, default=5, choices=[2, 5])
  w.add_argument('--clouds', type=int, default=None)
  w.add_argument('--iters', type=int, default=10)
  w.add_argument('--no-flush', dest='flush', action='store_false')
  o = sub.add_parser('ops')
  o.add_argument('--depth', type=int, default=6)
  o.add_argument('--shapes', type=int, default=32)
  o.add_argument('--points', type=int, default=20000)
  o.add_argument('--channels', type=int, default=32)
  o.add_argument('--iters', type=int, default=20)
  o.add_argument('--no-flush', dest='flush', action='store_false')
  args = ap.parse_args()
  {'conv': run_conv, 'build': run_build, 'merge': run_merge, 'net': run_net, 'ops': run_ops}[args.cmd](args)


if __name__ == '__main__':
  main()
