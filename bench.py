#!/usr/bin/env python
"""Benchmark of the octree hot path on B200: points -> batch octree (+ neighbour table) ->
ResNet O-CNN depth-6 forward, batch 32 per GPU, bf16 with fp32 accumulation.

    python bench.py [--gpus N] [--steps K] [--warmup W]           # this implementation
    python bench.py --impl reference [--gpus N] [--steps K] [--warmup W]   # reference CPU path

Prints ONE JSON line.  `value` = shapes/s with the point clouds already resident in HBM; `e2e` =
the same step fed from pinned host memory (H2D of the points inside the timed region) with the
logits read back (D2H).  Inputs are seeded synthetic point clouds (no dataset, random weights).
Multi-GPU (launched by torchrun): every rank processes its own 32 shapes — shards are independent,
there is no collective on the data path; the only collective is the max-over-ranks of the timing.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, 'o-cnn_b200')):
  if _p not in sys.path:
    sys.path.insert(0, _p)

BATCH = 32            # shapes per GPU
NPT = 20000           # points per shape
DEPTH, FULL_DEPTH = 6, 2
METRIC = 'resnet_ocnn_d6_forward_throughput'
UNIT = 'shapes/s'
BUILD_ARGS = (DEPTH, FULL_DEPTH, False, False, False, False, 4, 0.1, 2.0, False, False, False)


def parse_args():
  ap = argparse.ArgumentParser()
  ap.add_argument('--gpus', type=int, default=1)
  ap.add_argument('--steps', type=int, default=50)
  ap.add_argument('--warmup', type=int, default=5)
  ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
  ap.add_argument('--no-tensor-core', action='store_true',
                  help='run every convolution on the CUDA-core kernel')
  ap.add_argument('--cpu-sample', type=int, default=32, help='shapes in the CPU baseline sample')
  return ap.parse_args()


def workload_config(n_gpus):
  return {'workload': 'ResNet O-CNN forward incl. octree build, depth 6, full depth 2, '
                      '%d shapes x %d points per GPU, bottleneck blocks x2 per level, '
                      'channels 32-64-128-256-512 over depths 6..2, FC 40' % (BATCH, NPT),
          'shapes_per_gpu': BATCH, 'points_per_shape': NPT, 'depth': DEPTH,
          'global_batch': BATCH * n_gpus, 'parallelism': 'shard-by-shape x%d, no collective' % n_gpus,
          'key_bits': 64,
          'l2': 'flushed between timed steps by a 256 MiB write (outside the timed events)'}


def make_clouds(rank, count=BATCH):
  from ocnn_harness import synth
  return [synth.primitive_union(NPT, 3000 + rank * BATCH + i) for i in range(count)]


# =================================================================================================
# CPU side (oracle / compiled reference): checker and baseline only
# =================================================================================================
class CpuOps:
  """Operator set for the CPU forward: the reference's own compiled CPU code when
  oracle/_ref/libocnn_ref64.so is present, else the C oracle port."""

  def __init__(self, use_blas=True):
    from oracle import oracle as oc
    from oracle import ref
    self.oc = oc
    self.kind = 'port'
    self.R = None
    if ref.available(64):
      self.R = ref.get(64)
      self.kind = 'reference'
      if use_blas:
        import numpy as np

        def gemm(M, N, K, A, B, C):
          a = np.ctypeslib.as_array(A, shape=(M, K))
          b = np.ctypeslib.as_array(B, shape=(K, N))
          c = np.ctypeslib.as_array(C, shape=(M, N))
          np.matmul(a, b, out=c)
        self.R.set_gemm(gemm)

  def points_new(self, p, q):
    return self.oc.points_new(p, q)

  def build(self, pts):
    if self.R is not None:
      return self.R.octree_batch([self.R.points2octree(p, DEPTH, FULL_DEPTH) for p in pts])
    return self.oc.octree_batch([self.oc.points2octree(p, DEPTH, FULL_DEPTH, key_bits=64)
                                 for p in pts])

  def octree_conv(self, x, w, octree, d, cout, ks, stride):
    if self.R is not None:
      return self.R.octree_conv(x, w, octree, d, cout, ks, stride)
    return self.oc.octree_conv(x, w, octree, d, cout, ks, stride)

  def max_pool(self, x):
    return self.R.max_pool(x) if self.R is not None else self.oc.max_pool(x)

  def pad(self, x, child, val):
    return self.R.pad_forward(x, child, val) if self.R is not None else self.oc.pad(x, child, val)


_WORKER = {}


def _worker_init(seed_base, shape_ids):
  from ocnn_harness import models, synth
  ops = CpuOps()
  _WORKER['ops'] = ops
  _WORKER['net'] = models.CpuNet(models.resnet_params(DEPTH, 3, 40, 2, seed=0), ops,
                                 ops.oc.OctreeView)
  _WORKER['pts'] = {i: ops.points_new(*synth.primitive_union(NPT, seed_base + i)) for i in shape_ids}


def _worker_step(shape_ids):
  ops, net = _WORKER['ops'], _WORKER['net']
  if not shape_ids:
    return 0
  octree = ops.build([_WORKER['pts'][i] for i in shape_ids])
  logits = net.forward(octree)
  return int(logits.shape[0])


def cpu_forward_time(sample):
  """Seconds for build + merge + forward of `sample` shapes on ONE core (rank 0's first shapes)."""
  _worker_init(3000, list(range(sample)))
  _worker_step(list(range(min(2, sample))))          # touch code and data once
  t0 = time.perf_counter()
  _worker_step(list(range(sample)))
  return time.perf_counter() - t0, _WORKER['ops'].kind


def run_reference(args):
  rank = int(os.environ.get('RANK', '0'))
  if rank != 0:
    return
  import multiprocessing as mp
  cores = os.cpu_count() or 1
  procs = max(1, min(cores, BATCH))
  # each step = the 32-shape batch split over `procs` worker processes (as the reference's
  # DataLoader workers split the build; the forward is split the same way since inference
  # BatchNorm makes shapes independent)
  shares = [list(range(BATCH))[i::procs] for i in range(procs)]
  ctx = mp.get_context('fork')
  pools = [ctx.Pool(1, initializer=_worker_init, initargs=(3000, share)) for share in shares]
  kind = CpuOps(use_blas=False).kind

  def step():
    res = [pool.apply_async(_worker_step, (share,)) for pool, share in zip(pools, shares)]
    return sum(r.get() for r in res)

  for _ in range(max(1, min(args.warmup, 2))):
    step()
  # bound the run: at most ~90 s of timed work whatever K asks for
  t0 = time.perf_counter()
  step()
  one = time.perf_counter() - t0
  steps = max(1, min(args.steps, int(90.0 / max(one, 1e-3))))
  t0 = time.perf_counter()
  for _ in range(steps):
    n = step()
    assert n == BATCH
  total = time.perf_counter() - t0
  for pool in pools:
    pool.terminate()
  value = BATCH * steps / total
  sample = ('%d timed steps of the full %d-shape batch (build + merge + fp32 forward) over %d '
            'worker processes' % (steps, BATCH, procs))
  line = {'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': steps,
          'warmup': args.warmup, 'ms_per_step': 1e3 * total / steps, 'higher_is_better': True,
          'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
          'impl': 'reference', 'config': workload_config(args.gpus),
          'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': procs, 'kind': kind,
                           'sample': sample},
          'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
          'gpu_launches': 0}
  print(json.dumps(line))


# =================================================================================================
# GPU side
# =================================================================================================
class ClockSampler:
  QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
           'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
           'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

  def __init__(self, gpu_index):
    self.gpu_index = gpu_index
    self.proc = None
    try:
      self.proc = subprocess.Popen(['nvidia-smi', '--query-gpu=' + self.QUERY,
                                    '--format=csv,noheader,nounits', '-lms', '100'],
                                   stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      self.proc = None

  def stop(self):
    if self.proc is None:
      return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
    self.proc.terminate()
    try:
      out, _ = self.proc.communicate(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
      out, _ = self.proc.communicate()
    sm, smax, reasons = [], [], set()
    for row in out.splitlines():
      f = [x.strip() for x in row.split(',')]
      if len(f) < 9 or not f[0].isdigit() or int(f[0]) != self.gpu_index:
        continue
      try:
        sm.append(float(f[1]))
        smax.append(float(f[2]))
      except ValueError:
        continue
      for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown',
                            'sw_power_cap'), f[5:9]):
        if val.lower().startswith('active'):
          reasons.add(name)
    if not sm:
      return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['no samples'], 'samples': 0}
    return {'sm_mhz': statistics.median(sm), 'sm_max_mhz': max(smax), 'reasons': sorted(reasons),
            'samples': len(sm), 'window': 'warm-up + timed + e2e steps'}


def physical_gpu_index(local):
  vis = os.environ.get('CUDA_VISIBLE_DEVICES')
  if vis:
    ids = [v for v in vis.split(',') if v.strip() != '']
    if local < len(ids) and ids[local].strip().isdigit():
      return int(ids[local])
  return local


def conv_work(p, h, nm_bytes=2):
  """Algorithmic work of one convolution launch: flops = 2*Cout*Cin*K*H (the reference's dense
  GEMM count, octree_conv.cpp:287-289); bytes = input + output (+ residual) activations, 32 B of
  neighbour indices per node for 3x3x3, and the weights once."""
  kd = 27 if p['ks'] == [3, 3, 3] else 1
  cin = p['cin']
  flops = 2.0 * p['cout'] * cin * kd * h
  byts = (cin + p['cout']) * h * nm_bytes + (32 * h if kd > 1 else 0) + p['cout'] * cin * kd * nm_bytes
  return flops, byts


def load_peaks():
  path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  if os.path.exists(path):
    with open(path) as f:
      pk = json.load(f)
    return {'hbm_gbs': pk['hbm_gbs'], 'bf16_tflops': pk.get('bf16_tflops_sustained', pk['bf16_tflops']),
            'source': 'measured'}
  return {'hbm_gbs': 6650.0, 'bf16_tflops': 1400.0, 'source': 'fallback'}


def run_ours(args):
  import numpy as np
  import torch
  import ocnn
  from ocnn_harness import models

  rank = int(os.environ.get('RANK', '0'))
  world = int(os.environ.get('WORLD_SIZE', '1'))
  local = int(os.environ.get('LOCAL_RANK', '0'))
  torch.cuda.set_device(local)
  if world > 1:
    import torch.distributed as dist
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
  dev = torch.device('cuda', local)
  ocnn.set_key_bits(64)

  clouds = make_clouds(rank)
  pts = [ocnn.points_new(torch.from_numpy(p), torch.from_numpy(q), torch.zeros(0), torch.zeros(0))
         for p, q in clouds]
  packed_host, meta = ocnn.points_pack(pts, True)
  headers = torch.cat([p[:88] for p in pts]).contiguous()
  packed_dev = packed_host.to(dev)
  net = models.GpuNet(models.resnet_params(DEPTH, 3, 40, 2, seed=0), 'bf16',
                      tensor_core=not args.no_tensor_core, device=dev)
  flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

  def step_resident():
    octree = ocnn.points2octree_packed(packed_dev, meta, headers, *BUILD_ARGS, True)
    return octree, net.forward(octree)

  # End-to-end step: the points come from pinned host memory and the logits go back to pinned host
  # memory, every step.  The copies are double-buffered the way a data loader feeds a GPU: while
  # step k builds and runs on the compute stream, the copy stream already moves the points of step
  # k+1 into the other device buffer, so each timed step contains exactly one H2D of a full batch
  # (the next one's) and one D2H (its own logits).
  copy_stream = torch.cuda.Stream(device=dev)
  dev_bufs = [torch.empty_like(packed_dev) for _ in range(2)]
  copied = [torch.cuda.Event() for _ in range(2)]
  consumed = [torch.cuda.Event() for _ in range(2)]
  logits_host = [torch.empty((BATCH, 40), dtype=torch.float32).pin_memory() for _ in range(2)]
  e2e_state = {'k': 0}
  for ev in consumed:
    ev.record()

  def prefetch(slot):
    with torch.cuda.stream(copy_stream):
      copy_stream.wait_event(consumed[slot])          # the build of two steps ago has read it
      dev_bufs[slot].copy_(packed_host, non_blocking=True)
      copied[slot].record(copy_stream)

  def step_e2e():
    slot = e2e_state['k'] & 1
    if e2e_state['k'] == 0:
      prefetch(slot)
    prefetch(slot ^ 1)
    torch.cuda.current_stream().wait_event(copied[slot])
    octree = ocnn.points2octree_packed(dev_bufs[slot], meta, headers, *BUILD_ARGS, True)
    consumed[slot].record()
    logits_host[slot].copy_(net.forward(octree).float().reshape(BATCH, 40), non_blocking=True)
    e2e_state['k'] += 1

  sampler = ClockSampler(physical_gpu_index(local)) if rank == 0 else None

  # ---- warm-up; one warm-up step is instrumented per layer to find the dominant kernel ----
  layer_ms = {}
  octree, logits = step_resident()
  torch.cuda.synchronize()
  info = ocnn.octree_info(octree)
  nnum = info[4:20]
  net.exec.set_trace(-1)
  step_resident()
  torch.cuda.synchronize()
  for index, ms in net.exec.trace_ms():
    layer_ms[net.exec_layers[index]] = ms
  net.exec.set_trace(-2)
  conv_names = {p['name'] for _, p in models.conv_layers(net.net)}
  top_layer = max((k for k in layer_ms if k in conv_names), key=layer_ms.get)
  top_index = net.exec_layers.index(top_layer)
  for _ in range(max(args.warmup, 3)):
    step_resident()
  torch.cuda.synchronize()
  assert net.error_status() == 0, 'a kernel reported an error status'

  def timed(step_fn, steps):
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()
    for k in range(steps):
      flush.zero_()
      starts[k].record()
      step_fn()
      ends[k].record()
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
    total_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
    if world > 1:
      t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      total_ms = float(t.item())
    return total_ms

  # ---- timed region: K steps, inputs resident in HBM; only the dominant layer carries events ----
  net.exec.set_trace(top_index)
  launches0 = ocnn.nn.launch_count()
  t_host0 = time.perf_counter()
  total_ms = timed(step_resident, args.steps)
  host_ms = (time.perf_counter() - t_host0) * 1e3
  launches = ocnn.nn.launch_count() - launches0
  top_times = [ms for _, ms in net.exec.trace_ms()]
  top_ms = statistics.mean(top_times) if top_times else None
  net.exec.set_trace(-2)

  # ---- end to end: pinned host points -> H2D -> build -> forward -> logits D2H ----
  for _ in range(3):
    step_e2e()
  e2e_ms = timed(step_e2e, args.steps)
  assert all(bool(torch.isfinite(t).all()) for t in logits_host), 'end-to-end logits are not finite'
  clocks = sampler.stop() if sampler else None
  assert net.error_status() == 0, 'a kernel reported an error status'

  if world > 1:
    dist.destroy_process_group()
  if rank != 0:
    return

  shapes = BATCH * world * args.steps
  peaks = load_peaks()
  # roofline of the dominant kernel (the layer with the largest device time in a step)
  layer = {p['name']: (d, p) for d, p in models.conv_layers(net.net)}
  d_top, p_top = layer[top_layer]
  h_top = int(nnum[d_top])
  pp = dict(p_top)
  pp['cin'] = p_top.get('_cin', p_top['cin'])
  flops, byts = conv_work(pp, h_top)
  if p_top is not None and top_layer.endswith('1x1b'):
    byts += p_top['cout'] * h_top * 2            # fused residual read
  roofline = None
  if top_ms:
    ai = flops / byts
    ridge = peaks['bf16_tflops'] * 1e12 / (peaks['hbm_gbs'] * 1e9)
    if ai >= ridge:
      ach = flops / (top_ms * 1e-3) / 1e12
      roofline = {'bound': 'tensor', 'achieved': ach, 'peak': peaks['bf16_tflops'],
                  'unit': 'TFLOP/s', 'frac': ach / peaks['bf16_tflops']}
    else:
      ach = byts / (top_ms * 1e-3) / 1e9
      roofline = {'bound': 'hbm', 'achieved': ach, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                  'frac': ach / peaks['hbm_gbs']}
    # DRAM traffic of this kernel per launch: dram__bytes_read + dram__bytes_write from the ncu
    # capture summarised in profiles/conv_tc_kernel_group_8to32_d6_ncu.md (59.7 B per node at
    # 931 k nodes), scaled by the node count of this launch; only known for that kernel shape
    traffic = None
    if top_layer == 'conv1' and pp['cin'] == 8 and p_top['cout'] == 32:
      traffic = 59.7 * h_top
    roofline.update({'traffic': traffic, 'kernel': 'octree_conv ' + top_layer,
                     'shape': {'cin': pp['cin'], 'cout': p_top['cout'], 'taps': 27 if p_top['ks'][0] == 3 else 1,
                               'nodes': h_top},
                     'ms_per_launch': top_ms, 'algorithmic_bytes': byts, 'flops': flops,
                     'peak_source': peaks['source'],
                     'share_of_step': top_ms / (total_ms / args.steps)})

  line = {'metric': METRIC, 'value': shapes / (total_ms * 1e-3), 'unit': UNIT, 'n_gpus': world,
          'steps': args.steps, 'warmup': max(args.warmup, 3) + 2, 'ms_per_step': total_ms / args.steps,
          'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16',
          'data': 'synthetic', 'config': workload_config(world),
          'e2e': {'value': shapes / (e2e_ms * 1e-3), 'unit': UNIT,
                  'h2d_bytes_per_step': int(packed_host.numel()) * world,
                  'd2h_bytes_per_step': BATCH * 40 * 4 * world,
                  'ms_per_step': e2e_ms / args.steps,
                  'pipeline': 'pinned host buffers; H2D of the next batch on a copy stream while '
                              'this one runs; logits copied back to pinned memory every step'},
          'gpu_launches': int(launches), 'clocks': clocks, 'roofline': roofline,
          'tensor_core_layers': sum(1 for _, p in models.conv_layers(net.net) if p.get('_packed') is not None),
          'layer_ms': {k: round(v, 4) for k, v in layer_ms.items()},
          'finest_nodes': int(nnum[DEPTH]), 'host_ms_per_step_incl_flush': host_ms / args.steps}

  if world == 1:
    sample = max(1, min(args.cpu_sample, BATCH))
    secs, kind = cpu_forward_time(sample)
    line['cpu_baseline'] = {'value': sample / secs, 'unit': UNIT, 'cores': 1, 'kind': kind,
                            'sample': 'build + merge + fp32 forward of the first %d shapes of the '
                                      'batch on one core (%.1f s)' % (sample, secs)}
  else:
    line['cpu_baseline'] = None
  print(json.dumps(line))


def main():
  args = parse_args()
  if args.impl == 'reference':
    for k in ('OMP_NUM_THREADS', 'MKL_NUM_THREADS', 'OPENBLAS_NUM_THREADS'):
      os.environ[k] = '1'
    run_reference(args)
  else:
    run_ours(args)


if __name__ == '__main__':
  main()
