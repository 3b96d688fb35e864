"""Multi-rank host logic on CPU (gloo, world size 2): the shard plan is identical on every rank,
covers every shape exactly once, balances cost, and results come back in batch order.  Each rank
'processes' its shapes with the CPU oracle so the test needs no GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

from ocnn_harness import shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_is_balanced_and_complete():
  costs = [20000, 5000, 100000, 7000, 64000, 64000, 1000, 30000, 30000]
  for world in (1, 2, 3, 8):
    shards = shard.plan_shards(costs, world)
    assert sorted(i for s in shards for i in s) == list(range(len(costs)))
    loads = [sum(costs[i] for i in s) for s in shards]
    assert max(loads) - min(l for l in loads) <= max(costs)
  assert shard.plan_shards([], 2) == [[], []]
  with pytest.raises(ValueError):
    shard.plan_shards(costs, 0)


def _free_port():
  with socket.socket() as s:
    s.bind(('127.0.0.1', 0))
    return s.getsockname()[1]


def _worker(rank, world, port, npts, out_dir):
  for p in (ROOT, os.path.join(ROOT, 'o-cnn_b200')):
    if p not in sys.path:
      sys.path.insert(0, p)
  import torch.distributed as dist
  from oracle import oracle as oc
  from ocnn_harness import shard as sh, synth
  os.environ['MASTER_ADDR'] = '127.0.0.1'
  os.environ['MASTER_PORT'] = str(port)
  dist.init_process_group('gloo', rank=rank, world_size=world)
  shards = sh.plan_shards(npts, world)
  mine = shards[rank]
  rows = []
  for i in mine:
    p, q = synth.primitive_union(npts[i], 40 + i)
    v = oc.OctreeView(oc.points2octree(oc.points_new(p, q), 5, 2, key_bits=64))
    rows.append([i, int(v.nnum[5]), int(v.nnum_nempty[5])])
  full = sh.gather_rows(rows, mine, shards)
  np.save(os.path.join(out_dir, 'rank%d.npy' % rank), np.array(full))
  dist.barrier()
  dist.destroy_process_group()


def test_two_ranks_gather_in_batch_order(tmp_path):
  npts = [3000, 800, 5000, 1200, 2500, 4000, 600]
  port = _free_port()
  mp.spawn(_worker, args=(2, port, npts, str(tmp_path)), nprocs=2, join=True)
  a = np.load(tmp_path / 'rank0.npy')
  b = np.load(tmp_path / 'rank1.npy')
  assert np.array_equal(a, b)                       # every rank holds the whole batch's results
  assert list(a[:, 0]) == list(range(len(npts)))    # in batch order
  # and they are what a single process computes
  from oracle import oracle as oc
  from ocnn_harness import synth
  for i, n in enumerate(npts):
    p, q = synth.primitive_union(n, 40 + i)
    v = oc.OctreeView(oc.points2octree(oc.points_new(p, q), 5, 2, key_bits=64))
    assert list(a[i]) == [i, int(v.nnum[5]), int(v.nnum_nempty[5])]
