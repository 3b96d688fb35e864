"""Sharding a batch of independent shapes over the GPUs of one box.

Octrees of different shapes never exchange data (neighbour indices stay inside one octree,
octree/octree/octree_nn.cpp:414; children are rebased per octree, merge_octrees.cpp:136-144), so a
batch splits by shape with no collective on the data path: every rank builds the octree of its own
shapes and runs the network with replicated weights.  Only results (logits) or timings are gathered
afterwards."""


def plan_shards(costs, world_size):
  """Longest-processing-time-first bin packing: shapes sorted by decreasing cost (e.g. point
  count), each assigned to the currently lightest rank.  Deterministic: every rank computes the same
  plan from the same costs.  Returns world_size lists of shape indices, each in increasing order."""
  if world_size < 1:
    raise ValueError('world_size must be positive')
  order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
  load = [0] * world_size
  shards = [[] for _ in range(world_size)]
  for i in order:
    r = min(range(world_size), key=lambda k: (load[k], k))
    shards[r].append(i)
    load[r] += costs[i]
  return [sorted(s) for s in shards]


def gather_rows(local_rows, shard, shards, group=None):
  """Reassemble per-shape result rows computed by each rank into batch order.  `local_rows[j]` is
  the result of shape `shard[j]`.  Uses torch.distributed (any backend) when initialised."""
  import torch.distributed as dist
  if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
    pieces = [list(local_rows)]
  else:
    pieces = [None] * dist.get_world_size(group)
    dist.all_gather_object(pieces, list(local_rows), group=group)
  total = sum(len(s) for s in shards)
  out = [None] * total
  for rank_rows, idx in zip(pieces, shards):
    if len(rank_rows) != len(idx):
      raise RuntimeError('rank returned %d rows for %d shapes' % (len(rank_rows), len(idx)))
    for row, i in zip(rank_rows, idx):
      out[i] = row
  if any(r is None for r in out):
    raise RuntimeError('some shapes were not processed by any rank')
  return out
