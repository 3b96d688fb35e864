"""Inference forward passes of the networks the benchmark configurations name, assembled from the
octree operators.  Architectures follow the reference's modules (pytorch/ocnn/modules.py:23-139,
resnet.py:5-31, lenet.py:5-32) with BatchNorm in inference mode folded into a per-channel
scale/bias.  Weights are seeded random: no trained checkpoint exists for the PyTorch reference.

Two executors share one parameter set:
  * `GpuNet`  — the CUDA operators of `ocnn` (fp32 channel-major, or bf16 node-major);
  * `CpuNet`  — a numpy chain over a CPU implementation of the operators (the oracle, or the
                compiled reference), used as the checker and as the timed CPU baseline.  It lives
                here so that tests and the benchmark drive both from the same description; it is
                handed its operator module by the caller and imports nothing from oracle/ itself.
"""
import os

import numpy as np

# 1x1x1 layers with few channels go to the streaming pointwise kernel from this many nodes up
# (below it the tensor-core kernel is faster)
PW_MIN_NODES = int(os.environ.get('OCNN_PW_MIN_NODES', '100000'))
# a residual block's conv1x1b + shortcut conv1x1c as one two-input layer (0: two launches)
BLOCK_PAIR = int(os.environ.get('OCNN_BLOCK_PAIR', '1'))
# global pool + FC of the classification networks as one launch of the executor (0: torch ops)
HEAD_FUSED = int(os.environ.get('OCNN_HEAD_FUSED', '1'))
# a level's last 1x1x1 layer and its max-pool as one pass on big levels (0: two launches)
# (the value is the largest output channel count that is fused)
POOL_FUSED = int(os.environ.get('OCNN_POOL_FUSED', '64'))
# a block's conv1x1b and the next block's conv1x1a as one pass on big levels (0: two launches)
CHAIN_FUSED = int(os.environ.get('OCNN_CHAIN_FUSED', '1'))

BN_EPS = 0.001   # pytorch/ocnn/modules.py:5


def _bn_fold(rng, c):
  gamma = rng.uniform(0.5, 1.5, size=c)
  beta = rng.normal(scale=0.1, size=c)
  mean = rng.normal(scale=0.1, size=c)
  var = rng.uniform(0.5, 1.5, size=c)
  scale = gamma / np.sqrt(var + BN_EPS)
  return scale.astype(np.float32), (beta - mean * scale).astype(np.float32)


def _conv_param(rng, cin, cout, kdim, name, bn=True, relu=True):
  """Xavier-uniform weights [cout, cin*kdim] (pytorch/ocnn/octree_conv.py:90-91) + folded BN."""
  bound = np.sqrt(6.0 / (cin * kdim + cout))
  w = rng.uniform(-bound, bound, size=(cout, cin * kdim)).astype(np.float32)
  scale, bias = _bn_fold(rng, cout) if bn else (None, None)
  return {'name': name, 'w': w, 'scale': scale, 'bias': bias, 'relu': relu, 'cin': cin,
          'cout': cout, 'ks': [3, 3, 3] if kdim == 27 else [1, 1, 1]}


def resnet_params(depth=6, channel_in=3, nout=40, resblk_num=2, seed=0, min_depth=2):
  """ResNet O-CNN: conv3x3x3 at `depth`, then per level `resblk_num` bottleneck blocks
  (1x1 -> 3x3x3 at Cout/4 -> 1x1, skip, ReLU; modules.py:110-139) and a max-pool, channels
  2^max(11-d, 2) per level d (resnet.py:9) down to `min_depth`, global average pool, FC.

  With the default min_depth = 2 this is the network the benchmark configuration names (blocks
  on depths 6..2, channels 32-64-128-256-512, the average taken over the 64 nodes of depth 2).  It
  is one level deeper than the reference's own ResNet class, which stops its blocks at depth 3
  (256 channels), max-pools once more and averages depth 2 (resnet.py:12-20); that network is
  `ocnn.ResNet`, checked in the module-route tests."""
  rng = np.random.default_rng(seed)
  ch = lambda d: 2 ** max(11 - d, 2)
  net = {'kind': 'resnet', 'depth': depth, 'min_depth': min_depth, 'channel_in': channel_in,
         'nout': nout}
  net['conv1'] = _conv_param(rng, channel_in, ch(depth), 27, 'conv1')
  levels = []
  cin = ch(depth)
  for d in range(depth, min_depth - 1, -1):
    cout = ch(d)
    blocks = []
    for b in range(resblk_num):
      cb = cout // 4
      blk = {'a': _conv_param(rng, cin, cb, 1, 'd%d.b%d.1x1a' % (d, b)),
             'conv': _conv_param(rng, cb, cb, 27, 'd%d.b%d.3x3' % (d, b)),
             'b': _conv_param(rng, cb, cout, 1, 'd%d.b%d.1x1b' % (d, b), relu=False),
             'c': _conv_param(rng, cin, cout, 1, 'd%d.b%d.1x1c' % (d, b), relu=False)
             if cin != cout else None}
      blocks.append(blk)
      cin = cout
    levels.append({'depth': d, 'blocks': blocks, 'pool': d > min_depth})
  net['levels'] = levels
  bound = 1.0 / np.sqrt(cin)
  net['fc_w'] = rng.uniform(-bound, bound, size=(nout, cin)).astype(np.float32)
  net['fc_b'] = rng.uniform(-bound, bound, size=nout).astype(np.float32)
  return net


def lenet_params(depth=5, channel_in=3, nout=40, seed=0, channels=(32, 64, 128, 256)):
  """LeNet-style classifier: per level conv3x3x3 + BN + ReLU + max-pool from `depth` down to
  level 2, then FC on the flattened 8x8x8... full-level voxels' global average (lenet.py:24-32,
  with the channel plan of the benchmark configuration)."""
  rng = np.random.default_rng(seed)
  net = {'kind': 'lenet', 'depth': depth, 'channel_in': channel_in, 'nout': nout}
  convs = []
  cin = channel_in
  for i, d in enumerate(range(depth, depth - len(channels), -1)):
    convs.append({'depth': d, 'conv': _conv_param(rng, cin, channels[i], 27, 'd%d.conv' % d)})
    cin = channels[i]
  net['convs'] = convs
  net['out_depth'] = depth - len(channels)
  bound = 1.0 / np.sqrt(cin)
  net['fc_w'] = rng.uniform(-bound, bound, size=(nout, cin)).astype(np.float32)
  net['fc_b'] = rng.uniform(-bound, bound, size=nout).astype(np.float32)
  return net


def unet_params(depth=9, channel_in=6, nout=20, seed=0, channels=(32, 64, 128, 256)):
  """Segmentation U-Net of the scene configuration: encoder conv3x3x3 + BN + ReLU per level with
  max-pool between levels (channels 32-64-128-256 over depth .. depth-3), decoder = nearest
  upsampling to the finer level (octree_depad to the non-empty nodes, each repeated for its eight
  children), concatenation with the encoder's output of that level, conv3x3x3 + BN + ReLU, and a
  1x1x1 head to `nout` classes per finest node.  Built from the hot-path operators only (the
  reference's UNet down/up-samples with stride-2 (de)convolutions on non-empty nodes, unet.py:21-36,
  which are outside this path)."""
  rng = np.random.default_rng(seed)
  n = len(channels)
  net = {'kind': 'unet', 'depth': depth, 'channel_in': channel_in, 'nout': nout,
         'channels': list(channels)}
  net['conv1'] = _conv_param(rng, channel_in, channels[0], 27, 'conv1')
  net['enc'] = []
  cin = channels[0]
  for i in range(n):
    net['enc'].append(_conv_param(rng, cin, channels[i], 27, 'enc%d' % (depth - i)))
    cin = channels[i]
  net['dec'] = []
  for i in range(n - 2, -1, -1):
    net['dec'].append(_conv_param(rng, channels[i + 1] + channels[i], channels[i], 27,
                                  'dec%d' % (depth - i)))
  net['head'] = _conv_param(rng, channels[0], nout, 1, 'head', bn=False, relu=False)
  return net


def conv_layers(net):
  """Every convolution of the network with the level it runs at: (depth, param dict)."""
  if net['kind'] == 'lenet':
    return [(c['depth'], c['conv']) for c in net['convs']]
  if net['kind'] == 'unet':
    d, n = net['depth'], len(net['channels'])
    out = [(d, net['conv1'])]
    out += [(d - i, net['enc'][i]) for i in range(n)]
    out += [(d - (n - 2 - k), net['dec'][k]) for k in range(n - 1)]
    out.append((d, net['head']))
    return out
  out = [(net['depth'], net['conv1'])]
  for lv in net['levels']:
    for blk in lv['blocks']:
      for k in ('a', 'conv', 'b', 'c'):
        if blk[k] is not None:
          out.append((lv['depth'], blk[k]))
  return out


# ---- CPU executor ---------------------------------------------------------------------------------
class CpuNet:
  """fp32 forward over a CPU operator module exposing octree_conv / max_pool / pad and an
  OctreeView-like reader (`view`).  `ops` is oracle.oracle or an adapter around the compiled
  reference; the caller chooses."""

  def __init__(self, net, ops, view, round_fn=None):
    """round_fn (e.g. rounding to bf16) is applied to every convolution's input; with `trace` set
    to a list, every convolution appends (name, depth, input as used, output before the skip)."""
    self.net, self.ops, self.view = net, ops, view
    self.round = round_fn
    self.trace = None

  def _conv(self, x, p, octree, d):
    if self.round is not None:
      x = self.round(x)
    y = self._conv_raw(x, p, octree, d)
    if self.trace is not None:
      self.trace.append((p['name'], d, x, y))
    return y

  def _conv_raw(self, x, p, octree, d):
    if p['ks'] == [1, 1, 1]:
      y = p['w'] @ x                      # torch Conv1d(kernel 1) in the reference, modules.py:71-83
    else:
      y = self.ops.octree_conv(x, p['w'], octree, d, p['cout'], p['ks'], 1)
    if p['scale'] is not None:
      y = y * p['scale'][:, None] + p['bias'][:, None]
    return y

  def _pool(self, x, v, d):
    top, _ = self.ops.max_pool(x)
    return self.ops.pad(top, v.prop('child', d - 1), 0.0)

  def _unet(self, octree, v, x):
    net = self.net
    d0, n = net['depth'], len(net['channels'])
    x = np.maximum(self._conv(x, net['conv1'], octree, d0), 0)
    skips = []
    for i in range(n):
      d = d0 - i
      x = np.maximum(self._conv(x, net['enc'][i], octree, d), 0)
      if i < n - 1:
        skips.append(x)
        x = self._pool(x, v, d)
    for k in range(n - 1):
      d = d0 - (n - 2 - k)                 # level being reconstructed
      child = v.prop('child', d - 1)
      nne = int(v.nnum_nempty[d - 1])
      up = np.repeat(self.ops.depad(x, child, nne), 8, axis=1)
      x = np.concatenate([up, skips[n - 2 - k]], axis=0)
      x = np.maximum(self._conv(x, net['dec'][k], octree, d), 0)
    return self._conv(x, net['head'], octree, d0).T          # [nnum[depth], nout]

  def forward(self, octree):
    net = self.net
    v = self.view(octree)
    x = np.ascontiguousarray(v.prop('feature', net['depth']))
    if net['kind'] == 'unet':
      return self._unet(octree, v, x)
    if net['kind'] == 'lenet':
      for c in net['convs']:
        x = np.maximum(self._conv(x, c['conv'], octree, c['depth']), 0)
        x = self._pool(x, v, c['depth'])
      d_out = net['out_depth']
    else:
      x = np.maximum(self._conv(x, net['conv1'], octree, net['depth']), 0)
      for lv in net['levels']:
        d = lv['depth']
        for blk in lv['blocks']:
          y = np.maximum(self._conv(x, blk['a'], octree, d), 0)
          y = np.maximum(self._conv(y, blk['conv'], octree, d), 0)
          y = self._conv(y, blk['b'], octree, d)
          skip = x if blk['c'] is None else self._conv(x, blk['c'], octree, d)
          x = np.maximum(y + skip, 0)
        if lv['pool']:
          x = self._pool(x, v, d)
      d_out = net['min_depth'] if not net['levels'][-1]['pool'] else net['min_depth'] - 1
    per = 8 ** d_out
    pooled = x.reshape(x.shape[0], -1, per).mean(axis=2)        # FullOctreeGlobalPool
    return pooled.T @ net['fc_w'].T + net['fc_b']


# ---- GPU executor ---------------------------------------------------------------------------------
class GpuNet:
  """Forward on the CUDA operators.  mode = 'fp32' (reference layout, parity path) or 'bf16'
  (node-major activations; 3x3x3 and 1x1 convolutions on the tensor-core kernel when
  `tensor_core` is set and the shape allows, fp32-accumulating CUDA-core kernel otherwise)."""

  def __init__(self, net, mode='bf16', tensor_core=True, device='cuda', executor=True):
    import torch
    import ocnn
    self.torch, self.ocnn = torch, ocnn
    self.net, self.mode = net, mode
    self.bf16 = mode == 'bf16'
    self.device = device
    self.status = torch.zeros(1, dtype=torch.int32, device=device)
    self.tc = bool(tensor_core) and self.bf16
    for _, p in conv_layers(net):
      self._upload(p)
    if self.tc and BLOCK_PAIR and net['kind'] == 'resnet':
      for lv in net['levels']:
        for blk in lv['blocks']:
          self._pair(blk)
    if net['kind'] != 'unet':
      self.fc_w = torch.from_numpy(net['fc_w']).to(device)
      self.fc_b = torch.from_numpy(net['fc_b']).to(device)
    self.launches = 0
    self.exec = self._record() if (self.bf16 and executor and net['kind'] != 'unet') else None
    # per-layer CUDA-event tracing (benchmark only): trace = {layer name: [(start, end), ...]};
    # trace_only restricts it to one layer
    self.trace = None
    self.trace_only = None

  def error_status(self):
    """Non-zero if a tensor-core kernel gave up on a bounded wait (never expected)."""
    code = int(self.status.item())
    if self.exec is not None:
      code = code or int(self.exec.status())
    return code

  def _record(self):
    """The bf16 forward as one recorded op sequence for ocnn.nn.NetExecutor (C++ replay: no Python
    between the kernel launches).  Activation slots are recycled: 0/1 ping-pong the block
    input/output, 2-4 hold the bottleneck's intermediates and the projected skip."""
    net = self.net
    ex = self.ocnn.nn.NetExecutor()
    self.exec_layers = []

    def conv(p, d, src, dst, relu, res=-1):
      # few-channel 1x1 layers stream through the pointwise kernel on big levels (HBM-bound there),
      # everything else that fits runs on the tensor-core kernel
      ex.add_conv(p['name'], d, p['_cin'], p['_cout'], p['ks'], 1, p['_w'], p['_packed'],
                  p['_scale'], p['_bias'], relu, src, dst, res,
                  PW_MIN_NODES if p["_pointwise"] else -1)
      self.exec_layers.append(p['name'])

    cur, other = 0, 1
    ex.add_feature(net['depth'], (net['channel_in'] + 7) // 8 * 8, cur)
    self.exec_layers.append('feature')
    if net['kind'] == 'lenet':
      for c in net['convs']:
        conv(c['conv'], c['depth'], cur, other, True)
        ex.add_pool(c['depth'], c['conv']['cout'], other, cur)
        self.exec_layers.append('pool%d' % c['depth'])
      self.exec_out_depth = net['out_depth']
    else:
      conv(net['conv1'], net['depth'], cur, other, True)
      cur, other = other, cur
      spare = 5          # third slot of the block input / output rotation (see the pooled layer below)
      for lv in net['levels']:
        d = lv['depth']
        pooled = False
        a_done = False       # this block's conv1x1a was chained onto the previous block's conv1x1b
        for bi, blk in enumerate(lv['blocks']):
          if not a_done:
            conv(blk['a'], d, cur, 2, True)
          a_done = False
          conv(blk['conv'], d, 2, 3, True)
          skip = cur
          pr = blk.get('_pair')
          if pr is not None:
            ex.add_conv_pair(pr['name'], d, pr['cb'], pr['cc'], pr['cout'], pr['packed'], None,
                             pr['bias'], True, 3, cur, other)
            self.exec_layers.append(pr['name'])
            cur, other = other, cur
            continue
          if blk['c'] is not None:
            conv(blk['c'], d, cur, 4, False)
            skip = 4
          p = blk['b']
          if (POOL_FUSED and lv['pool'] and bi == len(lv['blocks']) - 1 and p['_pointwise'] and
              p['_cout'] <= POOL_FUSED):
            # the level's last layer and its max-pool: one pass on big levels (the executor falls
            # back to the two operators through slot `other` elsewhere); the pooled rows go to the
            # rotation's spare slot, the block input `skip` is still being read as the shortcut
            ex.add_conv_pool(p['name'], d, p['_cin'], p['_cout'], p['_w'], p['_packed'], p['_scale'],
                             p['_bias'], True, 3, other, skip, spare, PW_MIN_NODES)
            self.exec_layers.append(p['name'] + '+pool')
            cur, spare = spare, cur
            pooled = True
            continue
          conv(p, d, 3, other, True, skip)
          nxt = lv['blocks'][bi + 1]['a'] if bi + 1 < len(lv['blocks']) else None
          if (CHAIN_FUSED and nxt is not None and p['_pointwise'] and nxt['_pointwise'] and
              (p['_cin'], p['_cout'], nxt['_cout']) in ((8, 32, 8), (16, 64, 16), (16, 32, 8), (8, 16, 8))):
            # the next block's first layer reads exactly the rows this one writes: on big levels
            # both run as one pass (slot 2 is free again: the 3x3x3 layer has consumed it)
            ex.add_chain(nxt['name'], nxt['_cout'], nxt['_w'], nxt['_packed'], nxt['_scale'], nxt['_bias'],
                         True, 2, PW_MIN_NODES, PW_MIN_NODES if nxt['_pointwise'] else -1)
            self.exec_layers[-1] = p['name'] + '+' + nxt['name'].split('.', 1)[1]
            a_done = True
          cur, other = other, cur
        if lv['pool'] and not pooled:
          ex.add_pool(d, lv['blocks'][-1]['b']['cout'], cur, other)
          self.exec_layers.append('pool%d' % d)
          cur, other = other, cur
      self.exec_out_depth = net['min_depth'] if not net['levels'][-1]['pool'] else net['min_depth'] - 1
    # global average pool over the (full) output level + the classifier's Linear layer: one launch
    self.exec_head = False
    if HEAD_FUSED and self.exec_out_depth <= net.get('full_depth', 2):
      c_out = net['fc_w'].shape[1]
      ex.add_head(self.exec_out_depth, c_out, net['fc_w'].shape[0], self.fc_w, self.fc_b, cur, other)
      self.exec_layers.append('head')
      self.exec_head = True
    return ex

  def _traced(self, name, fn):
    if self.trace is None or (self.trace_only is not None and self.trace_only != name):
      return fn()
    t = self.torch
    a, b = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
    a.record()
    out = fn()
    b.record()
    self.trace.setdefault(name, []).append((a, b))
    return out

  def _upload(self, p):
    t = self.torch
    cin = p['cin']
    w = p['w']
    if self.bf16 and cin % 8 != 0:
      # node-major bf16 activations are padded to 8 channels (the octree's 3 normal channels):
      # widen the weight matrix with zero columns to match
      kd = w.shape[1] // cin
      cpad = (cin + 7) // 8 * 8
      wp = np.zeros((w.shape[0], cpad, kd), np.float32)
      wp[:, :cin, :] = w.reshape(w.shape[0], cin, kd)
      w, cin = wp.reshape(w.shape[0], cpad * kd), cpad
    if self.bf16 and p['cout'] % 8 != 0 and p['ks'] == [1, 1, 1] and p['scale'] is None:
      # a head with e.g. 20 classes: widen to the next size the bf16 kernels take (zero rows); the
      # caller slices the extra channels off
      cpad = 8 if p['cout'] <= 8 else 16 if p['cout'] <= 16 else (p['cout'] + 31) // 32 * 32
      wp = np.zeros((cpad, w.shape[1]), np.float32)
      wp[:p['cout']] = w
      w = wp
    p['_cin'] = cin
    p['_cout'] = w.shape[0]
    p['_w'] = t.from_numpy(np.ascontiguousarray(w)).to(self.device)
    p['_scale'] = None if p['scale'] is None else t.from_numpy(p['scale']).to(self.device)
    p['_bias'] = None if p['bias'] is None else t.from_numpy(p['bias']).to(self.device)
    p['_packed'] = None
    # few-channel 1x1 layers stream through the pointwise kernel behind octree_conv; everything
    # else that fits goes to the tensor-core kernel
    cout = p['_cout']
    # (the streaming mma.sync kernel behind octree_conv wins on big levels while Cin * Cout <= 1024:
    # 8 -> 32 + shortcut 0.030 ms against 0.045 and 32 -> 8 0.022 against 0.026 at 972 k nodes,
    # 16 -> 64 + shortcut 0.025 against 0.035 and 64 -> 16 0.019 against 0.021 at 250 k nodes; beyond
    # that its weight fragments no longer fit the registers beside the accumulators)
    p['_pointwise'] = (p['ks'] == [1, 1, 1] and cout in (8, 16, 32, 64) and cin in (8, 16, 32, 64) and
                       cin * cout <= int(os.environ.get('OCNN_PW_PRODUCT_MAX', '1024')))
    if self.tc and cin % 8 == 0 and cout % 8 == 0 and (cout <= 256 or cout % 256 == 0):
      try:
        p['_packed'] = self.ocnn.nn.conv_pack_weights(p['_w'], cin, cout, p['ks'])
      except RuntimeError:
        p['_packed'] = None

  def _pair(self, blk):
    """conv1x1b(y) + conv1x1c(x) of a block with a projected shortcut as ONE 1x1x1 layer over the
    concatenated channels [y | x]: weights [diag(scale_b) Wb | diag(scale_c) Wc], bias_b + bias_c.
    The shortcut tensor is neither written nor read and the block is three launches instead of
    four."""
    t = self.torch
    blk['_pair'] = None
    b, c = blk['b'], blk['c']
    if c is None or b['_packed'] is None or c['_packed'] is None:
      return
    cb, cc, cout = b['_cin'], c['_cin'], b['_cout']
    if cb % 8 or cc % 8 or (cb + cc) in (8, 16, 32) or c['_cout'] != cout:
      return
    if (cb, cc, cout) != (b['cin'], c['cin'], b['cout']):      # padded by _upload
      return
    def scaled(p):
      w = p['w'].reshape(cout, -1).astype(np.float32)
      return w if p['scale'] is None else w * p['scale'][:, None]
    w = np.ascontiguousarray(np.concatenate([scaled(b), scaled(c)], axis=1))
    bias = np.zeros(cout, np.float32)
    for p in (b, c):
      if p['bias'] is not None:
        bias = bias + p['bias']
    try:
      packed = self.ocnn.nn.conv_pack_weights(t.from_numpy(w).to(self.device), cb + cc, cout, [1, 1, 1])
    except RuntimeError:
      return
    blk['_pair'] = {'packed': packed, 'bias': t.from_numpy(bias.astype(np.float32)).to(self.device),
                    'cb': cb, 'cc': cc, 'cout': cout, 'name': b['name']}

  def _conv_pair(self, y, x, pr):
    self.launches += 1
    return self._traced(pr['name'], lambda: self.ocnn.nn.pointwise_conv_tc_pair(
        y, x, pr['packed'], pr['cout'], None, pr['bias'], None, True, self.status))

  def _conv(self, x, p, octree, d, relu, residual=None):
    nn = self.ocnn.nn
    self.launches += 1
    if p['_packed'] is not None and not (p['_pointwise'] and x.shape[2] >= PW_MIN_NODES):
      return self._traced(p['name'], lambda: nn.octree_conv_tc(
          x, p['_packed'], octree, d, p['_cout'], p['ks'], 1, p['_scale'], p['_bias'], residual,
          relu, self.status))
    return self._traced(p['name'], lambda: nn.octree_conv_fused(
        x, p['_w'], octree, d, p['_cout'], p['ks'], 1, p['_scale'], p['_bias'], residual, relu))

  def _pool(self, x, octree, d):
    nn = self.ocnn.nn
    if self.bf16 and x.shape[1] % 8 == 0:
      self.launches += 1
      return nn.octree_max_pool_pad(x, octree, d)          # pool + pad in one kernel
    top, _ = nn.octree_max_pool(x, octree, d)
    self.launches += 2
    return nn.octree_pad(top, octree, d - 1, 0.0)

  def _unet(self, octree, x):
    t, net = self.torch, self.net
    d0, n = net['depth'], len(net['channels'])
    fmt = dict(memory_format=t.channels_last) if self.bf16 else {}
    x = self._conv(x, net['conv1'], octree, d0, True)
    skips = []
    for i in range(n):
      d = d0 - i
      x = self._conv(x, net['enc'][i], octree, d, True)
      if i < n - 1:
        skips.append(x)
        x = self._pool(x, octree, d)
    for k in range(n - 1):
      d = d0 - (n - 2 - k)
      up = self.ocnn.octree_tile(x, octree, d - 1)            # OctreeTile: nearest upsampling
      x = t.cat([up, skips[n - 2 - k]], dim=1).contiguous(**fmt)
      x = self._conv(x, net['dec'][k], octree, d, True)
    y = self._conv(x, net['head'], octree, d0, False)
    return y[0, :net['nout'], :, 0].t().float()               # [nnum[depth], nout]

  def forward(self, octree):
    t, net = self.torch, self.net
    nn = self.ocnn.nn
    if self.exec is not None:
      with t.no_grad():
        x = self.exec.forward(octree)
        if self.exec_head:
          return x                                               # [batch, nout] fp32
        per = 8 ** self.exec_out_depth
        C = x.shape[1]
        pooled = x.permute(0, 2, 1, 3).reshape(-1, per, C).float().mean(dim=1)
        return pooled @ self.fc_w.t() + self.fc_b
    with t.no_grad():
      if self.bf16:
        x = nn.feature_node_major(octree, (net['channel_in'] + 7) // 8 * 8, True)
        self.launches += 1
      else:
        x = self.ocnn.octree_property(octree, 'feature', net['depth'])
      if net['kind'] == 'unet':
        return self._unet(octree, x)
      if net['kind'] == 'lenet':
        for c in net['convs']:
          x = self._conv(x, c['conv'], octree, c['depth'], True)
          x = self._pool(x, octree, c['depth'])
        d_out = net['out_depth']
      else:
        x = self._conv(x, net['conv1'], octree, net['depth'], True)
        for lv in net['levels']:
          d = lv['depth']
          for blk in lv['blocks']:
            y = self._conv(x, blk['a'], octree, d, True)
            y = self._conv(y, blk['conv'], octree, d, True)
            if blk.get('_pair') is not None:
              x = self._conv_pair(y, x, blk['_pair'])
              continue
            skip = x if blk['c'] is None else self._conv(x, blk['c'], octree, d, False)
            x = self._conv(y, blk['b'], octree, d, True, residual=skip)
          if lv['pool']:
            x = self._pool(x, octree, d)
        d_out = net['min_depth'] if not net['levels'][-1]['pool'] else net['min_depth'] - 1
      per = 8 ** d_out
      C = x.shape[1]
      if x.is_contiguous():                                     # [C, B*per]
        pooled = x.view(C, -1, per).float().mean(dim=2).t()
      else:                                                     # node-major [B*per, C]
        pooled = x.permute(0, 2, 1, 3).reshape(-1, per, C).float().mean(dim=1)
      return pooled @ self.fc_w.t() + self.fc_b


# ---- the same networks assembled from the `ocnn` modules (the route a reference user takes) ---------
def module_resnet(net, device='cuda'):
  """A torch.nn.Module built from ocnn.OctreeConvBnRelu / OctreeResBlock / OctreeMaxPool that computes
  the ResNet described by `net` (resnet_params), with the weights and BatchNorm statistics of that
  description loaded: forward(octree, data) -> logits.  Input channels are padded to a multiple of 8
  when `data` is 16-bit channels_last."""
  import torch
  import ocnn

  def load_bn(bn, p):
    # scale / bias of the description are a folded BatchNorm: store them as weight / bias of a
    # BatchNorm with zero mean and unit variance (eps compensated)
    with torch.no_grad():
      bn.weight.copy_(torch.from_numpy(p['scale'] * np.sqrt(1.0 + bn.eps).astype(np.float32)))
      bn.bias.copy_(torch.from_numpy(p['bias']))
      bn.running_mean.zero_()
      bn.running_var.fill_(1.0)

  class Net(torch.nn.Module):
    def __init__(self, cin_pad):
      super().__init__()
      c1 = net['conv1']
      self.cin_pad = cin_pad
      self.conv1 = ocnn.OctreeConvBnRelu(net['depth'], cin_pad, c1['cout'])
      w = np.zeros((c1['cout'], cin_pad, 27), np.float32)
      w[:, :c1['cin']] = c1['w'].reshape(c1['cout'], c1['cin'], 27)
      with torch.no_grad():
        self.conv1.conv.weights.copy_(torch.from_numpy(w.reshape(c1['cout'], -1)))
      load_bn(self.conv1.bn, c1)
      self.levels = torch.nn.ModuleList()
      self.pools = torch.nn.ModuleDict()
      for lv in net['levels']:
        blocks = torch.nn.ModuleList()
        for blk in lv['blocks']:
          m = ocnn.OctreeResBlock(lv['depth'], blk['a']['cin'], blk['b']['cout'])
          with torch.no_grad():
            m.conv1x1a.conv1x1.conv1x1.weight.copy_(torch.from_numpy(blk['a']['w'])[:, :, None])
            m.conv3x3.conv.weights.copy_(torch.from_numpy(blk['conv']['w']))
            m.conv1x1b.conv1x1.conv1x1.weight.copy_(torch.from_numpy(blk['b']['w'])[:, :, None])
            if blk['c'] is not None:
              m.conv1x1c.conv1x1.conv1x1.weight.copy_(torch.from_numpy(blk['c']['w'])[:, :, None])
          load_bn(m.conv1x1a.bn, blk['a'])
          load_bn(m.conv3x3.bn, blk['conv'])
          load_bn(m.conv1x1b.bn, blk['b'])
          if blk['c'] is not None:
            load_bn(m.conv1x1c.bn, blk['c'])
          blocks.append(m)
        self.levels.append(blocks)
        if lv['pool']:
          self.pools[str(lv['depth'])] = ocnn.OctreeMaxPool(lv['depth'])
      self.out_depth = net['min_depth'] if not net['levels'][-1]['pool'] else net['min_depth'] - 1
      self.fc = torch.nn.Linear(net['fc_w'].shape[1], net['fc_w'].shape[0])
      with torch.no_grad():
        self.fc.weight.copy_(torch.from_numpy(net['fc_w']))
        self.fc.bias.copy_(torch.from_numpy(net['fc_b']))

    def forward(self, octree, data):
      x = self.conv1(data, octree)
      for lv, blocks in zip(net['levels'], self.levels):
        for m in blocks:
          x = m(x, octree)
        if lv['pool']:
          x = self.pools[str(lv['depth'])](x, octree)
      per = 8 ** self.out_depth
      pooled = x.float().permute(0, 2, 1, 3).reshape(-1, per, x.shape[1]).mean(dim=1)
      return self.fc(pooled)

  return Net


def module_resnet_build(net, sixteen_bit=True, device='cuda'):
  cin = net['channel_in']
  cin_pad = (cin + 7) // 8 * 8 if sixteen_bit else cin
  return module_resnet(net, device)(cin_pad).to(device).eval()
