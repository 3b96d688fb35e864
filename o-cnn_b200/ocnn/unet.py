"""The reference's segmentation U-Net (pytorch/ocnn/unet.py:6-92): a 3x3x3 stem, four encoder
stages (kernel-2 stride-2 convolution down, then residual blocks), four decoder stages (kernel-2
stride-2 deconvolution up, concatenation with the encoder's output of that level, residual blocks),
optional interpolation at query points and a two-layer 1x1 head.  Forward only."""
import torch
from torch import nn as _nn

from .modules import (OctreeConvBnRelu, OctreeDeConvBnRelu, OctreeResBlocks, OctreeResBlock2,
                      OctreeConv1x1BnRelu, OctreeConv1x1, OctreeInterp, octree_feature)


class UNet(_nn.Module):
  def __init__(self, depth, channel_in, nout, nempty=False, interp='linear', use_checkpoint=False):
    super().__init__()
    self.depth, self.channel_in, self.nempty = depth, channel_in, nempty
    self.use_checkpoint = use_checkpoint
    self.config_network()
    enc, dec = self.encoder_channel, self.decoder_channel
    self.stages = len(self.encoder_blocks)
    blocks = lambda d, cin, cout, n: OctreeResBlocks(d, cin, cout, n, self.bottleneck, nempty,
                                                    self.resblk, use_checkpoint)
    self.conv1 = OctreeConvBnRelu(depth, channel_in, enc[0], nempty=nempty)
    self.downsample = _nn.ModuleList(
        OctreeConvBnRelu(depth - i, enc[i], enc[i + 1], kernel_size=[2], stride=2, nempty=nempty)
        for i in range(self.stages))
    self.encoder = _nn.ModuleList(
        blocks(depth - i - 1, enc[i + 1], enc[i + 1], self.encoder_blocks[i]) for i in range(self.stages))
    low = depth - self.stages
    self.upsample = _nn.ModuleList(
        OctreeDeConvBnRelu(low + i, dec[i], dec[i + 1], kernel_size=[2], stride=2, nempty=nempty)
        for i in range(self.stages))
    self.decoder = _nn.ModuleList(
        blocks(low + i + 1, dec[i + 1] + enc[-i - 2], dec[i + 1], self.decoder_blocks[i])
        for i in range(self.stages))
    self.octree_interp = OctreeInterp(depth, interp, nempty)
    self.header = self.make_predict_module(dec[-1], nout)

  def config_network(self):
    self.encoder_channel = [32, 32, 64, 128, 256]
    self.decoder_channel = [256, 256, 128, 96, 96]
    self.encoder_blocks = [2, 3, 4, 6]
    self.decoder_blocks = [2, 2, 2, 2]
    self.bottleneck = 1
    self.resblk = OctreeResBlock2

  def make_predict_module(self, channel_in, channel_out=2, num_hidden=64):
    return _nn.Sequential(OctreeConv1x1BnRelu(channel_in, num_hidden),
                          OctreeConv1x1(num_hidden, channel_out, use_bias=True))

  def forward(self, octree, pts=None, data=None):
    """`data` overrides the octree's stored signal (e.g. a bfloat16 channels_last copy, with the
    channel count padded to what `channel_in` says)."""
    depth = self.depth
    if data is None:
      data = octree_feature(octree, depth, self.nempty)
    assert data.size(1) == self.channel_in
    level = {depth: self.conv1(data, octree)}
    for i in range(self.stages):
      d = depth - i - 1
      level[d] = self.encoder[i](self.downsample[i](level[d + 1], octree), octree)
    d = depth - self.stages
    x = level[d]
    for i in range(self.stages):
      d += 1
      up = self.upsample[i](x, octree)
      fmt = torch.channels_last if up.is_contiguous(memory_format=torch.channels_last) and \
          not up.is_contiguous() else torch.contiguous_format
      x = torch.cat([level[d], up], dim=1).contiguous(memory_format=fmt)
      x = self.decoder[i](x, octree)
    if pts is not None:
      x = self.octree_interp(x, octree, pts)
    logits = self.header(x)
    return logits.squeeze(0).squeeze(-1).t()     # (1, C, H, 1) -> (H, C)
