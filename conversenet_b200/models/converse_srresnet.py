"""Converse-SRResNet x4 (`models/converse_srresnet.py:50-80`)."""
import torch.nn as nn
import torch.nn.functional as F

from ..util_converse import Converse2D, ConverseBlock


class ConverseMSRResNet(nn.Module):
    """1x1 (3->64)+GELU, 16 ConverseBlocks (k=5, padding 4, replicate), then twice
    [ConverseBlock, Converse2D(k=2, scale 2, padding 2, replicate, eps 1e-3), GELU], a last
    block, GELU, 1x1 (64->3, no bias), plus the bilinear x4 of the input."""

    def __init__(self, in_channels=3, out_channels=3, num_features=64, num_blocks=16, upscale=4):
        super().__init__()
        self.upscale = upscale
        blk = lambda: ConverseBlock(num_features, num_features, 5, 1, 4, padding_mode="replicate", eps=1e-5)
        self.conv_first = nn.Conv2d(in_channels, num_features, 1, 1, 0, bias=True)
        self.conv_body = nn.Sequential(*[blk() for _ in range(num_blocks)])
        self.upconv1 = blk()
        self.up1 = Converse2D(num_features, num_features, 2, 2, 2, padding_mode="replicate", eps=1e-3)
        self.upconv2 = blk()
        self.up2 = Converse2D(num_features, num_features, 2, 2, 2, padding_mode="replicate", eps=1e-3)
        self.conv_hres = blk()
        self.conv_last = nn.Conv2d(num_features, out_channels, 1, 1, 0, bias=False)
        self.gelu = nn.GELU()

    def _up(self, conv, x):
        # the GELU that follows each upsampling operator runs inside its kernel
        conv.fuse_gelu = True
        try:
            return conv(x)
        finally:
            conv.fuse_gelu = False

    def forward(self, x):
        x1 = self.gelu(self.conv_first(x))
        x1 = self.conv_body(x1)
        x1 = self._up(self.up1, self.upconv1(x1))
        x1 = self._up(self.up2, self.upconv2(x1))
        x1 = self.conv_last(self.gelu(self.conv_hres(x1)))
        x = F.interpolate(x, scale_factor=self.upscale, mode="bilinear", align_corners=False)
        return x1 + x
