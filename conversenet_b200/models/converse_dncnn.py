"""Converse-DnCNN (`models/converse_dncnn.py:11-35`)."""
import torch.nn as nn

from ..util_converse import ConverseBlock


class ConverseDnCNN(nn.Module):
    """1x1 head (in->64), 20 ConverseBlocks (k=7, padding 6, circular), 1x1 tail.

    As in the reference the body always has 20 blocks: `num_blocks` is accepted and
    ignored (`models/converse_dncnn.py:24`).

    `activation_dtype` (not in the reference; None = the input's dtype): with torch.bfloat16 the
    parameters stay fp32 and the tensors between the kernels of the body are bf16 (spectra and
    accumulation fp32), which halves the body's memory traffic; head and tail run in fp32."""

    def __init__(self, in_channels=1, kernel_size=7, num_features=64, padding=6, padding_mode="circular",
                 eps=1e-5, num_blocks=20):
        super().__init__()
        self.num_features = num_features
        self.kernel_size = kernel_size
        self.padding = padding
        self.padding_mode = padding_mode
        self.eps = eps
        self.num_blocks = num_blocks
        self.m_head = nn.Sequential(nn.Conv2d(in_channels, num_features, 1, 1, 0))
        self.m_body = nn.Sequential(*[ConverseBlock(num_features, num_features, kernel_size=kernel_size, scale=1,
                                                    padding=padding, padding_mode=padding_mode, eps=1e-5)
                                      for _ in range(20)])
        self.m_tail = nn.Sequential(nn.Conv2d(num_features, in_channels, 1, 1, 0))
        self.activation_dtype = None

    def forward(self, x):
        if self.activation_dtype is None:
            return self.m_tail(self.m_body(self.m_head(x)))
        w = self.m_head[0].weight.dtype
        y = self.m_body(self.m_head(x.to(w)).to(self.activation_dtype))
        return self.m_tail(y.to(w)).to(x.dtype)
