"""Short causal convolution over time with one filter per channel, and its per-sequence state (the last ``taps - 1``
inputs), so that a sequence can be fed in portions of any length.

    y_t = [x_t +] b + sum_j w[:, j] * x_(t - taps + 1 + j)        (the last column of w weighs the current token)

Used on a layer's normed input before its mixer (residual form, no bias) and inside state-space mixers (bias and silu).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _native as N


class ShortConv(nn.Module):
    def __init__(self, channels: int, taps: int, bias: bool, device) -> None:
        super().__init__()
        if not 1 <= taps <= 8:
            raise ValueError(f"short convolution of {taps} taps (1 to 8)")
        self.channels, self.taps = channels, taps
        f32 = dict(dtype=torch.float32, device=device)
        self.weight = nn.Parameter(torch.zeros((channels, taps), **f32), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(channels, **f32), requires_grad=False) if bias else None

    def state_shape(self, B: int):
        return (B, max(1, self.taps - 1), self.channels)

    def load(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        if tuple(weight.shape) != (self.channels, self.taps):
            raise ValueError(f"convolution weight {tuple(weight.shape)}, expected {(self.channels, self.taps)}")
        self.weight.copy_(weight.float())
        if self.bias is not None:
            self.bias.copy_(bias.float())

    def forward(self, x: torch.Tensor, col0: int, state: torch.Tensor, pos_ids: torch.Tensor, B: int, T: int,
                out_dtype: torch.dtype, residual: bool = False, silu: bool = False) -> torch.Tensor:
        """``x [B*T, stride]``: the channels are its columns ``col0 .. col0 + channels``.  Returns ``[B*T, channels]``."""
        y = torch.empty((B * T, self.channels), dtype=out_dtype, device=x.device)
        N.call("ll_short_conv", N.ptr(x), N.dtype_code(x.dtype), x.stride(0), col0, N.ptr(self.weight), N.ptr(self.bias),
               N.ptr(state), N.ptr(pos_ids), N.ptr(y), N.dtype_code(out_dtype), self.channels, B, T, self.channels, self.taps,
               (1 if residual else 0) | (2 if silu else 0), N.stream())
        return y
