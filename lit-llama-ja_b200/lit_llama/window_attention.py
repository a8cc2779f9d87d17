"""Softmax attention over a sliding window plus kept first tokens, without rotation: positions enter through the mask and
a logarithmic distance penalty.  Grouped key/value heads, a soft cap on the scores, the heads' softmax weights mixed by a
learned [H, H] matrix before they meet the values, and a sigmoid gate per head on the head's output:

    s_h(i, j) = cap * tanh(scale * q_h(i).k_g(j) / cap) - r1_h * ln(1 + r2_h (i - j))
    visible:    j <= i and (i - j < window  or  j < keep_first)
    o_h(i)    = sigmoid(g_h(i)) * sum_j ( sum_h' talk[h, h'] softmax_j(s_h')(i, j) ) v_g(h)(j)

Cache: key rows and value rows in one tensor each, ``[B, keep_first + R, G * dim]`` / ``[.., G * vdim]``: the kept tokens own
the first slots for good, everything later lives in a ring of ``R`` slots (csrc/window_attn.cu).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import _native as N
from .cache import max_portion, ring_length

UNBOUNDED = 1 << 30


@dataclass
class WindowAttentionSpec:
    width: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                 # 0: scores are not capped
    window: Optional[int]          # None: everything before the query
    keep_first: int = 0

    def __post_init__(self):
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads over {self.kv_heads} key/value heads")

    def ring(self, max_seq_length: int, portion: int) -> int:
        """Ring slots (beside the kept ones) for sequences of up to ``max_seq_length`` fed ``portion`` tokens at a time."""
        return max(1, ring_length(max(1, max_seq_length - self.keep_first), self.window, portion))

    def portion(self, ring: int, max_seq_length: int) -> int:
        return max_portion(ring, max(1, max_seq_length - self.keep_first), self.window)


class WindowAttention(nn.Module):
    def __init__(self, spec: WindowAttentionSpec, dtype: torch.dtype, device) -> None:
        super().__init__()
        s = self.spec = spec
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        hd, gd, gv = s.heads * s.dim, s.kv_heads * s.dim, s.kv_heads * s.vdim
        self.cols = dict(q=0, k=hd, v=hd + gd, g=hd + gd + gv)
        self.n_in = hd + gd + gv + s.heads
        self.r1 = nn.Parameter(torch.zeros(s.heads, **f32), requires_grad=False)
        self.r2 = nn.Parameter(torch.zeros(s.heads, **f32), requires_grad=False)
        self.talk = nn.Parameter(torch.eye(s.heads, **f32), requires_grad=False)
        self.w_o = nn.Parameter(torch.zeros((s.width, s.heads * s.vdim), **kw), requires_grad=False)

    def cache_shapes(self, B: int, ring: int) -> List[Tuple[int, ...]]:
        s = self.spec
        return [(B, s.keep_first + ring, s.kv_heads * s.dim), (B, s.keep_first + ring, s.kv_heads * s.vdim)]

    def in_weight(self, get) -> torch.Tensor:
        """The rows this mixer adds to a stacked input projection: [q; k; v; g]."""
        return torch.cat([get("q"), get("k"), get("v"), get("g")], dim=0)

    def load(self, get) -> None:
        self.r1.copy_(get("r1").float())
        self.r2.copy_(get("r2").float())
        self.talk.copy_(get("talk").float())
        self.w_o.copy_(get("o"))

    def forward(self, proj: torch.Tensor, col0: int, B: int, T: int, pos_ids: torch.Tensor, caches, splits: int = 1) -> torch.Tensor:
        return F.linear(self.attend(proj, col0, B, T, pos_ids, caches, splits), self.w_o)

    def attend(self, proj: torch.Tensor, col0: int, B: int, T: int, pos_ids: torch.Tensor, caches, splits: int = 1) -> torch.Tensor:
        """``proj``: the stacked input projection's output, this mixer's columns starting at ``col0``; ``caches`` = (keys,
        values), appended to here.  Returns the gated heads ``[B*T, heads * vdim]`` (before the output projection)."""
        s = self.spec
        c = self.cols
        kc, vc = caches
        M = B * T
        dtc = N.dtype_code(proj.dtype)
        ring = kc.shape[1] - s.keep_first
        st = N.stream()
        N.call("ll_sink_ring_append", N.ptr_at(proj, col0 + c["k"]), proj.stride(0), N.ptr_at(proj, col0 + c["v"]), proj.stride(0), dtc,
               N.ptr(pos_ids), N.ptr(kc), N.ptr(vc), B, T, s.kv_heads * s.dim, s.kv_heads * s.vdim, s.keep_first, ring, st)
        scratch = torch.empty(N.call_ret("ll_window_attn_scratch_bytes", M, s.heads, s.vdim, splits) // 4, dtype=torch.float32,
                              device=proj.device)
        y = torch.empty((M, s.heads * s.vdim), dtype=proj.dtype, device=proj.device)
        N.call("ll_window_attn", N.ptr_at(proj, col0 + c["q"]), proj.stride(0), N.ptr_at(proj, col0 + c["g"]), proj.stride(0), N.ptr(kc),
               N.ptr(vc), dtc, N.ptr(pos_ids), N.ptr(self.r1), N.ptr(self.r2), N.ptr(self.talk), float(s.scale), float(s.softcap), B, T,
               s.heads, s.kv_heads, s.dim, s.vdim, s.window if s.window is not None else UNBOUNDED, s.keep_first, ring, splits,
               N.ptr(scratch), N.ptr(y), st)
        return y
