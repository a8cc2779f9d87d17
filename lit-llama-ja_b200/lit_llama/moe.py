"""Mixture-of-experts feed-forward with gated-linear-unit experts and an optional always-on shared expert.

    z = W_r h + b  (fp32)      the ``top`` largest logits choose the experts
    weights: softmax over the chosen logits (``score`` "chosen"), or the chosen entries of the softmax over ALL experts
             divided by their sum + 1e-20 (``score`` "all")
    groups:  the experts form ``groups`` equal groups of neighbours; only experts of the ``keep_groups`` groups with the
             largest best expert can be chosen
    expert(h) = W_down( g * sigmoid(alpha * g) * (u + up_shift) ),  g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit)
                (limit inf, alpha 1, up_shift 0: the plain silu-gated unit)
    y = sum_k w_k expert_k(h)  +  sigmoid(w_sg . h) * shared(h)

The experts' weights are stacked ([X, 2 ff, width] for [gate; up], [X, width, ff] for down) and run as two grouped GEMMs
over the (token, choice) pairs sorted by expert; counts, offsets and the permutation never leave the device, so a step
is one fixed launch sequence.  Steps with many rows per expert (prefill in bfloat16) gather the rows into sorted order
and run both GEMMs on the tcgen05 tensor cores (TMA-tiled operands, accumulators in TMEM, the gated unit as the first
GEMM's epilogue); small steps use the mma.sync / FMA kernels that take rows in place.  The shared expert is dense
(library GEMMs) with its gate logit as one more output row.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import _native as N

# the tcgen05 path: at least this many (token, choice) rows in the step, and on average per expert
TC_MIN_ROWS = int(os.environ.get("LLB200_MOE_TC_MIN_ROWS", "1024"))
TC_MIN_ROWS_PER_EXPERT = int(os.environ.get("LLB200_MOE_TC_MIN_ROWS_PER_EXPERT", "48"))


@dataclass
class MoESpec:
    width: int
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: Optional[int] = None      # None: no shared expert
    shared_limit: Optional[float] = None
    shared_gate: bool = True             # the shared expert is scaled by sigmoid(w_sg . h)
    router_bias: bool = True
    alpha: float = 1.702                 # slope inside the sigmoid of the gated unit
    up_shift: float = 1.0                # the up branch enters as (u + up_shift): 1 or 0
    score: str = "chosen"                # "chosen": softmax over the chosen logits; "all": over all experts, renormalised
    groups: int = 1                      # equal groups of neighbouring experts
    keep_groups: int = 1                 # groups whose experts can be chosen (groups == 1: all)


def glu_clamp(gu: torch.Tensor, ff: int, limit: float, alpha: float) -> torch.Tensor:
    """``gu [rows, >= 2 ff]`` (columns [gate | up | ...]) -> ``[rows, ff]``: the clamped gated unit of this module."""
    out = torch.empty((gu.shape[0], ff), dtype=gu.dtype, device=gu.device)
    N.call("ll_glu_clamp", N.ptr(gu), gu.stride(0), ff, float(limit), float(alpha), N.ptr(out), N.dtype_code(gu.dtype),
           gu.shape[0], N.stream())
    return out


class MoE(nn.Module):
    def __init__(self, spec: MoESpec, dtype: torch.dtype, device) -> None:
        super().__init__()
        s = self.spec = spec
        if not 0 < s.top <= s.experts:
            raise ValueError(f"top {s.top} of {s.experts} experts")
        if s.up_shift not in (0.0, 1.0) or s.score not in ("chosen", "all"):
            raise ValueError(f"up_shift {s.up_shift} (0 or 1), score {s.score!r} ('chosen' or 'all')")
        if s.groups < 1 or s.experts % s.groups or not 1 <= s.keep_groups <= s.groups \
                or s.top > s.keep_groups * (s.experts // s.groups):
            raise ValueError(f"{s.experts} experts in {s.groups} groups, {s.keep_groups} kept, cannot give {s.top} choices")
        self.glu_mode = 1 if s.up_shift == 1.0 else 2
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.w_router = nn.Parameter(torch.empty((s.experts, s.width), **f32), requires_grad=False)
        self.b_router = nn.Parameter(torch.zeros(s.experts, **f32), requires_grad=False) if s.router_bias else None
        self.w_gu = nn.Parameter(torch.empty((s.experts, 2 * s.ff, s.width), **kw), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty((s.experts, s.width, s.ff), **kw), requires_grad=False)
        if s.shared_ff:
            rows = (2 * s.shared_ff + (1 if s.shared_gate else 0) + 7) // 8 * 8     # zero rows up to a multiple of 8
            self.w_shared_in = nn.Parameter(torch.empty((rows, s.width), **kw), requires_grad=False)   # [gate; up; sg]
            self.w_shared_down = nn.Parameter(torch.empty((s.width, s.shared_ff), **kw), requires_grad=False)

    def load(self, get) -> None:
        """``get(suffix)`` returns the tensor '<layer>.mlp.<suffix>'."""
        s = self.spec
        self.w_router.copy_(get("router").float())
        if self.b_router is not None:
            self.b_router.copy_(get("router.b").float())
        for e in range(s.experts):
            self.w_gu[e, : s.ff].copy_(get(f"e{e}.gate"))
            self.w_gu[e, s.ff:].copy_(get(f"e{e}.up"))
            self.w_down[e].copy_(get(f"e{e}.down"))
        if s.shared_ff:
            f = s.shared_ff
            self.w_shared_in.zero_()
            self.w_shared_in[:f].copy_(get("shared.gate"))
            self.w_shared_in[f:2 * f].copy_(get("shared.up"))
            if s.shared_gate:
                self.w_shared_in[2 * f:2 * f + 1].copy_(get("shared.sg").reshape(1, s.width))
            self.w_shared_down.copy_(get("shared.down"))

    def route(self, x_act: torch.Tensor):
        """(expert_idx [M, top] int32, expert_w [M, top] fp32, offsets [X + 1], perm [M * top])."""
        s = self.spec
        M, dev = x_act.shape[0], x_act.device
        i32 = dict(dtype=torch.int32, device=dev)
        idx = torch.empty((M, s.top), **i32)
        w = torch.empty((M, s.top), dtype=torch.float32, device=dev)
        counts, rank = torch.empty(s.experts, **i32), torch.empty(M * s.top, **i32)
        offsets, perm = torch.empty(s.experts + 1, **i32), torch.empty(M * s.top, **i32)
        N.call("ll_moe_route_scored", N.ptr(x_act), N.dtype_code(x_act.dtype), N.ptr(self.w_router), N.ptr(self.b_router), M, s.width,
               s.experts, s.top, 1 if s.score == "all" else 0, s.groups, s.keep_groups if s.groups > 1 else 1, N.ptr(idx), N.ptr(w),
               N.ptr(counts), N.ptr(rank), N.ptr(offsets), N.ptr(perm), N.stream())
        return idx, w, offsets, perm

    def takes_tensor_cores(self, n_rows: int, x_act: torch.Tensor) -> bool:
        """Whether a step of ``n_rows`` (token, choice) rows runs its expert GEMMs on the tcgen05 kernels: bfloat16, rows
        that TMA can tile (16-byte multiples), and enough rows per expert to fill 128-row tiles."""
        s = self.spec
        return (x_act.dtype == torch.bfloat16 and s.width % 8 == 0 and s.ff % 8 == 0 and x_act.stride(0) % 8 == 0
                and n_rows >= TC_MIN_ROWS and n_rows >= TC_MIN_ROWS_PER_EXPERT * s.experts and N.has("ll_moe_grouped_gemm_tc"))

    def forward(self, x_act: torch.Tensor) -> torch.Tensor:
        s = self.spec
        M, dev, dtype = x_act.shape[0], x_act.device, x_act.dtype
        dt, st = N.dtype_code(dtype), N.stream()
        _, w, offsets, perm = self.route(x_act)
        n = M * s.top
        h = torch.empty((n, s.ff), dtype=dtype, device=dev)
        y = torch.empty((n, s.width), dtype=dtype, device=dev)
        if self.takes_tensor_cores(n, x_act):
            xs = torch.empty((n, s.width), dtype=dtype, device=dev)
            N.call("ll_moe_gather_rows", N.ptr(x_act), x_act.stride(0), N.ptr(perm), s.top, n, s.width, N.ptr(xs), st)
            N.call("ll_moe_grouped_gemm_tc", N.ptr(xs), N.ptr(self.w_gu), N.ptr(offsets), N.ptr(perm), self.glu_mode, n, s.experts, s.ff,
                   s.width, float(s.limit), float(s.alpha), N.ptr(h), s.ff, st)
            N.call("ll_moe_grouped_gemm_tc", N.ptr(h), N.ptr(self.w_down), N.ptr(offsets), N.ptr(perm), 0, n, s.experts, s.width, s.ff,
                   0.0, 0.0, N.ptr(y), s.width, st)
        else:
            N.call("ll_moe_grouped_gemm", N.ptr(x_act), x_act.stride(0), N.ptr(self.w_gu), N.ptr(offsets), N.ptr(perm), self.glu_mode,
                   dt, n, s.top, s.experts, s.ff, s.width, float(s.limit), float(s.alpha), N.ptr(h), s.ff, st)
            N.call("ll_moe_grouped_gemm", N.ptr(h), s.ff, N.ptr(self.w_down), N.ptr(offsets), N.ptr(perm), 0, dt, n, s.top, s.experts,
                   s.width, s.ff, 0.0, 0.0, N.ptr(y), s.width, st)
        ys = gate = None
        gate_ld = 0
        if s.shared_ff:
            gu = F.linear(x_act, self.w_shared_in)
            hs = glu_clamp(gu, s.shared_ff, s.shared_limit if s.shared_limit is not None else s.limit, s.alpha)
            ys = F.linear(hs, self.w_shared_down)
            if s.shared_gate:
                gate, gate_ld = gu[:, 2 * s.shared_ff:], gu.stride(0)
        out = torch.empty((M, s.width), dtype=dtype, device=dev)
        N.call("ll_moe_combine", N.ptr(y), N.ptr(w), s.top, N.ptr(ys), s.width, N.ptr(gate), gate_ld, N.ptr(out), dt, M, s.width, st)
        return out
