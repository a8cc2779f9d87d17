"""Lepalorn: a decoder-only model of latent-attention layers with sliding windows (some reading another layer's cache
rows), mixture-of-experts feed-forwards, a norm on every sublayer's OUTPUT with a one-number gain, and a learned weighted
average over the outputs of all earlier layers (depth-weighted average) after every layer.

    x = embed[token] * embedding.scale                                     X_0 = x
    layer i:   x <- x + g1 * rmsnorm(mixer(x));  x <- x + g2 * rmsnorm(ff(x));   X_(i+1) = x
               x <- sum_{j <= i+1} dwa_i[j] X_j                              (what the next layer, or the head, reads)
    logits = head (g_f * rmsnorm(x))

The residual stream, the X_j, the norms, rotary angles, attention scores and router logits are fp32 whatever the dtype of
the GEMMs.  ``forward`` is the package's common step function (stepping.PortionedDecoder: LLaMA's signature, prompts in passes,
single-token steps as one CUDA graph per (batch, ring length)); per-token state lives in ring tensors from the package's
``TensorPool`` (cache.py) and is written in place.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from . import _native as N
from .cache import TensorPool, max_portion, ring_length
from .latent_attention import LatentAttention, LatentAttentionSpec, build_rope_table
from .moe import MoE, MoESpec
from .stepping import PortionedDecoder, head_logits

ARCHITECTURE = "Lepalorn"


@dataclass
class LepalornLayer:
    mixer: LatentAttentionSpec
    mlp: Optional[MoESpec]


@dataclass
class LepalornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: List[LepalornLayer] = field(default_factory=list)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    @property
    def block_size(self) -> int:
        """No learned or tabulated position limit: rotary angles are computed for whatever length the cache is given."""
        return 1 << 30

    @classmethod
    def from_dict(cls, cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "LepalornConfig":
        """From the dictionary of a ``config.json``; sizes it leaves out are taken from the tensors' shapes."""
        shapes = shapes or {}

        def pick(value, name, axis, div=1):
            if value is not None:
                return int(value)
            if name in shapes:
                return shapes[name][axis] // div
            raise KeyError(f"config.json gives no size that tensor {name!r} would determine, and the tensor is absent")

        width = pick(cfg.get("width"), "embed", 1)
        vocab = pick(cfg.get("vocab"), "embed", 0)
        eps = float(cfg["norm"]["eps"])
        layers = []
        for i, lc in enumerate(cfg["layers"]):
            if lc.get("type") != "latent_attention":
                raise ValueError(f"layer {i}: unknown mixer type {lc.get('type')!r}")
            m, p = lc["mixer"], f"l{i}.mix."
            heads = pick(m.get("heads"), p + "g", 0)
            kv_rank = pick(m.get("kv_rank"), p + "uk", 1)
            nope = pick(m.get("dim"), p + "uk", 0, heads)
            rot_dim = int(m["rot_dim"]) if m.get("rot_dim") is not None else shapes[p + "q"][0] // heads - nope
            rot = m.get("rot") or {}
            mask = m.get("mask") or {}
            mixer = LatentAttentionSpec(
                width=width, heads=heads, nope_dim=nope, rot_dim=rot_dim, v_dim=pick(m.get("vdim"), p + "uv", 0, heads),
                kv_rank=kv_rank, window=int(mask["size"]) if mask.get("size") is not None else None, scale=float(m["scale"]),
                rot_base=float(rot.get("base", 10000.0)), rot_dims=int(rot["dims"]) if rot.get("dims") is not None else None,
                eps=eps, kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else None)
            mlp = None
            if lc.get("mlp") is not None:
                f, q = lc["mlp"], f"l{i}.mlp."
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
                sh = f.get("shared")
                mlp = MoESpec(width=width, experts=pick(f["router"].get("experts"), q + "router", 0), top=int(f["router"]["top"]),
                              ff=pick(f["expert"].get("ff"), q + "e0.gate", 0), limit=float(f["expert"]["limit"]),
                              shared_ff=pick(sh.get("ff"), q + "shared.gate", 0) if sh else None,
                              shared_limit=float(sh["limit"]) if sh else None,
                              shared_gate=bool(sh) and (not shapes or (q + "shared.sg") in shapes),
                              router_bias=not shapes or (q + "router.b") in shapes)
            layers.append(LepalornLayer(mixer, mlp))
        for i, l in enumerate(layers):
            j = l.mixer.kv_from
            if j is not None:
                src = layers[j].mixer if 0 <= j < i else None
                if src is None or src.kv_from is not None:
                    raise ValueError(f"layer {i}: kv_from {j} must name an earlier layer with a cache of its own")
                if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != (l.mixer.kv_rank, l.mixer.rot_dim, l.mixer.rot_dims,
                                                                              l.mixer.rot_base):
                    raise ValueError(f"layer {i}: its latent row differs from that of layer {j}")
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=float(cfg["embedding"]["scale"]), layers=layers)


def gain_norm_add_mix(x, y, gain, eps, out=None, stack=None, mix_w=None, n_mix=0, nxt=None, nxt_act=None):
    """``r = x + gain * y / rms(y)`` (``x`` None: the norm alone) -> ``out``; then the weighted sum over ``stack[:n_mix-1]``
    and r -> ``nxt`` (fp32) / ``nxt_act`` (one launch; see ``ll_gain_norm_add_mix``)."""
    rows, dim = y.shape
    act = nxt_act.dtype if nxt_act is not None else y.dtype
    N.call("ll_gain_norm_add_mix", N.ptr(x), N.ptr(y), N.dtype_code(y.dtype), N.ptr(gain), float(eps), N.ptr(out), N.ptr(stack),
           stack.stride(0) if stack is not None else 0, N.ptr(mix_w), n_mix, N.ptr(nxt), N.ptr(nxt_act), N.dtype_code(act), rows,
           dim, N.stream())


class LepalornBlock(nn.Module):
    def __init__(self, index: int, layer: LepalornLayer, dtype, device) -> None:
        super().__init__()
        f32 = dict(dtype=torch.float32, device=device)
        self.index = index
        self.mix = LatentAttention(layer.mixer, dtype, device)
        self.mlp = MoE(layer.mlp, dtype, device) if layer.mlp is not None else None
        self.norm1 = nn.Parameter(torch.ones(1, **f32), requires_grad=False)
        self.norm2 = nn.Parameter(torch.ones(1, **f32), requires_grad=False) if self.mlp is not None else None
        self.dwa = nn.Parameter(torch.zeros(index + 2, **f32), requires_grad=False)

    def load(self, get) -> None:
        p = f"l{self.index}."
        self.mix.load(lambda s: get(p + "mix." + s))
        self.norm1.copy_(get(p + "norm1").float().reshape(1))
        if self.mlp is not None:
            self.mlp.load(lambda s: get(p + "mlp." + s))
            self.norm2.copy_(get(p + "norm2").float().reshape(1))
        self.dwa.copy_(get(p + "dwa").float())


class Lepalorn(PortionedDecoder):
    architecture = ARCHITECTURE

    def __init__(self, config: LepalornConfig, dtype: torch.dtype = torch.bfloat16, device="cuda") -> None:
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Lepalorn runs in bfloat16 or float32")
        self.config = config
        self.dtype, self.device = dtype, torch.device(device)
        kw = dict(dtype=dtype, device=self.device)
        self.embed = nn.Parameter(torch.empty((config.vocab, config.width), **kw), requires_grad=False)
        self.blocks = nn.ModuleList(LepalornBlock(i, l, dtype, self.device) for i, l in enumerate(config.layers))
        self.final_norm = nn.Parameter(torch.ones(1, dtype=torch.float32, device=self.device), requires_grad=False)
        self.head = nn.Parameter(torch.zeros(((config.vocab + 7) // 8 * 8, config.width), **kw), requires_grad=False)   # zero rows to 8
        self._pool = TensorPool(max_sets=2, on_evict=self._drop_graphs)
        self._rope: Dict[Tuple[float, int], torch.Tensor] = {}
        self._rope_len = 0
        self.kv_caches: List[torch.Tensor] = []       # one ring per layer that owns a cache (index: _cache_of[layer])
        self._ring = 0
        self._cache_of: List[int] = []
        n = 0
        for l in config.layers:
            if l.mixer.kv_from is None:
                self._cache_of.append(n)
                n += 1
            else:
                self._cache_of.append(self._cache_of[l.mixer.kv_from])
        # the longest look-back over each ring (its own layer's window and those of the layers reading it)
        self._windows: List[Optional[int]] = []
        for c in range(n):
            ws = [l.mixer.window for i, l in enumerate(config.layers) if self._cache_of[i] == c]
            self._windows.append(None if any(w is None for w in ws) else max(ws))

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_tensors(self, get) -> None:
        """``get(name)`` returns the checkpoint tensor of that name (any float dtype, CPU or GPU)."""
        self.embed.copy_(get("embed"))
        self.head[: self.config.vocab].copy_(get("head"))
        self.final_norm.copy_(get("final.norm").float().reshape(1))
        for b in self.blocks:
            b.load(get)

    @classmethod
    def from_dir(cls, path, dtype: torch.dtype = torch.bfloat16, device="cuda") -> "Lepalorn":
        """A folder with ``config.json`` and ``model.safetensors``."""
        from .safetensors_io import SafetensorsFile

        path = Path(path)
        with open(path / "config.json") as f:
            cfg = json.load(f)
        with SafetensorsFile(path / "model.safetensors") as st:
            model = cls(LepalornConfig.from_dict(cfg, st.shapes()), dtype=dtype, device=device)
            model.load_tensors(st.get)
        return model.eval()

    # ------------------------------------------------------------------ cache
    def reset_cache(self) -> None:
        """The sequences end: their rows are given back (the rings stay allocated and are written over from position 0)."""
        self.kv_caches = []

    def _ensure_cache(self, B: int, max_seq_length: int, pooled: bool = True) -> None:
        ring = max(ring_length(max_seq_length, w, min(self.prefill_portion, max_seq_length)) for w in self._windows)
        if self.kv_caches and self.kv_caches[0].shape[0] == B and self._ring == ring:
            return
        shapes = [(B, ring, l.mixer.row) for l in self.config.layers if l.mixer.kv_from is None]
        if pooled:
            self.kv_caches = self._pool.get(shapes, self.dtype, self.device, zero=False)
        else:                      # a forward that keeps nothing: scratch rings, the pool's sets stay as they are
            self.kv_caches = [torch.empty(s, dtype=self.dtype, device=self.device) for s in shapes]
        self._ring = ring

    def _ensure_rope(self, n_pos: int) -> None:
        if n_pos <= self._rope_len:
            return
        n = max(n_pos, 2 * self._rope_len, 1024)
        for l in self.config.layers:
            key = (l.mixer.rot_base, l.mixer.rot_dims)
            if key not in self._rope or self._rope[key].shape[0] < n:
                self._rope[key] = build_rope_table(n, l.mixer.rot_dims, l.mixer.rot_base, self.device)
        self._rope_len = n
        self._drop_graphs()

    # ------------------------------------------------------------------ hooks of the common step function (stepping.py)
    def _begin(self, B: int, max_seq_length: int, keep: bool) -> None:
        self._ensure_cache(B, max_seq_length, pooled=keep)
        self._ensure_rope(max_seq_length)

    def _piece(self, max_seq_length: int) -> int:
        return min(max_portion(self._ring, max_seq_length, w) for w in self._windows)

    def _graph_key(self, B: int) -> tuple:
        return (B, self._ring, self.kv_caches[0].data_ptr())

    def _save_memory(self):
        saved = (self.kv_caches, self._ring)
        self.kv_caches = []
        return saved

    def _restore_memory(self, saved) -> None:
        self.kv_caches, self._ring = saved

    def _forward_portion(self, idx: torch.Tensor, pos_ids: torch.Tensor, sel) -> torch.Tensor:
        cfg = self.config
        B, T = idx.shape
        M, E, L = B * T, cfg.width, cfg.n_layer
        dev = idx.device
        st = N.stream()
        act = N.dtype_code(self.dtype)
        stack = torch.empty((L + 1, M, E), dtype=torch.float32, device=dev)      # X_0 .. X_L
        x_act = torch.empty((M, E), dtype=self.dtype, device=dev)                # what the next GEMM reads
        x = stack[0]                                                             # the stream the layer adds to
        N.call("ll_embed_scaled", N.ptr(self.embed), act, N.ptr(idx.reshape(-1).contiguous()), float(cfg.embedding_scale),
               N.ptr(x), N.ptr(x_act), act, M, E, st)
        mixed = torch.empty((2, M, E), dtype=torch.float32, device=dev)
        # splits: share a long window among blocks when the step has few queries (decoding)
        sms = N.call_ret("ll_sm_count")
        for i, blk in enumerate(self.blocks):
            spec = blk.mix.spec
            span = spec.window if spec.window is not None else self._ring
            splits = max(1, min(16, (2 * sms) // max(1, M * ((spec.heads + 31) // 32)), (min(span, self._ring) + 63) // 64))
            rope = self._rope[(spec.rot_base, spec.rot_dims)]
            y = blk.mix(x_act, B, T, pos_ids, rope, self.kv_caches[self._cache_of[i]], splits)
            nxt = mixed[i & 1]
            if blk.mlp is not None:
                mid = nxt                                                        # scratch for the stream between the sublayers
                gain_norm_add_mix(x, y, blk.norm1, cfg.eps, out=mid, nxt_act=x_act)
                y2 = blk.mlp(x_act)
                gain_norm_add_mix(mid, y2, blk.norm2, cfg.eps, out=stack[i + 1], stack=stack, mix_w=blk.dwa, n_mix=i + 2,
                                  nxt=nxt, nxt_act=x_act)
            else:
                gain_norm_add_mix(x, y, blk.norm1, cfg.eps, out=stack[i + 1], stack=stack, mix_w=blk.dwa, n_mix=i + 2,
                                  nxt=nxt, nxt_act=x_act)
            x = nxt
            if self.layer_probe is not None:
                self.layer_probe(i, x)
        if sel is not None and len(sel) == 0:      # the step only fills the cache
            return torch.empty((B, 0, cfg.vocab), dtype=torch.float32, device=dev)
        if sel is not None:
            ridx = (torch.arange(B, device=dev)[:, None] * T + torch.tensor(sel, device=dev, dtype=torch.long)[None]).reshape(-1)
            x = x.index_select(0, ridx).contiguous()
        xn = torch.empty((x.shape[0], E), dtype=self.dtype, device=dev)
        gain_norm_add_mix(None, x, self.final_norm, cfg.eps, nxt_act=xn)
        return head_logits(xn, self.head, cfg.vocab).reshape(B, -1, cfg.vocab)
