"""Replaying a trace of steps through a model: each step brings the next tokens of some request and asks for the
logits at some of them.  The session keeps, per live request, how many tokens the model's cache holds for it, and drives
the model's own ``forward(idx, max_seq_length, input_pos)`` - the call ``generate()`` makes - so a trace exercises
exactly the serving path: prefill portions of any length, single-token steps (graph replays), rings that are reused.

The models of this package keep one set of rings per batch shape, so a session serves one request at a time (requests
follow one another; a new one starts when the previous has ended).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


class TraceSession:
    def __init__(self, model, max_tokens: int, device="cuda") -> None:
        self.model = model
        self.max_tokens = int(max_tokens)
        self.device = torch.device(device)
        self.live: Dict[str, int] = {}          # request id -> tokens in the cache

    def step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[torch.Tensor]:
        """``entries``: ``{"id", "tokens", "want"}``.  Returns the fp32 logits ``[wanted, vocab]`` at the wanted places
        (entries in order), or None when nothing is wanted."""
        rows: List[torch.Tensor] = []
        for e in entries:
            rid, toks, want = e["id"], list(e["tokens"]), list(e.get("want", ()))
            if rid not in self.live:
                if self.live:
                    raise RuntimeError(f"request {rid!r} starts while {sorted(self.live)} still hold the cache")
                self.model.reset_cache()
                self.live[rid] = 0
            at = self.live[rid]
            if not toks:
                continue
            if at + len(toks) > self.max_tokens:
                raise RuntimeError(f"request {rid!r} grows to {at + len(toks)} tokens; the session holds {self.max_tokens}")
            idx = torch.tensor([toks], dtype=torch.int64, device=self.device)
            pos = torch.arange(at, at + len(toks))
            out = self.model(idx, self.max_tokens, pos, out_rows=want)
            self.live[rid] = at + len(toks)
            if want:
                rows.append(out[0].float())
        for rid in end:
            if self.live.pop(rid, None) is not None and not self.live:
                self.model.reset_cache()
        return torch.cat(rows, dim=0) if rows else None
