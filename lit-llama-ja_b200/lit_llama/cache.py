"""Cache memory of the models: tensors with stable addresses, addressed as rings.

Every model of this package writes its per-token state in place at slot ``position % length`` of a
tensor that outlives ``reset_cache()``: captured CUDA graphs hold the addresses, and a request that
ends gives its slots back simply by the next request writing over them from position 0.  ``TensorPool``
is that storage (LLaMA's key/value tensors, the latent rows of latent attention); ``ring_length`` and
``max_portion`` say how long a ring must be and how many tokens one step may append when every reader
looks back over a bounded window.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


class TensorPool:
    """Sets of zero-initialised tensors keyed by (shapes, dtype, device); the SAME tensors are handed out again after a
    release, zeroed on request.  At most ``max_sets`` keys stay alive; ``on_evict`` is told when one is dropped."""

    def __init__(self, max_sets: int = 2, on_evict: Optional[Callable[[], None]] = None):
        self.max_sets = max_sets
        self.on_evict = on_evict
        self._sets: Dict[tuple, List] = {}

    def get(self, shapes: Sequence[Tuple[int, ...]], dtype: torch.dtype, device, zero: bool = True) -> List[torch.Tensor]:
        key = (tuple(tuple(s) for s in shapes), dtype, str(device))
        ts = self._sets.get(key)
        if ts is None:
            if len(self._sets) >= self.max_sets:
                self._sets.pop(next(iter(self._sets)))
                if self.on_evict is not None:
                    self.on_evict()
            ts = self._sets[key] = [torch.zeros(s, device=device, dtype=dtype) for s in shapes]
        elif zero:
            for t in ts:
                t.zero_()
        return list(ts)

    def __len__(self) -> int:
        return len(self._sets)

    def clear(self) -> None:
        self._sets.clear()


def ring_length(max_seq_length: int, window: Optional[int], portion: int) -> int:
    """Slots a ring needs so that a step of up to ``portion`` tokens never overwrites a slot some query of the same step
    still reads: the ``window - 1`` positions before the step's first token plus the step itself.  Never more than
    ``max_seq_length`` (then no slot is ever reused).  ``window`` None: unbounded look-back."""
    if window is None:
        return max_seq_length
    return min(max_seq_length, window - 1 + max(1, portion))


def max_portion(length: int, max_seq_length: int, window: Optional[int]) -> int:
    """Tokens one step may append to a ring of ``length`` slots (see ``ring_length``)."""
    if window is None or length >= max_seq_length:
        return max(1, length)
    return max(1, length - (window - 1))
