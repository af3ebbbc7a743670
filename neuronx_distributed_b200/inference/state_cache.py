"""Per-sequence state for models whose layers keep more than keys and values: ring caches of a sliding window, convolution
histories, recurrent states.  Every layer declares ``{name: (shape per sequence, dtype)}``; the manager owns one tensor
``[slots, *shape]`` per entry, hands out slots to requests and takes them back (a freed slot is reused as is: the first call of a
new sequence runs with ``fresh=True``, which makes every kernel ignore what the slot held).  Slots grow on demand.

The plain K/V manager next to this file (``kv_cache.py``) serves the Llama-family models: fixed batch rows, full-length caches."""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Sequence, Tuple

import torch

Spec = Dict[str, Tuple[Tuple[int, ...], torch.dtype]]


@dataclasses.dataclass
class StepContext:
    """What every stateful layer needs to know about the rows of a step (all device tensors int32 ``[B]``)."""
    lens: torch.Tensor          # real tokens per row in this step
    slots: torch.Tensor         # state slot of each row
    pos0: torch.Tensor          # position of each row's first token
    fresh: bool                 # the rows start their sequences in this step
    scratch: Dict = dataclasses.field(default_factory=dict)   # what one layer leaves for a later layer of the same step


class SequenceStateManager:
    def __init__(self, layer_specs: Sequence[Spec], num_slots: int = 8, device=None):
        self.specs, self.device = list(layer_specs), device
        self.num_slots = 0
        self.layers: List[Dict[str, torch.Tensor]] = [{} for _ in self.specs]
        self._free: List[int] = []
        self.length: Dict[int, int] = {}                      # slot → tokens the sequence holds so far (host side)
        self._grow(max(1, num_slots))

    def _grow(self, n: int) -> None:
        for spec, bufs in zip(self.specs, self.layers):
            for name, (shape, dtype) in spec.items():
                new = torch.zeros((n,) + tuple(shape), dtype=dtype, device=self.device)
                if name in bufs:
                    new[: self.num_slots].copy_(bufs[name])
                bufs[name] = new
        self._free.extend(range(self.num_slots, n))
        self.num_slots = n

    def alloc(self) -> int:
        if not self._free:
            self._grow(self.num_slots * 2)
        slot = min(self._free)
        self._free.remove(slot)
        self.length[slot] = 0
        return slot

    def free(self, slot: int) -> None:
        if slot not in self.length:
            raise KeyError(f"slot {slot} is not in use")
        del self.length[slot]
        self._free.append(slot)

    def advance(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        for s, c in zip(slots, counts):
            self.length[s] += int(c)

    @property
    def in_use(self) -> int:
        return len(self.length)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for bufs in self.layers for t in bufs.values())

    def layer(self, i: int) -> Dict[str, torch.Tensor]:
        return self.layers[i]
