"""Per-sequence state of fixed size, beside the paged cache: what a recurrent or convolutional token mixer carries from one step of a
sequence to the next (a matrix memory, the last few projected rows of a short convolution, ...).

The pool owns one slot per trackable sequence.  A model describes what a slot holds as named buffers (`StateBufferSpec`: a shape per slot
and a dtype); the pool allocates `[slots, *shape]` per buffer once.  A sequence gets a slot when it is created and gives it back when it is
flushed.  Slots are NOT cleared on reuse: the kernels that read a state take the sequence's first position as the sign that nothing has been
written yet (a sequence at position 0 starts from zeros), which keeps admission free of device work and of anything a captured decode
step could not replay."""
from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from ....accelerator import get_accelerator


@dataclass
class StateBufferSpec:
    name: str
    shape: Tuple[int, ...]  # per slot
    dtype: torch.dtype


class StateSlotPool:

    def __init__(self, n_slots: int, specs: List[StateBufferSpec], device=None):
        if n_slots < 1:
            raise ValueError(f"a state pool needs at least one slot, got {n_slots}")
        names = [s.name for s in specs]
        if len(set(names)) != len(names):
            raise ValueError("state buffer names must be unique")
        self._n = n_slots
        device = device if device is not None else get_accelerator().current_device_name()
        self._buffers: Dict[str, torch.Tensor] = {s.name: torch.zeros((n_slots, ) + tuple(int(x) for x in s.shape), dtype=s.dtype, device=device)
                                                  for s in specs}
        self._free = list(range(n_slots - 1, -1, -1))  # pop() hands out the lowest free slot
        self._held = set()

    @property
    def n_slots(self) -> int:
        return self._n

    @property
    def free_slots(self) -> int:
        return len(self._free)

    @property
    def bytes_per_slot(self) -> int:
        return sum(b[0].numel() * b.element_size() for b in self._buffers.values())

    def allocate(self) -> int:
        if not self._free:
            raise RuntimeError(f"all {self._n} state slots are in use")
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self._held:
            raise ValueError(f"state slot {slot} is not in use")
        self._held.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    def buffer(self, name: str) -> torch.Tensor:
        return self._buffers[name]

    def names(self):
        return list(self._buffers)
