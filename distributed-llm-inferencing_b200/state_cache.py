"""Per-sequence state SLOTS: fixed-size fp32 state that a layer carries from token to token (the matrix memory
of a recurrent layer, the last inputs of a short causal convolution), beside the paged key/value cache, which
holds what grows with the sequence (engine.PagedKVCache; a slot's index is also its row of the page table).

A slot is taken when a sequence is admitted and given back when it ends.  Nothing is cleared on either: every
kernel that reads a slot treats an entry whose first position is 0 as starting from zero, so a slot that is
used again cannot leak its previous sequence.
"""
from __future__ import annotations

from typing import Dict, List

import torch


class StateSlots:
    def __init__(self, n_slots: int, device):
        self.n_slots = int(n_slots)
        self.device = device
        self.free: List[int] = list(range(self.n_slots - 1, -1, -1))
        self.live: set = set()
        self.tensors: Dict[object, torch.Tensor] = {}

    def add(self, key, *shape) -> torch.Tensor:
        """Register float32 state of `shape` per slot under `key`; returns the [n_slots, *shape] tensor."""
        t = torch.zeros(self.n_slots, *shape, dtype=torch.float32, device=self.device)
        self.tensors[key] = t
        return t

    def __getitem__(self, key) -> torch.Tensor:
        return self.tensors[key]

    def alloc(self) -> int:
        if not self.free:
            raise RuntimeError("no free state slot")
        s = self.free.pop()
        self.live.add(s)
        return s

    def release(self, slot: int) -> None:
        if slot in self.live:
            self.live.remove(slot)
            self.free.append(slot)

    def bytes(self) -> int:
        return sum(t.numel() * 4 for t in self.tensors.values())
