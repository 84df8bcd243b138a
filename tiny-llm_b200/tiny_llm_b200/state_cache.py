"""Recurrent-state slots beside the paged key/value cache.

A recurrent mixer carries a fixed-size fp32 state per request instead of a row per token.  ``StateSlotPool`` holds
those states as rows of ONE tensor ``[slots, floats]`` (every recurrent layer of the model owns a column range of the
row, ``layer_view``), hands slots out LIFO like the page pool hands out pages, and grows geometrically unless it was
made for a fixed number of requests.  ``HybridPagedCache`` is a request's cache in a model that has both kinds of
layers: the page list of ``LatentPagedCache`` plus one state slot, taken at the request's first tokens and given back
with its pages.  A slot is not cleared when it changes hands: the kernels start a sequence at position 0 from zero.
"""

from __future__ import annotations

import torch

from .latent_kv_cache import LatentPagedCache, LatentPagedPool
from .paged_kv_cache import _SLAB_VERSIONS


class StateSlotPool:
    def __init__(self, floats_per_slot: int, device="cuda", max_slots: int | None = None):
        self.floats, self.device, self.max_slots = int(floats_per_slot), torch.device(device), max_slots
        self.storage = torch.zeros((0, max(self.floats, 1)), dtype=torch.float32, device=self.device)
        self.free_slots: list[int] = []
        self.used_slots: set[int] = set()
        self.num_allocated = 0
        self.reused_slot_allocations = self.storage_growths = 0
        self.version = 0
        if max_slots is not None:
            self._resize(max_slots)

    @property
    def capacity(self) -> int:
        return self.storage.shape[0]

    def _resize(self, slots: int) -> None:
        new = torch.zeros((slots, self.storage.shape[1]), dtype=torch.float32, device=self.device)
        if self.num_allocated:
            new[: self.num_allocated] = self.storage[: self.num_allocated]
        self.storage = new
        self.storage_growths += 1
        self.version = next(_SLAB_VERSIONS)

    def allocate(self) -> int:
        """Newest freed slot first, else the next never-used one."""
        if self.free_slots:
            slot = self.free_slots.pop()
            self.reused_slot_allocations += 1
        else:
            if self.num_allocated >= self.capacity:
                if self.max_slots is not None:
                    raise RuntimeError(f"state slots exhausted: the pool is fixed at {self.max_slots} requests")
                self._resize(max(4, 2 * self.capacity))
            slot = self.num_allocated
            self.num_allocated += 1
        self.used_slots.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self.used_slots:
            raise ValueError(f"state slot {slot} is already free")
        self.used_slots.remove(slot)
        self.free_slots.append(slot)

    def layer_view(self, offset: int, shape: tuple) -> torch.Tensor:
        """``[slots, *shape]`` view of the columns ``offset ..`` of every slot (slots stay ``floats`` apart)."""
        n = 1
        for d in shape:
            n *= int(d)
        return self.storage[:, offset : offset + n].unflatten(1, tuple(int(d) for d in shape))


class HybridPagedCache(LatentPagedCache):
    """Page list + state slot of one request.  ``ran_offset`` is how many of its tokens a model step has consumed: the
    state cannot be taken back, so only tokens that no step has run yet can be rewound (or everything, by release)."""

    def __init__(self, pool: LatentPagedPool, states: StateSlotPool | None):
        super().__init__(pool)
        self.states = states if states is not None and states.floats > 0 else None
        self.state_slot = -1
        self.ran_offset = 0

    def append_slots(self, count: int) -> None:
        if count <= 0:
            return
        took = False
        if self.states is not None and self.state_slot < 0:
            self.state_slot = self.states.allocate()
            took = True
        try:
            super().append_slots(count)
        except Exception:
            if took:
                self.states.free(self.state_slot)
                self.state_slot = -1
            raise

    def rewind(self, n: int):
        keep = self.offset - n
        if self.states is not None and 0 < keep < self.ran_offset:
            raise NotImplementedError("a recurrent state cannot be rewound past tokens that a step has consumed")
        super().rewind(n)

    def release(self):
        super().release()
        if self.state_slot >= 0:
            self.states.free(self.state_slot)
            self.state_slot = -1
        self.ran_offset = 0
