"""Paged storage for latent (low-rank) key/value caches.

A latent-attention layer caches one row per token: the normed latent ``c`` (``rank`` entries) followed by the rotated
key part shared by all heads (``rot`` entries).  ``LatentPagedPool`` extends the page allocator of
``TinyKvPagedPool`` (LIFO free list, stable page ids, geometric growth) to ONE allocator with one slab per caching
layer, ``[capacity, page_size, rank_k + rot_k]``: all layers of a request advance in lockstep, so a request owns one
page list (``LatentPagedCache``) and every layer - also a layer that reads another layer's cache - addresses its slab
with the same ids (``LatentCacheView``).  The bytes are written by the device-driven append kernel; the host only
keeps the integers.
"""

from __future__ import annotations

import torch

from .kv_cache import TinyKvCache
from .paged_kv_cache import _SLAB_VERSIONS, TinyKvPagedCache, TinyKvPagedPool


class LatentPagedPool(TinyKvPagedPool):
    def __init__(self, widths: list[int], page_size: int = 64, dtype=torch.bfloat16, device="cuda", max_pages: int | None = None):
        """``widths[k]`` = row width of slab ``k``.  ``max_pages`` fixes the capacity: an append that needs more pages
        than are free then fails instead of growing the slabs (a serving pool sized for its token budget)."""
        super().__init__(page_size=page_size)
        self.widths = [int(w) for w in widths]
        self.dtype, self.device = dtype, torch.device(device)
        self.max_pages = max_pages
        self.slabs: list[torch.Tensor] = []
        self._capacity = 0
        if max_pages is not None:
            self.reserve(max_pages)

    # ---- storage ---------------------------------------------------------------
    @property
    def capacity(self) -> int:
        return self._capacity

    @property
    def key_pages(self):
        raise AttributeError("a latent pool has one slab per layer: use .slabs[k]")

    value_pages = key_pages

    @property
    def storage_nbytes(self) -> int:
        return sum(s.numel() * s.element_size() for s in self.slabs)

    def reserve(self, num_pages: int, *_, **__) -> None:
        """Size every slab for ``num_pages`` pages (one counted growth; live pages are carried over)."""
        if self._capacity >= num_pages:
            return
        if self.max_pages is not None and num_pages > self.max_pages:
            raise RuntimeError(f"page pool exhausted: {num_pages} pages wanted, the pool is fixed at {self.max_pages}")
        new = [torch.zeros((num_pages, self.page_size, w), dtype=self.dtype, device=self.device) for w in self.widths]
        live = min(self.num_pages, self._capacity)
        if self.slabs and live:
            for old, fresh in zip(self.slabs, new):
                fresh[:live] = old[:live]
                self.copied_bytes_on_growth += old[:live].numel() * old.element_size()
            self.copied_pages_on_growth += live
        self.slabs = new
        self._capacity = num_pages
        self.storage_growths += 1
        self.slab_version = next(_SLAB_VERSIONS)

    def ensure_room(self, fresh_pages: int) -> None:
        """Make sure ``fresh_pages`` allocations will find storage (grow geometrically unless the pool is fixed)."""
        short = fresh_pages - len(self.free_page_ids) - (self._capacity - self.num_pages)
        if short <= 0:
            return
        if self.max_pages is not None:
            raise RuntimeError(f"page pool exhausted: {short} more pages wanted, the pool is fixed at {self.max_pages}")
        self.reserve(max(4, self._capacity + short, self._capacity * 2))

    def reset(self) -> None:
        if self.used_page_ids:
            raise ValueError("Cannot reset a page pool with live requests")
        self.slabs, self._capacity = [], 0
        self.slab_version = next(_SLAB_VERSIONS)
        self.free_page_ids.clear()
        self.num_allocated_pages = 0
        self.reused_page_allocations = self.storage_growths = self.copied_pages_on_growth = self.copied_bytes_on_growth = 0
        if self.max_pages is not None:
            self.reserve(self.max_pages)


class LatentPagedCache(TinyKvPagedCache):
    """A request's page list (shared by all its layers).  Only the integer side of ``TinyKvPagedCache`` applies:
    ``append_slots`` / ``rewind`` / ``release`` / ``block_table_host``; rows are written by the append kernel."""

    def __init__(self, pool: LatentPagedPool):
        super().__init__(pool)

    def _device(self):
        return self.pool.device

    def append_slots(self, count: int) -> None:
        if count <= 0:
            return
        tail_room = self.page_size - self.page_lens[-1] if self.page_ids else 0
        self.pool.ensure_room(max(0, -(-(count - tail_room) // self.page_size)))
        super().append_slots(count)

    def update_and_fetch(self, key, value, mask_length=None, mask=None):
        raise NotImplementedError("a latent cache is filled by the model's ragged step, not by dense K/V chunks")

    update_and_fetch_paged = update_and_fetch


class LatentCacheView(TinyKvCache):
    """The per-layer face of a request's ``LatentPagedCache``: which slab the layer reads (its own or, for a layer that
    attends another layer's latent, that layer's).  It owns nothing: ``release`` is the owner's business."""

    def __init__(self, owner: LatentPagedCache, slab_index: int):
        self.owner, self.slab_index = owner, slab_index
        self.pool, self.page_size = owner.pool, owner.page_size

    offset = property(lambda self: self.owner.offset)
    page_ids = property(lambda self: self.owner.page_ids)
    page_lens = property(lambda self: self.owner.page_lens)
    num_pages = property(lambda self: self.owner.num_pages)

    def logical_offset(self) -> int:
        return self.owner.logical_offset()

    def update_and_fetch(self, key, value, mask_length=None, mask=None):
        raise NotImplementedError("a latent cache is filled by the model's ragged step, not by dense K/V chunks")

    def release(self):
        return None
