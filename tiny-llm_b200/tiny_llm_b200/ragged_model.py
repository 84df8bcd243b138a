"""The step machinery shared by models that run ragged batches over paged caches.

``RaggedDecoderModel`` gives a model class the framework's entry points on top of ONE method, ``_forward_plan(plan)``
(the layers over a ``RaggedPlan``): ``forward_ragged`` (one step over any mix of prompt portions and single tokens;
what the batcher's mixed mode and the trace runner call), the CUDA-graph replay of decode-only steps, and the
rectangular ``model(inputs, offset, cache, logits_to_keep)`` call that ``greedy_generate_ids`` and the slot-table
scheduler use.  A subclass sets ``page_pool`` (a pool with ``slab_version``), ``page_size``, ``tile_sizes``,
``vocab_size``, ``device``, ``precision`` and implements ``create_kv_cache`` and ``_forward_plan``.
"""

from __future__ import annotations

import os

import torch

from .kv_cache import BatchingKvCache
from .ragged import RaggedEntry, RaggedPlan


class RaggedDecoderModel:
    graph_env = "TL_DECODE_GRAPH"

    def _init_step(self) -> None:
        self.h2d_bytes = 0
        # Decode-only steps (every entry brings one token) replay a captured CUDA graph, one per (number of entries, block
        # table width); the step's integers are data in one device block.  None = on for CUDA, False = always eager.
        self.use_decode_graph: bool | None = None if os.environ.get(self.graph_env, "1") != "0" else False
        self._graphs: dict = {}
        self.graph_replays = self.graph_captures = 0

    def _storage_version(self):
        """Changes whenever device storage that a captured graph addresses has been reallocated."""
        return self.page_pool.slab_version

    def _forward_plan(self, plan: RaggedPlan) -> torch.Tensor:
        raise NotImplementedError

    # ---- the step --------------------------------------------------------------------
    def forward_ragged(self, entries: list[RaggedEntry]) -> torch.Tensor:
        """One step over ``entries`` -> fp32 logits ``[sum of wanted places, vocab]`` in entry order.  Appends the
        entries' tokens to their caches."""
        if self.use_decode_graph is not False and self.device.type == "cuda" and all(len(e.tokens) == 1 and (e.want is None or list(e.want) == [0]) for e in entries):
            return self._decode_step(entries)
        plan = RaggedPlan(entries, self.device, self.tile_sizes)
        self.h2d_bytes += plan.h2d_bytes
        return self._forward_plan(plan)

    def _decode_step(self, entries: list[RaggedEntry]) -> torch.Tensor:
        """A step of one token per entry.  The first step of a shape runs eagerly (it warms every library up), the second
        is captured - its integers uploaded into the graph's own device block - and from then on a step is one
        host-to-device copy and one replay.  Shapes: the number of entries and the block table's width (a power of two,
        at least 4 pages), so a request growing by a page does not change the graph; slabs that moved do."""
        S = len(entries)
        pages = max(-(-(getattr(e.cache[0], "owner", e.cache[0]).offset + 1) // self.page_size) for e in entries)
        width = 4
        while width < pages:
            width *= 2
        key = (S, width)
        state = self._graphs.get(key)
        if state is not None and state.get("slabs") not in (None, self._storage_version()):
            state = None  # captured against slabs that have been reallocated since
        if state is None:
            self._graphs[key] = {"slabs": None}
            plan = RaggedPlan(entries, self.device, self.tile_sizes)
            self.h2d_bytes += plan.h2d_bytes
            return self._forward_plan(plan)
        if state["slabs"] is None:
            total = RaggedPlan.block_ints(S, S, S, width, S * len(self.tile_sizes))
            state["block"] = torch.zeros(total, dtype=torch.int32, device=self.device)
            plan = RaggedPlan(entries, self.device, self.tile_sizes, max_pages=width, into=state["block"])
            state["slabs"] = self._storage_version()  # the append may have grown the pool: read it after the plan
            torch.cuda.current_stream(self.device).synchronize()
            graph = torch.cuda.CUDAGraph()
            # The library's GEMM workspace is cached per stream, and all captures share one side stream: a workspace that was
            # allocated inside an earlier capture lives in THAT graph's memory pool and dangles once that graph is gone.
            # Dropping the cached workspaces around the capture keeps each graph's workspace its own.
            drop_workspaces = getattr(torch._C, "_cuda_clearCublasWorkspaces", lambda: None)
            drop_workspaces()
            try:
                with torch.cuda.graph(graph):
                    state["logits"] = self._forward_plan(plan)
            finally:
                drop_workspaces()
            state["graph"], state["plan"] = graph, plan
            self.graph_captures += 1
        else:
            plan = RaggedPlan(entries, self.device, self.tile_sizes, max_pages=width, into=state["block"])
            if self._storage_version() != state["slabs"]:  # this very append moved the slabs: run it eagerly, re-capture next time
                self._graphs.pop(key)
                return self._forward_plan(plan)
            state["host"] = plan._host
        self.h2d_bytes += plan.h2d_bytes
        state["graph"].replay()
        self.graph_replays += 1
        return state["logits"].clone()

    def __call__(self, inputs: torch.Tensor, offset, cache: list, logits_to_keep: int | None = None) -> torch.Tensor:
        """The framework's rectangular call: ``inputs [B, L]`` token ids, ``cache`` the per-layer caches of one request
        (B == 1) or the scheduler's per-layer slot tables (idle slots give zero logits).  ``offset`` must equal what
        the caches hold; -> fp32 ``[B, L or logits_to_keep, vocab]``."""
        if inputs.dim() != 2:
            raise ValueError("inputs must be [B, L]")
        B, L = inputs.shape
        keep = L if logits_to_keep is None else int(logits_to_keep)
        if keep <= 0:
            raise ValueError("logits_to_keep must be positive")
        keep = min(keep, L)
        first = cache[0]
        if isinstance(first, BatchingKvCache):
            if first.max_active_requests != B:
                raise ValueError(f"Expected batch size {first.max_active_requests}, got {B}")
            slots = [None if first.kv_caches[b] is None else [table.kv_caches[b] for table in cache] for b in range(B)]
            if all(s is None for s in slots):
                raise ValueError("Cannot build paged metadata without active requests")
        elif B == 1:
            slots = [cache]
        else:
            raise ValueError("a batch needs the scheduler's slot tables as its cache")
        if isinstance(offset, torch.Tensor):
            offsets = [int(v) for v in offset.reshape(-1).tolist()]
        elif isinstance(offset, int):
            offsets = [offset]
        else:
            offsets = [int(v) for v in offset]
        offsets = offsets * B if len(offsets) == 1 else offsets
        ids = inputs.tolist() if not inputs.is_cuda else inputs.cpu().tolist()
        entries, live = [], []
        for b, slot in enumerate(slots):
            if slot is None:
                continue
            if slot[0].offset != offsets[b]:
                raise ValueError(f"row {b}: offset {offsets[b]} but its cache holds {slot[0].offset} tokens")
            if isinstance(first, BatchingKvCache) and first.max_seq_len is not None and offsets[b] + L > first.max_seq_len:
                raise ValueError("Paged batch append exceeds max_seq_len")
            entries.append(RaggedEntry(ids[b], slot, want=range(L - keep, L)))
            live.append(b)
        logits = self.forward_ragged(entries).view(len(live), keep, self.vocab_size)
        if len(live) == B:
            return logits
        out = torch.zeros((B, keep, self.vocab_size), dtype=logits.dtype, device=logits.device)
        out[torch.tensor(live, device=logits.device)] = logits
        return out
