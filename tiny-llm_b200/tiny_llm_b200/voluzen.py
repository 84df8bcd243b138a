"""Voluzen: a decoder-only model of latent-attention layers (causal or sliding-window, some reading another layer's
latent cache) with dense or mixture-of-experts feed-forwards, sublayer-output norms with layer scale, and a residual
stream kept in fp32.

A layer is ``x <- x + ls1 * norm1(mixer(x))`` then ``x <- x + ls2 * norm2(ff(x))`` (norm weights stored around zero;
the sublayers read ``x`` itself, rounded to the compute dtype).  Everything the design lets vary comes from
``config.json``: ``vocab``, ``width``, ``norm.eps`` and per layer ``type`` (``latent_attention``: causal, half-pair
rotary layout; ``latent_attention_2``: sliding window ``mixer.mask.size``, interleaved rotary layout), the mixer's
sizes (``heads dim rot_dim vdim kv_rank scale rot.{dims,base}``, optional ``kv_from``) and ``mlp`` (``dense`` with
``ff`` and the tanh GELU; ``moe`` with ``router.{experts,top}``, ``expert.ff``, optional ``shared.ff`` and SiLU; or
none).  Weights: ``embed``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,o}``, ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.{router,router.b,e<k>.*,shared.*}``, ``l<i>.{norm1,norm2,ls1,ls2}``, ``final.norm``, ``head``.

The model is the framework's usual object: ``create_kv_cache()`` + ``model(inputs, offset, cache, logits_to_keep)``
serve ``greedy_generate_ids`` and ``ContinuousBatcher``; underneath both is ``forward_ragged``, one step over any mix
of prompt portions and single tokens (``ragged.py``), which the batcher's mixed mode calls directly.  Compute dtype
bf16 (serving) or fp32 (every product in true fp32); norms, softmax, router, residual sum are fp32 in both.
"""

from __future__ import annotations

import os

import torch

from extensions_b200.tiny_llm_ext_b200 import blocks

from .basics import linear_wide
from .kv_cache import BatchingKvCache
from .latent_attention import LatentAttention
from .latent_kv_cache import LatentCacheView, LatentPagedCache, LatentPagedPool
from .layer_norm import ResidualRMSNorm
from .mlp import GatedMLP, MixtureOfExperts, TopKRouter
from .ragged import RaggedEntry, RaggedPlan

MIXER_TYPES = {
    # type -> (interleaved rotary pairs, sliding window from mixer.mask.size)
    "latent_attention": (False, False),
    "latent_attention_2": (True, True),
}


class VoluzenLayer:
    def __init__(self, mixer: LatentAttention, norm1: ResidualRMSNorm, mlp, norm2: ResidualRMSNorm | None, slab_index: int):
        self.mixer, self.norm1, self.mlp, self.norm2, self.slab_index = mixer, norm1, mlp, norm2, slab_index


class VoluzenModel:
    architecture = "Voluzen"

    def __init__(self, config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda", page_size: int = 64, max_tokens: int | None = None):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Voluzen runs in bfloat16 or float32")
        self.config, self.precision, self.device = config, dtype, torch.device(device)
        self.vocab_size, self.hidden_size = int(config["vocab"]), int(config["width"])
        self.eps = float(config["norm"]["eps"])
        self.num_hidden_layers = len(config["layers"])
        self.page_size = page_size
        self.h2d_bytes = 0
        # Decode-only steps (every entry brings one token) replay a captured CUDA graph, one per (number of entries, block
        # table width); the step's integers are data in one device block.  None = on for CUDA, False = always eager.
        self.use_decode_graph: bool | None = None if os.environ.get("TL_VOLUZEN_GRAPH", "1") != "0" else False
        self._graphs: dict = {}
        self.graph_replays = self.graph_captures = 0

        def take(name: str) -> torch.Tensor:
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            t = tensors[name]
            return t.to(device=self.device, dtype=dtype if t.is_floating_point() else t.dtype).contiguous()

        self.embed = take("embed")
        if tuple(self.embed.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError("embed does not match vocab x width")
        self.layers: list[VoluzenLayer] = []
        slab_of: dict[int, int] = {}   # caching layer -> slab index
        widths: list[int] = []
        for i, spec in enumerate(config["layers"]):
            if spec["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {spec['type']!r}")
            interleaved, windowed = MIXER_TYPES[spec["type"]]
            m, p = spec["mixer"], f"l{i}.mix."
            source = m.get("kv_from")
            own = source is None
            if not own:
                src = config["layers"][source]["mixer"]
                if source not in slab_of or (src["kv_rank"], src["rot_dim"]) != (m["kv_rank"], m["rot_dim"]):
                    raise ValueError(f"layer {i}: kv_from={source} must name an earlier layer with its own latent of the same sizes")
            mixer = LatentAttention(
                heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"],
                rot_dims=m["rot"]["dims"], rot_base=m["rot"]["base"], interleaved=interleaved,
                window=m["mask"]["size"] if windowed else None, eps=self.eps,
                w_q=take(p + "q"), w_uk=take(p + "uk"), w_uv=take(p + "uv"), w_o=take(p + "o"),
                w_dkv=take(p + "dkv") if own else None, dkv_norm=take(p + "dkv.norm") if own else None)
            if own:
                slab_of[i] = len(widths)
                widths.append(mixer.cache_width)
            norm1 = ResidualRMSNorm(take(f"l{i}.norm1"), self.eps, weight_offset=1.0, scale=take(f"l{i}.ls1"))
            mlp, norm2 = self._feed_forward(spec.get("mlp"), f"l{i}.mlp.", take), None
            if mlp is not None:
                norm2 = ResidualRMSNorm(take(f"l{i}.norm2"), self.eps, weight_offset=1.0, scale=take(f"l{i}.ls2"))
            self.layers.append(VoluzenLayer(mixer, norm1, mlp, norm2, slab_of[i if own else source]))
        self.final_norm = ResidualRMSNorm(take("final.norm"), self.eps, weight_offset=1.0)
        self.head = take("head")
        max_pages = None if max_tokens is None else -(-int(max_tokens) // page_size)
        self.page_pool = LatentPagedPool(widths, page_size=page_size, dtype=dtype, device=self.device, max_pages=max_pages)
        # the attention work-list granularities the layers use (one list per size in every step's plan)
        self.tile_sizes = sorted({blocks.attention_kernel(dtype, l.mixer.heads, l.mixer.rank, l.mixer.rot_dim, page_size)[1] for l in self.layers})

    @staticmethod
    def _feed_forward(spec, prefix: str, take):
        if not spec:
            return None
        if spec["kind"] == "dense":
            return GatedMLP(take(prefix + "gate"), take(prefix + "up"), take(prefix + "down"), "gelu_tanh")
        if spec["kind"] != "moe":
            raise ValueError(f"unknown feed-forward kind {spec['kind']!r}")
        experts, top = int(spec["router"]["experts"]), int(spec["router"]["top"])
        router = TopKRouter(take(prefix + "router"), take(prefix + "router.b"), top)
        stack = lambda part: torch.stack([take(f"{prefix}e{k}.{part}") for k in range(experts)]).contiguous()
        shared = None
        if spec.get("shared"):
            shared = GatedMLP(take(prefix + "shared.gate"), take(prefix + "shared.up"), take(prefix + "shared.down"), "silu")
        return MixtureOfExperts(router, stack("gate"), stack("up"), stack("down"), "silu", shared)

    @classmethod
    def from_checkpoint(cls, config: dict, tensors: dict, **kwargs) -> "VoluzenModel":
        return cls(config, tensors, **kwargs)

    # ---- cache ---------------------------------------------------------------------
    def create_kv_cache(self) -> list:
        """One entry per layer (what the schedulers expect); all are faces of ONE page list, held by entry 0."""
        owner = LatentPagedCache(self.page_pool)
        return [owner] + [LatentCacheView(owner, layer.slab_index) for layer in self.layers[1:]]

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
        if state is not None and state.get("slabs") not in (None, self.page_pool.slab_version):
            state = None  # captured against slabs that have been reallocated since
        if state is None:
            self._graphs[key] = {"slabs": None}
            plan = RaggedPlan(entries, self.device, self.tile_sizes)
            self.h2d_bytes += plan.h2d_bytes
            return self._forward_plan(plan)
        if state["slabs"] is None:
            total = 3 * S + S + S * width + 3 * S * len(self.tile_sizes)
            state["block"] = torch.zeros(total, dtype=torch.int32, device=self.device)
            plan = RaggedPlan(entries, self.device, self.tile_sizes, max_pages=width, into=state["block"])
            state["slabs"] = self.page_pool.slab_version  # the append may have grown the pool: read it after the plan
            torch.cuda.current_stream(self.device).synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                state["logits"] = self._forward_plan(plan)
            state["graph"], state["plan"] = graph, plan
            self.graph_captures += 1
        else:
            plan = RaggedPlan(entries, self.device, self.tile_sizes, max_pages=width, into=state["block"])
            if self.page_pool.slab_version != state["slabs"]:  # this very append moved the slabs: run it eagerly, re-capture next time
                self._graphs.pop(key)
                return self._forward_plan(plan)
            state["host"] = plan._host
        self.h2d_bytes += plan.h2d_bytes
        state["graph"].replay()
        self.graph_replays += 1
        return state["logits"].clone()

    def _forward_plan(self, plan: RaggedPlan) -> torch.Tensor:
        exact = self.precision == torch.float32
        tf32 = torch.backends.cuda.matmul.allow_tf32
        if exact:
            torch.backends.cuda.matmul.allow_tf32 = False  # fp32 means fp32
        try:
            slabs = self.page_pool.slabs
            x32, h = blocks.embed_rows(plan.ids, self.embed)
            for layer in self.layers:
                h = layer.norm1(layer.mixer(h, plan, slabs[layer.slab_index]), residual=x32)
                if layer.mlp is not None:
                    y = layer.mlp(h, wide=True) if isinstance(layer.mlp, GatedMLP) else layer.mlp(h)
                    h = layer.norm2(y, residual=x32)
            if plan.num_want == 0:  # a portion whose logits nobody asked for: the caches are filled, that is all
                return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
            rows = x32.index_select(0, plan.want_rows.long())
            return linear_wide(self.final_norm(rows), self.head)
        finally:
            if exact:
                torch.backends.cuda.matmul.allow_tf32 = tf32

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
