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
of prompt portions and single tokens (``ragged.py``), which the batcher's mixed mode calls directly (all three come
from ``RaggedDecoderModel``; this class supplies the layers, ``_forward_plan``).  Compute dtype
bf16 (serving) or fp32 (every product in true fp32); norms, softmax, router, residual sum are fp32 in both.
"""

from __future__ import annotations

import torch

from extensions_b200.tiny_llm_ext_b200 import blocks

from .basics import linear_wide
from .latent_attention import LatentAttention
from .latent_kv_cache import LatentCacheView, LatentPagedCache, LatentPagedPool
from .layer_norm import ResidualRMSNorm
from .mlp import GatedMLP, MixtureOfExperts, TopKRouter
from .ragged import RaggedPlan
from .ragged_model import RaggedDecoderModel

MIXER_TYPES = {
    # type -> (interleaved rotary pairs, sliding window from mixer.mask.size)
    "latent_attention": (False, False),
    "latent_attention_2": (True, True),
}


class VoluzenLayer:
    def __init__(self, mixer: LatentAttention, norm1: ResidualRMSNorm, mlp, norm2: ResidualRMSNorm | None, slab_index: int):
        self.mixer, self.norm1, self.mlp, self.norm2, self.slab_index = mixer, norm1, mlp, norm2, slab_index


class VoluzenModel(RaggedDecoderModel):
    graph_env = "TL_VOLUZEN_GRAPH"
    architecture = "Voluzen"

    def __init__(self, config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda", page_size: int = 64, max_tokens: int | None = None,
                 max_requests: int | None = None):  # max_requests: accepted for all designs; no per-request state here
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Voluzen runs in bfloat16 or float32")
        self.config, self.precision, self.device = config, dtype, torch.device(device)
        self.vocab_size, self.hidden_size = int(config["vocab"]), int(config["width"])
        self.eps = float(config["norm"]["eps"])
        self.num_hidden_layers = len(config["layers"])
        self.page_size = page_size
        self._init_step()

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
