"""Bapovik: a decoder-only model whose layers add a mixer and a mixture-of-experts feed-forward, both reading ONE norm
of the residual stream (``x <- x + mixer(n) + ff(n)``, ``n = norm1(x)``), to a stream kept in fp32.

Two kinds of layers (``type``):

- ``attention``: grouped-query attention over a sliding window (``mixer.mask.size``) without positions in the scores,
  biased q / k / v projections, a sigmoid output gate per head; with ``mixer.kv_from = j`` the layer has no key / value
  projections and reads layer j's cache with its own queries and mask.
- ``parallel``: two mixers side by side on the same input, ``mixer.left`` = attention within chunks of
  ``mask.size`` positions, with per-head RMS norms of queries and keys, a tanh soft cap on the scores and a sink in the
  softmax; ``mixer.right`` = linear attention with a per-channel decay (``tau``) and a recurrent fp32 state.  Each
  output is RMS-normed over the width (``left.out`` / ``right.out``) and the layer takes half their sum.

The feed-forward (``mlp``, or none): a sigmoid router picks ``router.top`` of ``router.experts`` experts
``down(relu(up x)^2)``, each run on its score times the token.  Everything that can differ between models of the
design is read from ``config.json``: ``vocab``, ``width``, ``norm.eps``, the list ``layers`` with the sizes above
(``heads kv_heads dim vdim scale softcap tau``).  Weights: ``embed``, ``l<i>.norm1``, ``l<i>.mix.{q,k,v}`` with
``.b`` biases, ``l<i>.mix.{g,o}``, for a parallel layer ``l<i>.mix.left.{q,k,v,g,o,q.norm,k.norm,out}`` and
``l<i>.mix.right.{q,k,v,g,o,norm,a1,a2,a2.b,out}``, ``l<i>.mlp.{router,e<k>.up,e<k>.down}``, ``final.norm``, ``head``.

The model is the framework's usual object (``RaggedDecoderModel``): ``create_kv_cache()`` +
``model(inputs, offset, cache, logits_to_keep)`` serve ``greedy_generate_ids`` and ``ContinuousBatcher``, and
``forward_ragged`` runs one step over any mix of prompt portions and single tokens.  A request holds one page list for
all attention layers (``LatentPagedPool``: one slab per caching layer, rows of ``kv_heads * (dim + vdim)``) and one slot
of the ``StateSlotPool`` for all recurrent layers.  Compute dtype bf16 (serving) or fp32 (every product in true fp32);
norms, softmax, router, decays, recurrent state and the residual sum are fp32 in both.
"""

from __future__ import annotations

import torch

from extensions_b200.tiny_llm_ext_b200 import blocks

from .basics import linear_wide
from .latent_kv_cache import LatentCacheView, LatentPagedPool
from .linear_attention import DecayedLinearAttention
from .mlp import MixtureOfExperts, TopKRouter
from .paged_attention import FusedProjection, PagedGroupedAttention
from .ragged import RaggedPlan
from .ragged_model import RaggedDecoderModel
from .state_cache import HybridPagedCache, StateSlotPool


class BapovikLayer:
    def __init__(self, kind: str, norm_weight, proj: FusedProjection, attention: PagedGroupedAttention, prefix: str, slab_index: int, mlp,
                 recurrent: DecayedLinearAttention | None = None, state_offset: int = 0, out_weights=None):
        self.kind, self.norm_weight, self.proj, self.attention, self.prefix = kind, norm_weight, proj, attention, prefix
        self.slab_index, self.mlp, self.recurrent, self.state_offset, self.out_weights = slab_index, mlp, recurrent, state_offset, out_weights


class BapovikModel(RaggedDecoderModel):
    architecture = "Bapovik"
    graph_env = "TL_BAPOVIK_GRAPH"

    def __init__(self, config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda", page_size: int = 64, max_tokens: int | None = None,
                 max_requests: int | None = None):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Bapovik runs in bfloat16 or float32")
        self.config, self.precision, self.device = config, dtype, torch.device(device)
        self.vocab_size, self.hidden_size = int(config["vocab"]), int(config["width"])
        self.eps = float(config["norm"]["eps"])
        self.num_hidden_layers = len(config["layers"])
        self.page_size = page_size
        self.stream_tap: list | None = None  # a list here receives a copy of the residual stream after every layer
        self._init_step()

        def take(name: str) -> torch.Tensor:
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            t = tensors[name]
            return t.to(device=self.device, dtype=dtype if t.is_floating_point() else t.dtype).contiguous()

        self.embed = take("embed")
        if tuple(self.embed.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError("embed does not match vocab x width")
        self.layers: list[BapovikLayer] = []
        slab_of: dict[int, int] = {}  # caching layer -> slab index
        widths: list[int] = []
        state_floats = 0
        for i, spec in enumerate(config["layers"]):
            kind, m = spec["type"], spec["mixer"]
            if kind not in ("attention", "parallel"):
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            a = m if kind == "attention" else m["left"]
            p = f"l{i}.mix." + ("" if kind == "attention" else "left.")
            source = a.get("kv_from") if kind == "attention" else None
            own = source is None
            if not own:
                src = config["layers"][source] if isinstance(source, int) and 0 <= source < i else None
                src = None if src is None else (src["mixer"] if src["type"] == "attention" else src["mixer"]["left"])
                if source not in slab_of or (src["kv_heads"], src["dim"], src["vdim"]) != (a["kv_heads"], a["dim"], a["vdim"]):
                    raise ValueError(f"layer {i}: kv_from={source} must name an earlier layer with its own keys and values of the same sizes")
            normed = kind == "parallel"
            attention = PagedGroupedAttention(
                heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], vdim=a["vdim"], scale=a["scale"],
                mask="chunk" if kind == "parallel" else "window", mask_size=a["mask"]["size"], w_o=take(p + "o"), softcap=a.get("softcap"),
                sink=kind == "parallel", q_norm=take(p + "q.norm") if normed else None, k_norm=take(p + "k.norm") if normed and own else None,
                eps=self.eps, caches=own, page_size=page_size)
            parts = [(p + "q", take(p + "q"), take(p + "q.b"))]
            if own:
                parts += [(p + "k", take(p + "k"), take(p + "k.b")), (p + "v", take(p + "v"), take(p + "v.b"))]
                slab_of[i] = len(widths)
                widths.append(attention.cache_width)
            parts.append((p + "g", take(p + "g"), None))
            recurrent, offset, outs = None, 0, None
            if kind == "parallel":
                r, rp = m["right"], f"l{i}.mix.right."
                recurrent = DecayedLinearAttention(heads=r["heads"], dim=r["dim"], vdim=r["vdim"], tau=r["tau"], w_a2=take(rp + "a2"), a2_bias=take(rp + "a2.b"),
                                                   norm_weight=take(rp + "norm"), w_o=take(rp + "o"), eps=self.eps)
                parts += [(rp + name, take(rp + name), None) for name in ("q", "k", "v", "g", "a1")]
                offset = state_floats
                state_floats += r["heads"] * r["dim"] * r["vdim"]
                outs = (take(f"l{i}.mix.left.out"), take(f"l{i}.mix.right.out"))
            self.layers.append(BapovikLayer(kind, take(f"l{i}.norm1"), FusedProjection(parts, dtype, self.device), attention, p,
                                            slab_of[i if own else source], self._feed_forward(spec.get("mlp"), f"l{i}.mlp.", take), recurrent, offset, outs))
        self.final_norm = take("final.norm")
        self.head = take("head")
        max_pages = None if max_tokens is None else -(-int(max_tokens) // page_size)
        self.page_pool = LatentPagedPool(widths, page_size=page_size, dtype=dtype, device=self.device, max_pages=max_pages)
        self.state_pool = StateSlotPool(state_floats, device=self.device, max_slots=max_requests)
        self.tile_sizes = sorted({layer.attention.tile_tokens for layer in self.layers})

    @staticmethod
    def _feed_forward(spec, prefix: str, take):
        if not spec:
            return None
        if spec["kind"] != "moe":
            raise ValueError(f"unknown feed-forward kind {spec['kind']!r}")
        experts, top = int(spec["router"]["experts"]), int(spec["router"]["top"])
        router = TopKRouter(take(prefix + "router"), None, top, scoring="sigmoid")
        stack = lambda part: torch.stack([take(f"{prefix}e{k}.{part}") for k in range(experts)]).contiguous()
        return MixtureOfExperts(router, None, stack("up"), stack("down"), "relu_squared", weight_on="input")

    @classmethod
    def from_checkpoint(cls, config: dict, tensors: dict, **kwargs) -> "BapovikModel":
        return cls(config, tensors, **kwargs)

    # ---- cache ---------------------------------------------------------------------
    def create_kv_cache(self) -> list:
        """One entry per layer (what the schedulers expect); all are faces of ONE page list + state slot, held by entry 0."""
        owner = HybridPagedCache(self.page_pool, self.state_pool)
        return [owner] + [LatentCacheView(owner, layer.slab_index) for layer in self.layers[1:]]

    def _storage_version(self):
        return (self.page_pool.slab_version, self.state_pool.version)

    # ---- the layers over one plan ------------------------------------------------------
    def _forward_plan(self, plan: RaggedPlan) -> torch.Tensor:
        exact = self.precision == torch.float32
        tf32 = torch.backends.cuda.matmul.allow_tf32
        if exact:
            torch.backends.cuda.matmul.allow_tf32 = False  # fp32 means fp32
        try:
            slabs = self.page_pool.slabs
            x32, _ = blocks.embed_rows(plan.ids, self.embed)
            h = blocks.norm_residual(x32, self.layers[0].norm_weight, self.eps)
            for i, layer in enumerate(self.layers):
                y, p, a = layer.proj(h), layer.prefix, layer.attention
                mixed = a(y[p + "q"], y.get(p + "k"), y.get(p + "v"), y[p + "g"], plan, slabs[layer.slab_index])
                if layer.recurrent is not None:
                    r = layer.recurrent
                    rp = p[: -len("left.")] + "right."
                    state = self.state_pool.layer_view(layer.state_offset, r.state_shape)
                    right = r(y[rp + "q"], y[rp + "k"], y[rp + "v"], y[rp + "g"], y[rp + "a1"], plan, state)
                    mixed = blocks.norm_mix2(mixed, layer.out_weights[0], right, layer.out_weights[1], 0.5, self.eps)
                ff = layer.mlp(h) if layer.mlp is not None else None
                # the layer's sum, fused with the next layer's norm (the model's norm runs on the wanted rows only)
                following = self.layers[i + 1].norm_weight if i + 1 < len(self.layers) else None
                h = blocks.add_norm(x32, mixed, ff, following, self.eps)
                if self.stream_tap is not None:
                    self.stream_tap.append(x32.clone())
            if plan.num_want == 0:  # a portion whose logits nobody asked for: caches and states are filled, that is all
                return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
            rows = x32.index_select(0, plan.want_rows.long())
            return linear_wide(blocks.norm_residual(rows, self.final_norm, self.eps), self.head)
        finally:
            if exact:
                torch.backends.cuda.matmul.allow_tf32 = tf32
