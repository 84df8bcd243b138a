"""Plain, slow restatement of the Bapovik design on CPU tensors, one function per mechanism.

Written from the design's equations only; shares no code with the product path.  Every function
works on one whole sequence in the dtype of its inputs (float64 or float32), without a cache or a
carried state: a token's output is computed from all tokens before it, by explicit loops where
that is the clearest form.  Notation: ``T`` tokens, ``D`` model width, ``H`` query heads, ``G``
key/value heads, ``dk`` query/key and ``dv`` value entries per head.

``weights`` maps tensor names (``l<i>.mix.q`` ...) to tensors; ``config`` is the parsed
``config.json``.
"""

from __future__ import annotations

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def relu_squared(z):
    return torch.relu(z).pow(2)


def silu(z):
    return z * torch.sigmoid(z)


def visible(i: int, j: int, kind: str, size: int) -> bool:
    """May position i look at position j?  ``window``: itself and the size-1 positions before it;
    ``chunk``: earlier positions of its own block of ``size`` positions counted from 0."""
    if j > i:
        return False
    if kind == "causal":
        return True
    if kind == "window":
        return i - j < size
    if kind == "chunk":
        return i // size == j // size
    raise ValueError(kind)


def masked_attention(q, k, v, *, scale, kind, size, softcap=None, sink=False):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv].  Query head h reads key/value head
    h // (H / G).  Scores are scaled, optionally squashed to softcap * tanh(s / softcap); with
    ``sink`` the softmax's denominator has one extra term exp(0) that carries no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, kind, size)]
        idx = torch.tensor(js)
        for h in range(H):
            g = h // per
            s = (k[idx, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            m = s.max()
            if sink:
                m = torch.clamp(m, min=0.0)
            e = torch.exp(s - m)
            denom = e.sum() + (torch.exp(-m) if sink else 0.0)
            out[i, h] = (e / denom) @ v[idx, g]
    return out


def gated_attention(h, weights, prefix, spec, *, eps, kind, keys_values=None, qk_norm=False, softcap=None, sink=False):
    """The softmax-attention mixer: biased projections, optional per-head RMS norm of queries and
    keys, masked attention, one sigmoid gate per head, output projection.  ``keys_values`` = (k, v)
    of another layer replaces this layer's own.  Returns (output [T, D], (k, v) as cached)."""
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    w = lambda name: weights[prefix + name].to(h.dtype)
    q = (h @ w("q").T + w("q.b")).view(T, H, dk)
    if qk_norm:
        q = norm_plain(q, w("q.norm"), eps)
    if keys_values is None:
        k = (h @ w("k").T + w("k.b")).view(T, G, dk)
        v = (h @ w("v").T + w("v.b")).view(T, G, dv)
        if qk_norm:
            k = norm_plain(k, w("k.norm"), eps)
    else:
        k, v = keys_values
    o = masked_attention(q, k, v, scale=spec["scale"], kind=kind, size=spec["mask"]["size"], softcap=softcap, sink=sink)
    gate = torch.sigmoid(h @ w("g").T)                       # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ w("o").T, (k, v)


def decayed_linear_attention(q, k, v, alpha):
    """q, k, alpha [T, H, dk], v [T, H, dv] -> [T, H, dv].  Per head a matrix S [dk, dv] starts at
    zero; at every token its row c is multiplied by alpha[t, c], then k_t v_t^T is added, and the
    output is S^T q_t."""
    T, H, dk = q.shape
    dv = v.shape[2]
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    S = torch.zeros((H, dk, dv), dtype=q.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hc,hcv->hv", q[t], S)
    return out


def gated_linear_mixer(h, weights, prefix, spec, *, eps):
    """The recurrent mixer: queries scaled by dk^-1/2, a per-channel decay sigmoid(z)^(1/tau) from a
    low-rank projection, the decayed recurrence, per-head RMS norm, a SiLU gate, output projection."""
    H, dk, dv, tau = spec["heads"], spec["dim"], spec["vdim"], spec["tau"]
    T = h.shape[0]
    w = lambda name: weights[prefix + name].to(h.dtype)
    q = (h @ w("q").T).view(T, H, dk) * dk ** -0.5
    k = (h @ w("k").T).view(T, H, dk)
    v = (h @ w("v").T).view(T, H, dv)
    z = (h @ w("a1").T) @ w("a2").T + w("a2.b")
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, dk)
    o = decayed_linear_attention(q, k, v, alpha)
    o = norm_plain(o, w("norm"), eps).reshape(T, H * dv)
    return (o * silu(h @ w("g").T)) @ w("o").T


def expert_mixture(h, weights, prefix, spec):
    """Sigmoid router; the ``top`` largest scores choose the experts; each chosen expert runs on its
    score times h; the outputs are summed."""
    E, top = spec["router"]["experts"], spec["router"]["top"]
    w = lambda name: weights[prefix + name].to(h.dtype)
    scores = torch.sigmoid(h @ w("router").T)                 # [T, E]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(scores[t, e]), e))[:top]
        for e in order:
            x = scores[t, e] * h[t]
            out[t] += relu_squared(x @ w(f"e{e}.up").T) @ w(f"e{e}.down").T
    return out


def layer_forward(x, weights, config, i, cached):
    """One layer on the residual stream x [T, D]; ``cached[j]`` = (k, v) of caching layer j."""
    spec = config["layers"][i]
    eps = config["norm"]["eps"]
    h = norm_plain(x, weights[f"l{i}.norm1"].to(x.dtype), eps)
    m, p = spec["mixer"], f"l{i}.mix."
    if spec["type"] == "attention":
        src = m.get("kv_from")
        y, kv = gated_attention(h, weights, p, m, eps=eps, kind="window", keys_values=None if src is None else cached[src])
        if src is None:
            cached[i] = kv
    elif spec["type"] == "parallel":
        left, _ = gated_attention(h, weights, p + "left.", m["left"], eps=eps, kind="chunk", qk_norm=True,
                                  softcap=m["left"].get("softcap"), sink=True)
        right = gated_linear_mixer(h, weights, p + "right.", m["right"], eps=eps)
        y = 0.5 * (norm_plain(left, weights[p + "left.out"].to(x.dtype), eps) + norm_plain(right, weights[p + "right.out"].to(x.dtype), eps))
    else:
        raise ValueError(spec["type"])
    if spec.get("mlp"):
        y = y + expert_mixture(h, weights, f"l{i}.mlp.", spec["mlp"])
    return x + y


def forward(tokens, weights, config, dtype=torch.float64, trace=None):
    """Token ids [T] -> logits [T, vocab]; ``trace``, a list, receives the stream after every layer."""
    x = weights["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    cached: dict = {}
    for i in range(len(config["layers"])):
        x = layer_forward(x, weights, config, i, cached)
        if trace is not None:
            trace.append(x.clone())
    x = norm_plain(x, weights["final.norm"].to(dtype), config["norm"]["eps"])
    return x @ weights["head"].to(dtype).T


def greedy(tokens, weights, config, new: int, dtype=torch.float64) -> list:
    """``new`` greedy tokens after the prompt, by recomputing the whole sequence for each."""
    ids, out = list(tokens), []
    for _ in range(new):
        nxt = int(forward(ids, weights, config, dtype=dtype)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
