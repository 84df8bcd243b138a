"""Plain, slow restatement of the Voluzen design on CPU tensors, one function per mechanism.

Written from the design's equations only; shares no code with the product path.  Every function
works on whole sequences in the dtype of its inputs (float64 or float32), with no cache: a token's
output is computed from all tokens before it.  Notation: ``T`` tokens, ``D`` model width,
``H`` heads, ``dn`` un-rotated and ``dr`` rotated query/key dimensions per head, ``dv`` value
dimensions per head, ``R`` latent rank.

``weights`` maps tensor names (``l<i>.mix.q`` ...) to tensors; ``config`` is the parsed
``config.json``.
"""

from __future__ import annotations

import math

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def norm_zero_centred(x, w, eps):
    """The layers' and the model's norm: the stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    """The latent's norm: the stored weight multiplies as it is."""
    return rms_unit(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, interleaved: bool) -> torch.Tensor:
    """Rotary positions on the first ``dims`` entries of the last axis of ``x [T, ..., d]``.

    Pair i is (i, i + dims/2) in the half layout and (2i, 2i+1) in the interleaved one;
    angle = position * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]            # [T, half]
    cos, sin = torch.cos(angle).to(x.dtype), torch.sin(angle).to(x.dtype)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = cos.reshape(shape), sin.reshape(shape)
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def visible(T: int, window: int | None) -> torch.Tensor:
    """[T, T] boolean: query i sees key j when j <= i and, with a window, i - j < window."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    keep = j <= i
    if window is not None:
        keep = keep & (i - j < window)
    return keep


def latent_of(h, weights, prefix, mixer, eps, interleaved):
    """What a latent-attention layer caches: the normed latent ``c [T, R]`` and the rotated shared
    key part ``kr [T, dr]``."""
    R, dr = mixer["kv_rank"], mixer["rot_dim"]
    down = h @ weights[prefix + "dkv"].T
    c = norm_plain(down[:, :R], weights[prefix + "dkv.norm"], eps)
    positions = torch.arange(h.shape[0])
    kr = rotate(down[:, R : R + dr], positions, mixer["rot"]["dims"], mixer["rot"]["base"], interleaved)
    return c, kr


def latent_attention(h, weights, prefix, mixer, c, kr, interleaved, window):
    """Latent attention of one layer given the cached pair (its own, or another layer's)."""
    T = h.shape[0]
    H, dn, dr, dv, R = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    q = (h @ weights[prefix + "q"].T).reshape(T, H, dn + dr)
    q_plain = q[..., :dn]
    q_rot = rotate(q[..., dn:], torch.arange(T), mixer["rot"]["dims"], mixer["rot"]["base"], interleaved)
    k_plain = (c @ weights[prefix + "uk"].T).reshape(T, H, dn)
    value = (c @ weights[prefix + "uv"].T).reshape(T, H, dv)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, kr)
    scores = scores * mixer["scale"]
    scores = scores.masked_fill(~visible(T, window)[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", p, value).reshape(T, H * dv)
    return out @ weights[prefix + "o"].T


def gated_ff(h, weights, prefix, act):
    return (act(h @ weights[prefix + "gate"].T) * (h @ weights[prefix + "up"].T)) @ weights[prefix + "down"].T


def route(h, weights, prefix, top):
    """Indices [T, top] of the largest router logits and the softmax over those logits only."""
    z = h @ weights[prefix + "router"].T + weights[prefix + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def mixture_ff(h, weights, prefix, mlp):
    idx, gate = route(h, weights, prefix, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(idx.shape[1]):
            e = int(idx[t, slot])
            out[t] += gate[t, slot] * gated_ff(h[t : t + 1], weights, f"{prefix}e{e}.", silu)[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, weights, prefix + "shared.", silu)
    return out


def feed_forward(h, weights, prefix, mlp):
    if mlp["kind"] == "dense":
        return gated_ff(h, weights, prefix, gelu_tanh)
    return mixture_ff(h, weights, prefix, mlp)


def forward(config, weights, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept: dict[int, tuple] = {}
    stream = []
    for i, layer in enumerate(config["layers"]):
        mixer, p = layer["mixer"], f"l{i}.mix."
        interleaved = layer["type"] == "latent_attention_2"
        window = mixer["mask"]["size"] if (interleaved and mixer.get("mask")) else None
        if mixer.get("kv_from") is not None:
            c, kr = kept[mixer["kv_from"]]
        else:
            c, kr = latent_of(x, w, p, mixer, eps, interleaved)
            kept[i] = (c, kr)
        y = latent_attention(x, w, p, mixer, c, kr, interleaved, window)
        x = x + norm_zero_centred(y, w[f"l{i}.norm1"], eps) * w[f"l{i}.ls1"]
        if layer.get("mlp"):
            y = feed_forward(x, w, f"l{i}.mlp.", layer["mlp"])
            x = x + norm_zero_centred(y, w[f"l{i}.norm2"], eps) * w[f"l{i}.ls2"]
        stream.append(x)
    logits = norm_zero_centred(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(stream)) if return_layers else logits


def cache_attention(q_full, rows, positions, rank, window, scale):
    """Multi-query attention straight on cache rows: query ``q_full [T, H, rank+rot]`` at ``positions`` against keys
    ``rows [S, rank+rot]`` (key j at position j), values = the first ``rank`` entries of the rows."""
    scores = torch.einsum("thd,jd->thj", q_full, rows) * scale
    j = torch.arange(rows.shape[0])[None, :]
    p = positions[:, None]
    keep = j <= p
    if window:
        keep = keep & (p - j < window)
    scores = scores.masked_fill(~keep[:, None, :], float("-inf"))
    return torch.einsum("thj,jr->thr", torch.softmax(scores, dim=-1), rows[:, :rank])


def greedy(config, weights, prompt, steps):
    """Greedy continuation by full recomputation."""
    ids, out = list(prompt), []
    for _ in range(steps):
        ids.append(int(forward(config, weights, ids)[-1].argmax()))
        out.append(ids[-1])
    return out
