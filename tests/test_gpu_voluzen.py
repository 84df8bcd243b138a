"""Voluzen on a B200 against the plain CPU restatement (oracle/voluzen.py, float64): each mechanism of the
blocks library alone, then the model through every way of cutting and batching a sequence, the schedulers and the
entry points.  Small made-up configurations and random weights; where random weights would hide a fault (one far key
among hundreds, a window's edge) the inputs are built so that one score stands out.

Tolerances: relative root-mean-square error of a logits row (mean taken off) below 5e-5 in float32 mode - every
product in true fp32, so only summation order differs - and below 1e-1 in bfloat16 mode (at widths of 64 to 96 the
rounding of bf16 activations alone gives 1e-2 typically and up to 1e-1 on single rows, so whole schedules are held to a
median of 3e-2 and a worst row of 2e-1; a fault of the logic gives 3e-1 and more, and the float32 run is the sharp test).
"""

import math

import pytest
import torch

from oracle import voluzen as O
from extensions_b200.tiny_llm_ext_b200 import blocks
from tiny_llm_b200 import BatchingKvCache, ContinuousBatcher, greedy_generate_ids
from tiny_llm_b200.models import load_model, model_class
from tiny_llm_b200.ragged import RaggedEntry
from tiny_llm_b200.synthetic import save_voluzen, synthetic_voluzen, voluzen_config

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 5e-5, torch.bfloat16: 1e-1}


@pytest.fixture(scope="module")
def dev(cuda_device):
    return cuda_device


def row_error(got, want):
    d = (got.double().cpu() - want.double())
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max().item()


def rows_match(got, want, dtype):
    if dtype == torch.float32:
        return row_error(got, want) < TOL[dtype]
    d = (got.double().cpu() - want.double())
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)
    return err.median().item() < 3e-2 and err.max().item() < 2 * TOL[dtype]


def decisive_routers(tensors):
    """For runs in bfloat16: a random router has close calls that an 8-bit mantissa decides the other way for a few
    tokens, and such a row then differs by far more than rounding.  Here the bias separates the experts by a wide
    margin (the chosen set is fixed, the weights among the chosen still follow the token), so every row can be held
    to the rounding bound.  The float32 runs keep the random routers, with choices that change from token to token."""
    out = dict(tensors)
    for name, t in tensors.items():
        if name.endswith(".router"):
            out[name] = (0.05 * t.float()).to(t.dtype)
        elif name.endswith(".router.b"):
            order = torch.randperm(t.numel(), generator=torch.Generator().manual_seed(t.numel()))
            out[name] = order.to(torch.float32).to(t.dtype)
    return out


def close(got, want, tol):
    got, want = got.double().cpu(), want.double()
    err = (got - want).abs().max().item()
    scale = want.abs().max().item() + 1e-9
    assert err <= tol * scale, (err, scale)


def ids_for(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [48, 256, 1000])
def test_norm_with_offset_scale_and_residual(dev, dtype, dim):
    g = torch.Generator().manual_seed(dim)
    y, w, ls, x = torch.randn(5, dim, generator=g), 0.1 * torch.randn(dim, generator=g), torch.randn(dim, generator=g), torch.randn(5, dim, generator=g)
    yq, wq, lq = y.to(dtype), w.to(dtype), ls.to(dtype)
    want = x.double() + O.norm_zero_centred(yq.double(), wq.double(), 1e-5) * lq.double()
    res = x.to(dev).clone()
    h = blocks.norm_residual(yq.to(dev), wq.to(dev), 1e-5, weight_offset=1.0, scale=lq.to(dev), residual=res)
    close(res, want, 1e-6)                      # the residual is fp32 in both modes
    assert torch.equal(h.cpu(), res.cpu().to(dtype))
    plain = blocks.norm_residual(x.to(dev), wq.to(dev), 1e-3)  # fp32 input, plain weight, no residual
    close(plain, O.norm_plain(x.double(), wq.double(), 1e-3), 1e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rotary_layouts_and_far_positions(dev, interleaved):
    g = torch.Generator().manual_seed(3)
    heads, dn, dr, dims = 3, 8, 12, 8   # rotate 8 of the 12 trailing entries of each head
    x = torch.randn(6, heads * (dn + dr), generator=g)
    pos = torch.tensor([0, 1, 63, 64, 4097, 100000], dtype=torch.int32)
    want = x.double().reshape(6, heads, dn + dr).clone()
    want[..., dn:] = O.rotate(want[..., dn:], pos, dims, 5000.0, interleaved)
    got = blocks.rope_rows(x.to(dev), pos.to(dev), heads=heads, head_stride=dn + dr, first=dn, dims=dims, base=5000.0, interleaved=interleaved)
    close(got.reshape(6, heads, dn + dr), want, 2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activations(dev, dtype):
    gu = (3 * torch.randn(7, 2 * 40, generator=torch.Generator().manual_seed(0))).to(dtype)
    for act, fn in ((blocks.ACT_SILU, O.silu), (blocks.ACT_GELU_TANH, O.gelu_tanh)):
        want = fn(gu[:, :40].double()) * gu[:, 40:].double()
        close(blocks.gated_act(gu.to(dev), act), want, 1e-6 if dtype == torch.float32 else 8e-3)


def test_argmax_rows_takes_the_lowest_index_of_a_tie(dev):
    x = torch.randn(5, 3000, generator=torch.Generator().manual_seed(1))
    x[2, 17] = x[2, 2900] = 99.0
    assert blocks.argmax_rows(x.to(dev)).tolist() == [int(v) for v in x.argmax(-1)[:2]] + [17] + [int(v) for v in x.argmax(-1)[3:]]


def build_cache(dev, dtype, rows, page_size, page_order):
    """A slab whose pages are deliberately out of order, holding ``rows [S, width]``."""
    S, width = rows.shape
    n_pages = -(-S // page_size)
    slab = torch.full((len(page_order) + 1, page_size, width), 7.0, dtype=dtype)  # stale rows are finite garbage
    for logical in range(n_pages):
        part = rows[logical * page_size : (logical + 1) * page_size]
        slab[page_order[logical], : part.shape[0]] = part.to(dtype)
    table = torch.full((1, n_pages + 1), -1, dtype=torch.int32)
    table[0, :n_pages] = torch.tensor(page_order[:n_pages], dtype=torch.int32)
    return slab.to(dev), table.to(dev)


def run_attention(dev, dtype, q_full, rows, positions, rank, window, scale, page_size=32, kernel=None):
    S = rows.shape[0]
    chosen, tile_tokens = blocks.attention_kernel(dtype, q_full.shape[1], rank, rows.shape[1] - rank, page_size)
    if kernel == "general":
        chosen, tile_tokens = "general", blocks.ATTENTION_TILE_TOKENS
    elif kernel is not None:
        assert chosen == kernel, "these sizes should go to the tensor-core kernel"
    order = list(reversed(range(-(-S // page_size))))
    slab, table = build_cache(dev, dtype, rows, page_size, order)
    T, H, width = q_full.shape
    q = q_full.to(dtype).to(dev)
    out = torch.empty((H, T, rank), dtype=dtype, device=dev)
    tiles, first = [], 0
    while first < T:  # runs of consecutive positions, at most 4 long
        n = 1
        while first + n < T and n < tile_tokens and positions[first + n] == positions[first + n - 1] + 1:
            n += 1
        tiles.append((first, n, 0))
        first += n
    blocks.latent_attention(q[:, :, :rank], q[:, :, rank:], slab, table, torch.tensor(tiles, dtype=torch.int32, device=dev),
                            positions.to(torch.int32).to(dev), window=window, scale=scale, out=out.transpose(0, 1), kernel=chosen,
                            max_context=S)  # few query rows over a long cache: the key range is split over CTAs and merged
    return out.transpose(0, 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot,heads", [(32, 8, 2), (96, 16, 4), (130, 6, 5), (33, 6, 3), (512, 64, 3), (640, 32, 2)])
def test_latent_attention_against_plain_attention(dev, dtype, rank, rot, heads):
    g = torch.Generator().manual_seed(rank)
    S = 150
    rows = torch.randn(S, rank + rot, generator=g).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 31, 32, 33, 63, 64, 65, 66, 100, 149])
    q = torch.randn(len(positions), heads, rank + rot, generator=g).to(dtype)
    for window in (0, 1, 33, 40):
        want = O.cache_attention(q.double(), rows.double(), positions, rank, window, 0.11)
        got = run_attention(dev, dtype, q, rows, positions, rank, window, 0.11)
        close(got, want, 5e-6 if dtype == torch.float32 else 1.5e-2)  # fp32: scores are dot products of up to 672 terms


@pytest.mark.parametrize("rank,rot,heads", [(32, 8, 1), (96, 16, 4), (130, 6, 5), (64, 32, 16), (256, 64, 40), (64, 8, 70), (512, 64, 3)])
def test_tensor_core_attention_against_plain_attention_and_the_general_kernel(dev, rank, rot, heads):
    g = torch.Generator().manual_seed(rank + heads)
    S = 520
    rows = torch.randn(S, rank + rot, generator=g).to(torch.bfloat16)
    positions = torch.tensor(list(range(0, 9)) + [30, 31, 32, 33, 34, 63, 64, 65] + list(range(120, 150)) + [199, 383, 384, 519])
    q = torch.randn(len(positions), heads, rank + rot, generator=g).to(torch.bfloat16)
    for window in (0, 1, 33, 64):
        want = O.cache_attention(q.double(), rows.double(), positions, rank, window, 0.09)
        got = run_attention(dev, torch.bfloat16, q, rows, positions, rank, window, 0.09, page_size=64, kernel="mma")
        close(got, want, 1.5e-2)
        close(got, run_attention(dev, torch.bfloat16, q, rows, positions, rank, window, 0.09, kernel="general").double().cpu(), 1.5e-2)


@pytest.mark.parametrize("window", [0, 48])
def test_one_key_that_matters_far_away_at_page_borders_and_window_edges(dev, window):
    """Key j* carries all the weight when visible (its row is aligned with the query and scaled up) and a value unlike
    any other, so an output either IS that value or has nothing of it."""
    rank, rot, S, page = 64, 8, 700, 64
    g = torch.Generator().manual_seed(5)
    direction = torch.randn(rank + rot, generator=g)
    direction /= direction.norm()
    for star in (0, 31, 32, 63, 64, 127, 128, 350, 651, 652, 653, 698, 699):
        rows = 0.05 * torch.randn(S, rank + rot, generator=g)
        rows[star] = 30.0 * direction
        # with a window: the key itself, the last query that still sees it, the first that does not, the newest
        wanted = [star, star + window - 1, star + window, S - 1] if window else [star, (star + S) // 2, S - 1]
        positions = torch.unique(torch.tensor([min(S - 1, p) for p in wanted]))
        q = (30.0 * direction).repeat(len(positions), 2, 1)
        want = O.cache_attention(q.double(), rows.double(), positions, rank, window, 1.0)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):  # the general kernel, then the tensor-core one
            got = run_attention(dev, dtype, q, rows, positions, rank, window, 1.0, page).float().cpu()
            close(got, want, tol)
            for r, p in enumerate(positions.tolist()):
                sees = star <= p and (not window or p - star < window)
                share = float(got[r, 0] @ rows[star, :rank] / rows[star, :rank].pow(2).sum())
                assert (share > 0.98) if sees else (abs(share) < 0.02), (star, p, share, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_latent_append_norms_rotates_and_lands_on_the_right_slot(dev, dtype, interleaved):
    rank, rot, page = 40, 12, 32
    g = torch.Generator().manual_seed(11)
    down = torch.randn(6, rank + rot, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(rank, generator=g)).to(dtype)
    pos = torch.tensor([30, 31, 32, 33, 0, 95], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 0, 1, 1], dtype=torch.int32)
    table = torch.tensor([[3, 1, -1], [0, 4, 2]], dtype=torch.int32)
    slab = torch.zeros((5, page, rank + rot), dtype=dtype, device=dev)
    blocks.latent_append(down.to(dev), w.to(dev), 1e-5, rank=rank, rot_dims=8, interleaved=interleaved, base=777.0,
                         tok_pos=pos.to(dev), tok_seq=seq.to(dev), block_table=table.to(dev), slab=slab)
    c = O.norm_plain(down[:, :rank].double(), w.double(), 1e-5)
    kr = O.rotate(down[:, rank:].double(), pos, 8, 777.0, interleaved)  # 8 of the 12 rotated, 4 pass
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    written = 0
    for t in range(6):
        p = int(table[seq[t], pos[t] // page])
        row = slab[p, pos[t] % page].cpu()
        close(row[:rank], c[t], tol)
        close(row[rank:], kr[t], tol)
        written += 1
    assert int((slab.float().abs().sum(-1) > 0).sum()) == written  # nothing else was touched


@pytest.mark.parametrize("interleaved", [False, True])
def test_fused_prepare_rotates_the_queries_and_fills_the_cache_in_one_launch(dev, interleaved):
    heads, dn, dr, rank, page = 3, 10, 8, 24, 32
    g = torch.Generator().manual_seed(13)
    qd = torch.randn(5, heads * (dn + dr) + rank + dr, generator=g)
    w = 1 + 0.1 * torch.randn(rank, generator=g)
    pos = torch.tensor([31, 32, 33, 7, 8], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32)
    table = torch.tensor([[2, 0], [1, -1]], dtype=torch.int32)
    slab = torch.zeros((3, page, rank + dr), device=dev)
    got = qd.to(dev).clone()
    blocks.latent_prepare(got, w.to(dev), 1e-5, heads=heads, dim=dn, rot_dim=dr, rank=rank, rot_dims=dr, interleaved=interleaved, base=3000.0,
                          tok_pos=pos.to(dev), tok_seq=seq.to(dev), block_table=table.to(dev), slab=slab)
    q_width = heads * (dn + dr)
    want_q = qd[:, :q_width].double().reshape(5, heads, dn + dr).clone()
    want_q[..., dn:] = O.rotate(want_q[..., dn:], pos, dr, 3000.0, interleaved)
    close(got[:, :q_width].reshape(5, heads, dn + dr), want_q, 2e-6)
    assert torch.equal(got[:, q_width:].cpu(), qd[:, q_width:])  # the latent's columns are read, not written
    c = O.norm_plain(qd[:, q_width : q_width + rank].double(), w.double(), 1e-5)
    kr = O.rotate(qd[:, q_width + rank :].double(), pos, dr, 3000.0, interleaved)
    for t in range(5):
        row = slab[int(table[seq[t], pos[t] // page]), pos[t] % page].cpu()
        close(row[:rank], c[t], 2e-6)
        close(row[rank:], kr[t], 2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,shared,T", [(6, 2, True, 37), (5, 1, False, 37), (4, 4, True, 37), (40, 3, False, 37), (3, 2, True, 150)])
def test_router_and_experts_against_the_loop_over_tokens(dev, dtype, experts, top, shared, T):
    # (the last case gives every expert about 100 rows: the bf16 path then takes 64-row tiles)
    D, ff = 72, 40
    g = torch.Generator().manual_seed(experts)
    w = {"router": torch.randn(experts, D, generator=g).to(dtype), "router.b": torch.randn(experts, generator=g).to(dtype)}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (torch.randn(ff, D, generator=g) / 8).to(dtype), (torch.randn(ff, D, generator=g) / 8).to(dtype), (torch.randn(D, ff, generator=g) / 6).to(dtype)
    h = torch.randn(T, D, generator=g).to(dtype)
    w64 = {k: v.double() for k, v in w.items()}
    want_idx, want_gate = O.route(h.double(), w64, "", top)
    idx, gate = blocks.moe_route(h.to(dev), w["router"].to(dev), w["router.b"].to(dev), top)
    assert torch.equal(idx.cpu().long(), want_idx)
    close(gate, want_gate, 1e-5)
    mlp = {"router": {"top": top}}
    shared_out = None
    if shared:
        shared_out = torch.randn(T, D, generator=g).to(dtype)
    want = O.mixture_ff(h.double(), w64, "", mlp) + (shared_out.double() if shared else 0)
    stack = lambda part: torch.stack([w[f"e{e}.{part}"] for e in range(experts)]).to(dev)
    got = blocks.moe_experts(h.to(dev), idx, gate, stack("gate"), stack("up"), stack("down"), blocks.ACT_SILU, None if not shared else shared_out.to(dev))
    close(got, want, 2e-6 if dtype == torch.float32 else 1e-2)


# ---------------------------------------------------------------------------------------------- the model
CONFIGS = {
    # several layer orders and sizes; the second makes values equal that usually differ (dim = rot_dim = vdim, one
    # head, top = 1), the third has sizes that are not multiples of anything convenient and a window of one page
    "mixed": dict(pattern="WCSMw", width=96, vocab=160, heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=40, window=24, experts=6, top=2),
    "equal": dict(pattern="cWSN", width=64, vocab=97, heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=32, window=5, experts=3, top=1, ff=64),
    # nothing is a multiple of 8: the general attention kernel and the FMA expert products serve bfloat16 too
    "awkward": dict(pattern="CwSWcM", width=100, vocab=301, heads=3, dim=20, rot_dim=6, vdim=12, kv_rank=37, window=7, experts=5, top=3,
                    expert_ff=20, shared_ff=28, ff=52),
    "odd": dict(pattern="wMCS", width=80, vocab=131, heads=5, dim=12, rot_dim=6, vdim=10, kv_rank=34, window=64, experts=7, top=7, expert_ff=24, shared_ff=0),
}
_models = {}


def model_and_oracle(dev, name, dtype, max_tokens=None):
    key = (name, dtype, max_tokens)
    if key not in _models:
        config = voluzen_config(**CONFIGS[name])
        tensors = synthetic_voluzen(config, seed=len(name))
        if dtype == torch.bfloat16:
            tensors = decisive_routers(tensors)
        model = model_class("Voluzen").from_checkpoint(config, tensors, dtype=dtype, device=dev, max_tokens=max_tokens)
        _models[key] = (model, config, tensors)
    return _models[key]


def run_schedule(model, prompts, schedule):
    """``schedule``: steps of [(request, count)]; every position's logits are collected.  Requests end (and give their
    pages back) with their last token."""
    caches, at, got = {}, {r: 0 for r in prompts}, {r: [] for r in prompts}
    for step in schedule:
        entries = []
        for r, n in step:
            caches.setdefault(r, model.create_kv_cache())
            entries.append(RaggedEntry(prompts[r][at[r] : at[r] + n], caches[r], want=range(n)))
        logits = model.forward_ragged(entries).cpu()
        k = 0
        for r, n in step:
            got[r].append(logits[k : k + n])
            k += n
            at[r] += n
            if at[r] == len(prompts[r]):
                caches.pop(r)[0].release()
    return {r: torch.cat(v) for r, v in got.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_the_plain_model(dev, name, dtype):
    model, config, tensors = model_and_oracle(dev, name, dtype)
    prompt = ids_for(150, config["vocab"], 1)
    want = O.forward(config, tensors, prompt)
    got = run_schedule(model, {"a": prompt}, [[("a", len(prompt))]])["a"]
    assert rows_match(got, want, dtype)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_layers_one_by_one(dev, name):
    """The residual stream after every layer (float32 mode), read by running the model's own layers in order."""
    model, config, tensors = model_and_oracle(dev, name, torch.float32)
    prompt = ids_for(70, config["vocab"], 2)
    _, want = O.forward(config, tensors, prompt, return_layers=True)
    from tiny_llm_b200.ragged import RaggedPlan

    cache = model.create_kv_cache()
    plan = RaggedPlan([RaggedEntry(prompt, cache)], dev, model.tile_sizes)
    x32, h = blocks.embed_rows(plan.ids, model.embed)
    for i, layer in enumerate(model.layers):
        h = layer.norm1(layer.mixer(h, plan, model.page_pool.slabs[layer.slab_index]), residual=x32)
        if layer.mlp is not None:
            h = layer.norm2(layer.mlp(h), residual=x32)
        close(x32, want[i], 2e-5)
    cache[0].release()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["mixed", "equal"])
def test_prefill_then_token_by_token_decoding_across_windows_and_pages(dev, name, dtype):
    model, config, tensors = model_and_oracle(dev, name, dtype)
    prompt = ids_for(190 + 120, config["vocab"], 3)  # 120 decoded tokens: the window and two page borders pass by
    want = O.forward(config, tensors, prompt)
    replays = model.graph_replays
    got = run_schedule(model, {"a": prompt}, [[("a", 190)]] + [[("a", 1)]] * 120)["a"]
    assert rows_match(got, want, dtype)
    # single-token steps replay a captured graph from their third step on, also across the step at which the block
    # table outgrows 4 pages (a second graph) - and give what eager steps give
    assert model.graph_replays - replays >= 110 and model.graph_captures >= 2
    model.use_decode_graph = False
    try:
        eager = run_schedule(model, {"a": prompt}, [[("a", 190)]] + [[("a", 1)]] * 120)["a"]
    finally:
        model.use_decode_graph = None
    # (bfloat16: the captured step may cut the key range over another number of CTAs than the eager one: rounding)
    assert row_error(eager, got.double()) < (1e-6 if dtype == torch.float32 else 5e-2)
    alone = run_schedule(model, {"a": prompt[:30]}, [[("a", 1)]] * 30)["a"]  # the first tokens, one by one from nothing
    assert rows_match(alone, want[:30], dtype)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size_down_to_two(dev, name):
    model, config, tensors = model_and_oracle(dev, name, torch.float32)
    prompt = ids_for(203, config["vocab"], 4)
    want = O.forward(config, tensors, prompt)
    for sizes in ([2] * 20 + [3, 5, 64, 23, 2, 33, 31, 2], [63, 1, 64, 2, 62, 11], [7] * 29, [128, 75]):
        assert sum(sizes) == len(prompt)
        got = run_schedule(model, {"a": prompt}, [[("a", n)] for n in sizes])["a"]
        assert row_error(got, want) < TOL[torch.float32], sizes


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_requests_in_one_batch_equal_each_alone_and_pages_are_reused(dev, dtype):
    model, config, tensors = model_and_oracle(dev, "mixed", dtype, max_tokens=5 * 64)  # 5 pages in all
    prompts = {"a": ids_for(130, 160, 5), "b": ids_for(61, 160, 6), "c": ids_for(3, 160, 7), "d": ids_for(100, 160, 8), "e": ids_for(64, 160, 9)}
    want = {r: O.forward(config, tensors, p) for r, p in prompts.items()}
    schedule = [[("a", 60), ("b", 2)], [("a", 2), ("b", 58), ("c", 1)], [("a", 1), ("b", 1), ("c", 2)],   # b and c end: 2 pages back
                [("a", 30), ("d", 50)], [("a", 37), ("d", 1)],                                           # a ends (3 pages), d in a reused page
                [("d", 49), ("e", 64)]]                                                                  # e fills a whole reused page
    got = run_schedule(model, prompts, schedule)
    pool = model.page_pool
    assert pool.reused_page_allocations >= 3 and pool.capacity == 5 and not pool.used_page_ids
    for r in prompts:
        assert rows_match(got[r], want[r], dtype), r
    if dtype == torch.float32:  # and the same as alone up to the summation order of the library products (which follows the row count)
        alone = run_schedule(model, {"d": prompts["d"]}, [[("d", 50)], [("d", 1)], [("d", 49)]])["d"]
        assert row_error(alone, got["d"].double()) < 2e-5
    with pytest.raises(RuntimeError, match="exhausted"):
        run_schedule(model, {"x": ids_for(330, 160, 1)}, [[("x", 330)]])
    assert not pool.used_page_ids  # the refused step took nothing


def test_rectangular_call_scheduler_slots_and_offsets(dev):
    model, config, tensors = model_and_oracle(dev, "mixed", torch.float32)
    p0, p1 = ids_for(9, 160, 10), ids_for(5, 160, 11)
    c0, c1 = model.create_kv_cache(), model.create_kv_cache()
    l0 = model(torch.tensor([p0], dtype=torch.int32, device=dev), 0, c0)                 # all rows
    l1 = model(torch.tensor([p1], dtype=torch.int32, device=dev), 0, c1, logits_to_keep=1)
    assert l0.shape == (1, 9, 160) and l1.shape == (1, 1, 160)
    assert row_error(l0[0], O.forward(config, tensors, p0)) < 2e-5
    with pytest.raises(ValueError, match="offset"):
        model(torch.tensor([[1]], dtype=torch.int32, device=dev), 3, c0)
    tables = [BatchingKvCache(max_active_requests=3) for _ in range(model.num_hidden_layers)]
    for t, a, b in zip(tables, c0, c1):
        t.add_request(a, 2)
        t.add_request(b, 0)
    out = model(torch.tensor([[7], [0], [8]], dtype=torch.int32, device=dev), [5, 0, 9], tables, logits_to_keep=1)
    assert out.shape == (3, 1, 160) and float(out[1].abs().max()) == 0.0               # the idle slot
    assert row_error(out[2, 0], O.forward(config, tensors, p0 + [8])[-1]) < 2e-5
    assert row_error(out[0, 0], O.forward(config, tensors, p1 + [7])[-1]) < 2e-5
    for t in tables:
        t.remove_request(0), t.remove_request(2)
    assert not model.page_pool.used_page_ids


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_entry_points(dev, dtype, tmp_path):
    """greedy_generate_ids and the continuous batcher (mixed steps, 2 slots, 5 requests, pages reused) produce the plain
    model's greedy tokens; the checkpoint goes through a directory and load_model."""
    config = voluzen_config(**CONFIGS["mixed"])
    tensors = synthetic_voluzen(config, seed=21)
    if dtype == torch.bfloat16:
        tensors = decisive_routers(tensors)
    save_voluzen(config, tensors, tmp_path / "ckpt")
    model = load_model(tmp_path / "ckpt", device=dev, dtype=dtype, max_tokens=6 * 64)
    prompts = [ids_for(n, 160, 30 + n) for n in (5, 70, 2, 33, 64)]
    new = 12

    def plain(prompt):  # greedy by full recomputation, in the model's arithmetic class (ties in bf16 are not tested)
        return O.greedy(config, tensors, prompt, new)

    want = [plain(p) for p in prompts]
    if dtype == torch.float32:
        assert greedy_generate_ids(model, prompts[1], new, device=dev) == want[1]
    batcher = ContinuousBatcher(model, None, prompts, max_seq_len=128, batch_size=2, prefill_step=16, verbose=False, device=dev,
                                max_new_tokens=[new] * len(prompts))
    results = dict(batcher.run())
    got = [[int(t) for t in results[i].split()] for i in range(len(prompts))]
    if dtype == torch.float32:
        assert got == want
    else:  # bf16: the same tokens until a near-tie, at least the first one and most of the rest
        agree = sum(g[:1] == w[:1] for g, w in zip(got, want))
        assert agree >= len(prompts) - 1
    assert batcher.mixed and batcher.mixed_steps > 0 and model.page_pool.reused_page_allocations > 0 and not model.page_pool.used_page_ids


def test_trace_program_replays_steps_and_writes_logits(dev, tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    config = voluzen_config(**CONFIGS["equal"])
    tensors = synthetic_voluzen(config, seed=4)
    save_voluzen(config, tensors, tmp_path / "ckpt")
    a, b = ids_for(70, 97, 1), ids_for(9, 97, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:], "want": [0, 3]}, {"id": "b", "tokens": b, "want": [8]}], "end": ["a", "b"]},
             {"step": 2, "entries": [{"id": "c", "tokens": b, "want": [0]}], "end": ["c"]}]
    root = Path(__file__).resolve().parent.parent
    run = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path / "ckpt"), "--dtype", "float32",
                          "--out", str(tmp_path / "out"), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (tmp_path / "out" / "0.f32").exists()
    got = torch.from_numpy(np.fromfile(tmp_path / "out" / "1.f32", dtype="<f4").reshape(3, 97))
    wa, wb = O.forward(config, tensors, a), O.forward(config, tensors, b)
    assert row_error(got, torch.stack([wa[66], wa[69], wb[8]])) < 2e-5
    got = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(1, 97))
    assert row_error(got, wb[:1]) < 2e-5


def test_command_line_generates_and_batches(dev, tmp_path, capsys):
    """The two front doors on a checkpoint directory of this design: `generate` prints the plain model's greedy tokens,
    `batch` serves three prompts through two slots."""
    from tiny_llm_b200 import cli

    config = voluzen_config(**CONFIGS["equal"])
    tensors = synthetic_voluzen(config, seed=8)
    save_voluzen(config, tensors, tmp_path / "ckpt")
    prompt = ids_for(11, 97, 5)
    want = O.greedy(config, tensors, prompt, 6)
    assert cli.main(["generate", "--model", str(tmp_path / "ckpt"), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                     "--max-new-tokens", "6"]) == 0
    assert [int(t) for t in capsys.readouterr().out.split()] == want
    assert cli.main(["batch", "--model", str(tmp_path / "ckpt"), "--dtype", "float32", "--quiet", "--batch-size", "2", "--prefill-step", "4",
                     "--max-new-tokens", "6", "--prompt-ids", ";".join(",".join(map(str, ids_for(n, 97, n))) for n in (11, 3, 7))]) == 0
    out = capsys.readouterr().out
    assert out.count("--- request") == 3
    first = out.split("--- request 0\n")[1].split("\n")[0]
    assert [int(t) for t in first.split()] == O.greedy(config, tensors, ids_for(11, 97, 11), 6)
    assert cli.main(["generate", "--synthetic", "voluzen:WCS", "--prompt-ids", "5,17,3", "--max-new-tokens", "4"]) == 0
    assert len(capsys.readouterr().out.split()) == 4
