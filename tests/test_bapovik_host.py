"""Host-side logic of the Bapovik path, on the CPU: recurrent-state slots beside the page pool, the per-sequence rows
of a ragged plan, the registry, the config generator and the checkpoint directory, and the plain restatement's own
mechanisms on cases whose answer is known in closed form."""

import json

import pytest
import torch

from oracle import bapovik as O
from tiny_llm_b200.latent_kv_cache import LatentPagedPool
from tiny_llm_b200.models import ARCHITECTURES, model_class
from tiny_llm_b200.ragged import RaggedEntry, RaggedPlan
from tiny_llm_b200.state_cache import HybridPagedCache, StateSlotPool
from tiny_llm_b200.synthetic import bapovik_config, save_bapovik, synthetic_bapovik


def pools(max_pages=None, max_slots=None, floats=10):
    return (LatentPagedPool([12], page_size=8, dtype=torch.float32, device="cpu", max_pages=max_pages),
            StateSlotPool(floats, device="cpu", max_slots=max_slots))


def test_state_slots_grow_keep_their_numbers_and_are_reused_newest_first():
    pool = StateSlotPool(6, device="cpu")
    slots = [pool.allocate() for _ in range(4)]
    assert slots == [0, 1, 2, 3] and pool.capacity == 4
    pool.storage[2, 5] = 3.5
    version = pool.version
    assert pool.allocate() == 4 and pool.capacity == 8 and pool.version != version and pool.storage[2, 5] == 3.5
    pool.free(1), pool.free(3)
    assert pool.allocate() == 3 and pool.allocate() == 1 and pool.reused_slot_allocations == 2
    with pytest.raises(ValueError, match="already free"):
        pool.free(7)
    view = pool.layer_view(2, (2, 2))
    assert tuple(view.shape) == (8, 2, 2) and view.stride(0) == 6 and view[2, 1, 1] == 3.5


def test_fixed_state_pool_refuses_and_a_request_holds_one_slot_from_its_first_tokens_to_its_release():
    pages, states = pools(max_pages=4, max_slots=2)
    a, b, c = (HybridPagedCache(pages, states) for _ in range(3))
    assert a.state_slot == -1 and not states.used_slots  # nothing is held before the first tokens
    a.append_slots(3), b.append_slots(9)
    assert (a.state_slot, b.state_slot) == (0, 1)
    with pytest.raises(RuntimeError, match="state slots exhausted"):
        c.append_slots(1)
    assert c.offset == 0 and c.state_slot == -1 and len(pages.used_page_ids) == 3
    a.append_slots(2)
    assert a.state_slot == 0 and a.offset == 5
    a.release()
    assert a.state_slot == -1 and states.free_slots == [0]
    c.append_slots(1)
    assert c.state_slot == 0 and states.reused_slot_allocations == 1
    with pytest.raises(RuntimeError, match="exhausted"):
        c.append_slots(40)  # no pages: the slot it already holds stays, nothing else changes
    assert c.state_slot == 0 and c.offset == 1
    d = HybridPagedCache(pages, states)
    b.release()
    with pytest.raises(RuntimeError, match="exhausted"):
        d.append_slots(40)  # no pages for a new request: the slot it took for this append goes back
    assert d.state_slot == -1 and states.used_slots == {0}


def test_what_a_step_has_consumed_cannot_be_rewound_from_a_state():
    pages, states = pools()
    a = HybridPagedCache(pages, states)
    plan = RaggedPlan([RaggedEntry([1, 2, 3, 4, 5], [a])], "cpu", 4)
    assert a.ran_offset == 5 and plan.seq_info.tolist() == [[0, 5, 0, 0]]
    a.append_slots(3)     # a later step's tokens, not run yet
    a.rewind(3)           # ... can be given back
    assert a.offset == 5
    with pytest.raises(NotImplementedError):
        a.rewind(2)
    a.rewind(5)           # everything: the request starts over
    assert a.offset == 0 and a.state_slot == -1 and not states.used_slots
    stateless = HybridPagedCache(pages, StateSlotPool(0, device="cpu"))
    stateless.append_slots(9)
    assert stateless.state_slot == -1
    stateless.rewind(4)
    assert stateless.offset == 5


def test_plan_rows_name_each_sequence_its_start_and_its_slot():
    pages, states = pools()
    a, b = HybridPagedCache(pages, states), HybridPagedCache(pages, states)
    RaggedPlan([RaggedEntry([7] * 11, [a])], "cpu", [2, 4])
    plan = RaggedPlan([RaggedEntry([1, 2, 3], [b]), RaggedEntry([9], [a], want=[])], "cpu", [2, 4])
    assert plan.seq_info.tolist() == [[0, 3, 0, 1], [3, 1, 11, 0]]
    assert plan.tok_pos.tolist() == [0, 1, 2, 11] and plan.tok_seq.tolist() == [0, 0, 0, 1]
    assert plan.tiles_for(2).tolist() == [[0, 2, 0], [2, 1, 0], [3, 1, 1]] and plan.tiles_for(4).tolist() == [[0, 3, 0], [3, 1, 1]]
    assert plan.total_ints == RaggedPlan.block_ints(4, 1, 2, plan.max_pages, 5)
    with pytest.raises(RuntimeError):  # all-or-nothing also with slots: the second entry's failure gives the first one's slot back
        fixed_pages, fixed_states = pools(max_slots=1)
        RaggedPlan([RaggedEntry([1], [HybridPagedCache(fixed_pages, fixed_states)]), RaggedEntry([1], [HybridPagedCache(fixed_pages, fixed_states)])], "cpu", 4)
    assert not fixed_states.used_slots and not fixed_pages.used_page_ids


def test_registry_config_generator_and_checkpoint_directory(tmp_path):
    assert "Bapovik" in ARCHITECTURES
    config = bapovik_config(pattern="APSp", heads=6, kv_heads=3, top=1)
    assert [l["type"] for l in config["layers"]] == ["attention", "parallel", "attention", "parallel"]
    assert config["layers"][2]["mixer"]["kv_from"] == 0 and config["layers"][3]["mlp"] is None
    with pytest.raises(ValueError, match="before it"):
        bapovik_config(pattern="SA")
    tensors = synthetic_bapovik(config, seed=1)
    assert "l2.mix.k" not in tensors and "l2.mix.q" in tensors and tuple(tensors["l1.mix.left.k.norm"].shape) == (16,)
    assert tuple(tensors["l1.mix.right.a2"].shape)[0] == 2 * 16 and "l3.mlp.router" not in tensors
    save_bapovik(config, tensors, tmp_path / "ckpt")
    assert json.loads((tmp_path / "ckpt" / "config.json").read_text())["architecture"] == "Bapovik"
    from tiny_llm_b200.checkpoint import read_tensors

    back = read_tensors(tmp_path / "ckpt")
    assert set(back) == set(tensors) and torch.equal(back["l0.mix.q.b"], tensors["l0.mix.q.b"])
    with pytest.raises(ValueError, match="not supported"):
        model_class("Bapovik2")


def test_plain_masks_and_the_sink():
    assert [j for j in range(12) if O.visible(9, j, "window", 4)] == [6, 7, 8, 9]
    assert [j for j in range(12) if O.visible(9, j, "chunk", 4)] == [8, 9]
    assert [j for j in range(12) if O.visible(8, j, "chunk", 4)] == [8]
    assert [j for j in range(5) if O.visible(3, j, "window", 1)] == [3]
    q, k, v = torch.zeros(3, 1, 2, dtype=torch.float64), torch.zeros(3, 1, 2, dtype=torch.float64), torch.tensor([[[1.0]], [[2.0]], [[6.0]]], dtype=torch.float64)
    plain = O.masked_attention(q, k, v, scale=1.0, kind="causal", size=0)
    sunk = O.masked_attention(q, k, v, scale=1.0, kind="causal", size=0, sink=True)
    assert torch.allclose(plain[:, 0, 0], torch.tensor([1.0, 1.5, 3.0], dtype=torch.float64))
    assert torch.allclose(sunk[:, 0, 0], torch.tensor([0.5, 1.0, 2.25], dtype=torch.float64))  # sums over 1 + n equal terms


def test_plain_recurrence_has_the_closed_form_of_a_constant_decay():
    T = 6
    q = k = torch.ones(T, 1, 1, dtype=torch.float64)
    v = torch.arange(1.0, T + 1, dtype=torch.float64).view(T, 1, 1)
    out = O.decayed_linear_attention(q, k, v, torch.full((T, 1, 1), 0.5, dtype=torch.float64))
    want = [sum(0.5 ** (t - s) * (s + 1) for s in range(t + 1)) for t in range(T)]
    assert torch.allclose(out.view(-1), torch.tensor(want, dtype=torch.float64))


def test_plain_experts_weight_the_input_and_take_the_largest_scores():
    spec = {"router": {"experts": 3, "top": 2}, "expert": {"ff": 1}}
    w = {"m.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0]], dtype=torch.float64)}
    for e in range(3):
        w[f"m.e{e}.up"] = torch.tensor([[1.0, 1.0]], dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.tensor([[float(e + 1)], [0.0]], dtype=torch.float64)
    h = torch.tensor([[2.0, 1.0]], dtype=torch.float64)   # scores sigmoid(2), sigmoid(1), sigmoid(-2): experts 0 and 1
    s0, s1 = torch.sigmoid(torch.tensor(2.0, dtype=torch.float64)), torch.sigmoid(torch.tensor(1.0, dtype=torch.float64))
    want = 1.0 * (3 * s0) ** 2 + 2.0 * (3 * s1) ** 2         # relu(up . (s h))^2 = (3 s)^2, the score enters squared
    assert torch.allclose(O.expert_mixture(h, w, "m.", spec)[0, 0], want)
