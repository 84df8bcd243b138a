"""Host-side logic of the Voluzen path, on the CPU: the multi-slab page pool, ragged plans, the model registry and
the scheduler's mixed steps (driven by a fake model whose "logits" encode what it was asked to run)."""

import json

import pytest
import torch

from tiny_llm_b200.batch import ContinuousBatcher
from tiny_llm_b200.latent_kv_cache import LatentCacheView, LatentPagedCache, LatentPagedPool
from tiny_llm_b200.models import ARCHITECTURES, model_class
from tiny_llm_b200.ragged import RaggedEntry, RaggedPlan
from tiny_llm_b200.synthetic import save_voluzen, synthetic_voluzen, voluzen_config


def make_pool(**kw):
    return LatentPagedPool([12, 20], page_size=kw.pop("page_size", 8), dtype=torch.float32, device="cpu", **kw)


def test_pool_has_one_slab_per_caching_layer_and_grows():
    pool = make_pool()
    a = LatentPagedCache(pool)
    a.append_slots(19)  # 3 pages of 8
    assert a.page_ids == [0, 1, 2] and a.page_lens == [8, 8, 3] and a.offset == 19
    assert [tuple(s.shape) for s in pool.slabs] == [(4, 8, 12), (4, 8, 20)]
    pool.slabs[0][2, 1, 5] = 7.0
    a.append_slots(30)  # outgrows 4 pages: the slabs move, the rows stay
    assert pool.capacity >= 7 and pool.storage_growths == 2 and pool.slabs[0][2, 1, 5] == 7.0
    assert pool.storage_nbytes == sum(s.numel() * 4 for s in pool.slabs)


def test_fixed_pool_refuses_then_reuses_freed_pages():
    pool = make_pool(max_pages=4)
    a, b = LatentPagedCache(pool), LatentPagedCache(pool)
    a.append_slots(17)
    with pytest.raises(RuntimeError, match="exhausted"):
        b.append_slots(9)
    assert b.page_ids == [] and b.offset == 0 and pool.num_free_pages == 0 and len(pool.used_page_ids) == 3
    b.append_slots(8)
    a.release()
    c = LatentPagedCache(pool)
    c.append_slots(20)
    assert sorted(c.page_ids) == [0, 1, 2] and pool.reused_page_allocations == 3 and pool.storage_growths == 1


def test_views_share_the_owner_and_release_nothing():
    pool = make_pool()
    owner = LatentPagedCache(pool)
    view = LatentCacheView(owner, 1)
    owner.append_slots(5)
    assert view.offset == 5 and view.page_ids is owner.page_ids and view.slab_index == 1
    view.release()
    assert owner.offset == 5
    owner.release()
    assert view.offset == 0 and pool.num_free_pages == 1


def test_plan_lays_out_positions_tiles_wants_and_tables():
    pool = make_pool()
    a, b = LatentPagedCache(pool), LatentPagedCache(pool)
    a.append_slots(6)
    plan = RaggedPlan([RaggedEntry([1, 2, 3, 4, 5], [a], want=[0, 4]), RaggedEntry([9], [b])], "cpu", tile=4)
    assert plan.ids.tolist() == [1, 2, 3, 4, 5, 9]
    assert plan.tok_pos.tolist() == [6, 7, 8, 9, 10, 0]
    assert plan.tok_seq.tolist() == [0, 0, 0, 0, 0, 1]
    assert plan.want_rows.tolist() == [0, 4, 5]
    assert plan.tiles.tolist() == [[0, 4, 0], [4, 1, 0], [5, 1, 1]]
    assert plan.block_table.tolist() == [[0, 1], [2, -1]]  # entries take their new pages in entry order
    assert a.offset == 11 and b.offset == 1


def test_plan_is_all_or_nothing_and_rejects_duplicates():
    pool = make_pool(max_pages=2)
    a, b = LatentPagedCache(pool), LatentPagedCache(pool)
    with pytest.raises(RuntimeError):
        RaggedPlan([RaggedEntry([1] * 8, [a]), RaggedEntry([2] * 9, [b])], "cpu", tile=4)
    assert a.offset == 0 and b.offset == 0 and not pool.used_page_ids
    with pytest.raises(ValueError, match="once"):
        RaggedPlan([RaggedEntry([1], [a]), RaggedEntry([2], [LatentCacheView(a, 0)])], "cpu", tile=4)
    with pytest.raises(ValueError, match="outside"):
        RaggedPlan([RaggedEntry([1, 2], [a], want=[2])], "cpu", tile=4)


def test_registry_and_config_generator(tmp_path):
    assert "Voluzen" in ARCHITECTURES and model_class("Voluzen").architecture == "Voluzen"
    with pytest.raises(ValueError):
        model_class("nope")
    config = voluzen_config(pattern="WCSMNwc")
    kinds = [(l["type"], (l["mlp"] or {}).get("kind"), l["mixer"].get("kv_from")) for l in config["layers"]]
    assert kinds == [("latent_attention_2", "dense", None), ("latent_attention", "moe", None), ("latent_attention", "moe", 1),
                     ("latent_attention", "moe", None), ("latent_attention", None, None), ("latent_attention_2", "moe", None),
                     ("latent_attention", "dense", None)]
    assert "shared" not in config["layers"][3]["mlp"] and "shared" in config["layers"][1]["mlp"]
    tensors = synthetic_voluzen(config, seed=1)
    assert "l2.mix.dkv" not in tensors and "l1.mix.dkv" in tensors and "l4.norm2" not in tensors
    save_voluzen(config, tensors, tmp_path / "m")
    assert json.loads((tmp_path / "m" / "config.json").read_text())["architecture"] == "Voluzen"
    from tiny_llm_b200.checkpoint import read_tensors

    back = read_tensors(tmp_path / "m")
    assert set(back) == set(tensors) and torch.equal(back["head"], tensors["head"])


class FakeRaggedModel:
    """Next token = (last token of the entry + 1) % vocab; records every step's entry lengths."""

    num_hidden_layers = 2
    vocab = 50

    def __init__(self):
        self.pool = LatentPagedPool([4], page_size=4, dtype=torch.float32, device="cpu")
        self.steps = []

    def create_kv_cache(self):
        owner = LatentPagedCache(self.pool)
        return [owner, LatentCacheView(owner, 0)]

    def forward_ragged(self, entries):
        self.steps.append([len(e.tokens) for e in entries])
        plan = RaggedPlan(entries, "cpu", tile=4)
        out = torch.zeros((len(entries), self.vocab))
        for row, e in enumerate(entries):
            out[row, (e.tokens[-1] + 1) % self.vocab] = 1.0
        assert plan.num_want == len(entries)
        return out


def test_mixed_steps_put_a_prompt_portion_beside_decoding_slots():
    model = FakeRaggedModel()
    prompts = [[1, 2, 3, 4, 5, 6, 7], [10, 11], [20, 21, 22]]
    batcher = ContinuousBatcher(model, None, prompts, max_seq_len=64, batch_size=2, prefill_step=3, verbose=False,
                                max_new_tokens=[4, 3, 2])
    assert batcher.mixed
    results = dict(batcher.run())
    assert results == {0: "8 9 10 11", 1: "12 13 14", 2: "23 24"}
    assert any(len(step) > 1 and step[0] > 1 for step in model.steps), model.steps  # a portion rode with decode tokens
    assert [3, 3, 1] == [s[0] for s in model.steps[:3]]                              # prompt 0 in portions of 3, 3, 1
    assert not model.pool.used_page_ids  # every request gave its pages back


def test_unmixed_scheduler_still_rejects_a_model_without_ragged_step():
    class Plain:
        num_hidden_layers = 1

    with pytest.raises(ValueError):
        ContinuousBatcher(Plain(), None, [[1]], mixed=True, verbose=False)
    assert not ContinuousBatcher(Plain(), None, [[1]], verbose=False).mixed
