"""The Ronelorn configuration without a GPU: reading and refusing config.json, the parts and the schedule it
builds, tensor shapes, what the cache is asked for, the cache's bookkeeping of kept pages and of rows per run,
and the plain statement's own masks."""
import copy

import pytest
import torch

import plain_ronelorn as pr
import tiny_ronelorn as tr
from supersonic_b200.config import ConfigError, config_from_dict, load_config


def test_reads_every_key_and_round_trips(tmp_path):
    cfg = config_from_dict(tr.A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale, cfg.residual_mult) == (101, 48, 1e-5, 3.0, 0.4)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.architectures == ["Ronelorn"] and cfg.num_hidden_layers == 5
    from supersonic_b200.weights import write_model_folder
    folder = write_model_folder(cfg, 1, str(tmp_path / "m"), std=0.1)
    assert load_config(folder).to_dict() == cfg.to_dict()


def test_layers_that_run_with_another_layers_tensors():
    cfg = config_from_dict(tr.A)
    spec = cfg.build_spec()
    assert [b.mixer.kind for b in spec.blocks] == ["window_attention", "min_gru", "window_attention", "min_gru"]
    assert [(s.layer, s.cache) for s in spec.schedule] == [(0, 0), (1, 1), (2, 2), (0, 3), (3, 4)]
    shapes = cfg.tensor_shapes()
    assert not any(n.startswith("l3.") for n in shapes) and "l4.mix.z.b" in shapes
    assert shapes["l0.mix.q.norm"] == [16] and shapes["l2.mix.q.norm"] == [72] and shapes["l2.mix.k.norm"] == [36]
    assert shapes["l0.mix.v"] == [2 * 24, 48] and shapes["l0.mix.o"] == [48, 4 * 24]
    assert "l1.norm2" not in shapes and shapes["l4.mlp.up"] == [24, 48] and shapes["l4.mix.o"] == [48, 20]


def test_parts_and_their_parameters():
    spec = config_from_dict(tr.A).build_spec()
    assert spec.embedding.params["scale"] == 3.0
    b0, b2 = spec.blocks[0], spec.blocks[2]
    p = b0.mixer.params
    assert (p["window"], p["pool"], p["keep_first"], p["softcap"], p["sink"], p["qk_norm"]) == (20, 4, 0, 12.0, False, "head")
    assert p["value_rotation"] == {"theta": 1000.0, "pairing": "halves"} and p["out_scale"] == 0.4
    assert b0.position.params["scaling"] == {"kind": "linear", "factor": 4.0} and b0.position.params["rotary_dim"] == 8
    assert b0.mixer_norm.params["unit_offset"] and b0.feed_forward.params["activation"] == "relu_squared"
    p = b2.mixer.params
    assert (p["window"], p["pool"], p["keep_first"], p["softcap"], p["sink"], p["qk_norm"]) == (17, 0, 3, None, True, "row")
    assert p["value_rotation"] is None and b2.position.params["scaling"] is None
    assert spec.blocks[1].feed_forward is None and spec.blocks[1].feed_forward_norm is None
    # no cap, no scaling, factors of one: the keys may be absent
    spec_b = config_from_dict(tr.B).build_spec()
    assert spec_b.blocks[1].mixer.params["softcap"] is None and "scale" not in spec_b.embedding.params


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].__setitem__("type", "attention_3"), "not known"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda d: d["layers"][0]["mixer"]["mask"].pop("size"), "missing"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("vdim", 23), "even"),
    (lambda d: d["layers"][3].__setitem__("weights_of", 3), "another layer"),
    (lambda d: d["layers"][3].__setitem__("weights_of", 2), "differs"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "moe"), "not known"),
    (lambda d: d.pop("norm"), "missing"),
])
def test_refuses_what_it_cannot_run(change, message):
    d = copy.deepcopy(tr.A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_what_the_cache_is_asked_for():
    from supersonic_b200.cache import KvNeed, StateNeed
    from supersonic_b200.parts import MIXERS
    spec = config_from_dict(tr.B).build_spec()
    kept = MIXERS["window_attention"].cache_need_from(spec.blocks[0].mixer.params)
    assert kept == KvNeed(3, 16, 9, value_dim=16, keep_first=70)
    pooled = MIXERS["window_attention"].cache_need_from(spec.blocks[1].mixer.params)
    assert pooled == {"tokens": KvNeed(1, 24, 64, value_dim=10), "pooled": KvNeed(1, 24, None, value_dim=10, tokens_per_row=3)}
    assert MIXERS["min_gru"].cache_need_from(spec.blocks[2].mixer.params) == StateNeed(64)
    # runs longer than the window: the run's tokens stay until its last one has come
    long_runs = MIXERS["window_attention"].cache_need_from(config_from_dict(tr.C).build_spec().blocks[3].mixer.params)
    assert long_runs["tokens"].window == 9 and long_runs["pooled"].tokens_per_row == 9


def test_cache_keeps_first_pages_and_counts_a_row_per_run():
    """A window store gives pages back behind the window, never those of the kept first tokens; a store of one row
    per run of P tokens holds a page per 64 runs."""
    from supersonic_b200.cache import KvNeed, SequenceCache
    needs = {0: KvNeed(1, 8, 9, keep_first=70), 1: {"tokens": KvNeed(1, 8, 64), "pooled": KvNeed(1, 8, None, tokens_per_row=3)}}
    cache = SequenceCache(needs, 4096, 2048, torch.float32, "cpu")
    slot = cache.acquire()
    by_need = {g.need: g for g in cache.kv_groups}
    kept, tokens, pooled = by_need[needs[0]], by_need[needs[1]["tokens"]], by_need[needs[1]["pooled"]]
    for n in [700] + [1] * 100:
        cache.reserve(slot, n)
        cache.advance(slot, n)
    assert cache.length(slot) == 800
    assert set(kept.held[slot]) == {0, 1, 12} and set(tokens.held[slot]) == {11, 12}
    assert set(pooled.held[slot]) == set(range((800 // 3 + 63) // 64))
    cache.check()
    cache.release(slot)
    assert all(g.pool.n_held == 0 for g in cache.kv_groups)
    again = cache.acquire()
    cache.reserve(again, 5)
    cache.advance(again, 5)
    assert set(kept.held[again]) == {0} and set(pooled.held[again]) <= {0}
    cache.check()


def test_the_plain_statements_masks():
    assert pr.tokens_seen(10, 4, 0) == [7, 8, 9, 10] and pr.tokens_seen(10, 4, 2) == [0, 1, 7, 8, 9, 10]
    assert pr.tokens_seen(2, 4, 2) == [0, 1, 2] and pr.tokens_seen(4, 4, 3) == [0, 1, 2, 3, 4]
    # runs of 3 before a window of 4: run 0 (tokens 0..2) is seen from position 6 on, run 1 from 9 on
    assert pr.runs_seen(5, 4, 3) == [] and pr.runs_seen(6, 4, 3) == [0] and pr.runs_seen(8, 4, 3) == [0]
    assert pr.runs_seen(9, 4, 3) == [0, 1] and pr.runs_seen(100, 4, 0) == []


def test_a_cache_of_recurrent_state_alone():
    """A model of recurrent layers only has no key store at all."""
    from supersonic_b200.cache import SequenceCache, StateNeed
    cache = SequenceCache({0: StateNeed(4), 1: StateNeed(7)}, 256, 256, torch.float32, "cpu")
    slot = cache.acquire()
    cache.reserve(slot, 5)
    cache.advance(slot, 5)
    assert cache.length(slot) == 5 and cache.state(1).shape[1] == 7
    cache.check()
    cache.release(slot)
