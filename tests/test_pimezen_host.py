"""Host-side pieces of the Pimezen design: its configuration and registry entry, the tensors it
declares, the cache groups its layers form, and the cache manager's handling of windows that keep
the first tokens of a sequence."""

from __future__ import annotations

import copy
import json
import random

import pytest
import torch

from mini_engine_b200.cache import NULL_PAGE, CacheManager, GroupSpec
from mini_engine_b200.cache.storage import pages_of_group, plan_groups
from mini_engine_b200.config import PimezenConfig, load_model_config
from mini_engine_b200.config.qwen3 import ConfigError
from mini_engine_b200.parts.base import PagedCacheSpec
from mini_engine_b200.parts.model import DecoderModel, declared_weights
from mini_engine_b200.weights import WeightError, write_random_model
from mini_engine_b200.weights.loader import WeightSpec, check_specs


def raw_config(layers=2, mlp_in_last=True):
    def one(i):
        return {
            "type": "parallel",
            "mixer": {
                "left": {"heads": 4, "kv_heads": 2, "dim": 16 + 8 * i, "vdim": 8, "scale": 0.3,
                         "mask": {"size": 12 + i, "keep_first": 3}},
                "right": {"heads": 2, "dim": 8, "vdim": 24, "tau": 4.0, "decay_rank": 4 + i},
                "left_scale": 0.6, "right_scale": 1.3,
            },
            "mlp": {"kind": "dense", "ff": 56, "limit": 1.5} if (mlp_in_last or i < layers - 1) else None,
        }  # fmt: skip

    return {"architecture": "Pimezen", "vocab": 96, "width": 40, "norm": {"eps": 3e-5}, "layers": [one(i) for i in range(layers)]}


def test_config_round_trip_and_registry(tmp_path):
    cfg = PimezenConfig.from_dict(raw_config())
    assert PimezenConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.layers[1].left.dim == 24 and cfg.layers[1].left.window == 13 and cfg.layers[0].right.decay_rank == 4
    write_random_model(tmp_path, cfg, seed=1)
    arch, loaded = load_model_config(tmp_path)
    assert arch.name == "Pimezen" and loaded == cfg


def test_the_decay_rank_comes_from_the_checkpoint_when_the_config_is_silent(tmp_path):
    cfg = PimezenConfig.from_dict(raw_config())
    write_random_model(tmp_path, cfg, seed=1)
    stored = json.loads((tmp_path / "config.json").read_text())
    for entry in stored["layers"]:
        del entry["mixer"]["right"]["decay_rank"]
    (tmp_path / "config.json").write_text(json.dumps(stored))
    assert PimezenConfig.from_folder(tmp_path) == cfg
    with pytest.raises(ConfigError, match="rank"):
        PimezenConfig.from_dict(stored)


@pytest.mark.parametrize(
    "path,value,message",
    [
        (("layers", 0, "type"), "serial", "type"),
        (("layers", 1, "mlp", "kind"), "routed", "kind"),
        (("layers", 0, "mixer", "left", "kv_heads"), 3, "multiple"),
        (("layers", 0, "mixer", "left", "mask", "size"), 0, "positive"),
        (("layers", 0, "mixer", "right", "tau"), 0.0, "positive"),
        (("norm", "eps"), None, "eps"),
        (("architecture",), "Other", "architecture"),
    ],
)
def test_config_errors_name_the_key(path, value, message):
    raw = copy.deepcopy(raw_config())
    node = raw
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        PimezenConfig.from_dict(raw)


def test_declared_tensors_and_a_layer_without_feed_forward():
    cfg = PimezenConfig.from_dict(raw_config(layers=2, mlp_in_last=False))
    from mini_engine_b200.models.pimezen import pimezen_spec

    specs = declared_weights(pimezen_spec(cfg))
    names = {s.name: s for s in specs}
    assert names["l0.mix.left.q"].shape == (64, 40) and names["l0.mix.left.v"].shape == (16, 40)
    assert names["l0.mix.left.o"].shape == (40, 32) and names["l0.mix.left.talk"].shape == (4, 4)
    assert names["l1.mix.right.a1"].shape == (5, 40) and names["l1.mix.right.a2"].shape == (16, 5)
    assert names["l0.mix.right.a2"].role == "vector" and names["l0.mix.left.r1"].role == "vector"
    assert "l0.mlp.gate" in names and "l1.mlp.gate" not in names and "l1.norm1" in names
    # a checkpoint may or may not carry the unused norm and scale of the layer without feed-forward
    assert names["l1.norm2"].optional and names["l1.ls2"].optional and not names["l0.norm2"].optional
    entries = {s.name: (torch.bfloat16, s.shape) for s in specs if s.alias_of is None and not s.optional}
    check_specs(specs, entries)
    check_specs(specs, {**entries, "l1.norm2": (torch.bfloat16, (40,)), "l1.ls2": (torch.bfloat16, (40,))})
    with pytest.raises(WeightError, match="l1.mlp.up"):
        check_specs(specs, {**entries, "l1.mlp.up": (torch.bfloat16, (56, 40))})
    head = [s for s in specs if s.alias_of is not None]
    assert len(head) == 1 and head[0].alias_of == "embed"


def test_layers_with_equal_needs_share_a_cache_group_and_others_do_not():
    raw = raw_config(layers=3)
    raw["layers"][2] = copy.deepcopy(raw["layers"][0])
    from mini_engine_b200.models.pimezen import pimezen_spec

    needs = DecoderModel(pimezen_spec(PimezenConfig.from_dict(raw))).cache_needs()
    specs, group_of = plan_groups(needs)
    assert group_of == [0, 1, 0] and specs[0] == PagedCacheSpec(2, 16, 12, 8, 3) and specs[1].head_dim == 24
    assert all(state.shape == (2, 8, 24) and state.dtype == torch.float32 for _paged, state, _of in needs)
    assert pages_of_group(specs[0], 1000, 4, 2, 8) == 2 * (-(-(12 + 8) // 4) + 2 + 1)


def test_pages_of_kept_first_tokens_are_never_given_back():
    manager = CacheManager([GroupSpec("w", window=6, keep_first=5), GroupSpec("full")], 32, 4, 4, False)
    req = manager.new_request()
    assert manager.try_allocate(req, 30)
    kept = list(req.block_tables[0][:2])
    released = manager.release_behind_window(req, 30)
    # tokens 0..4 live in pages 0 and 1 and stay; the next query (position 30) reads keys 25..: page 6 on
    assert released == 4 and req.block_tables[0][:2] == kept
    assert req.block_tables[0][2:6] == [NULL_PAGE] * 4 and NULL_PAGE not in req.block_tables[0][6:]
    assert NULL_PAGE not in req.block_tables[1]
    manager.check_invariants([req])
    assert manager.release_behind_window(req, 30) == 0
    manager.free(req)
    manager.check_invariants([])
    assert manager.pools[0].num_free == 32 and manager.pools[1].num_free == 32


def test_random_orders_with_kept_tokens_lose_no_page():
    rng = random.Random(4)
    manager = CacheManager([GroupSpec("w", window=9, keep_first=7, num_blocks=40)], 40, 4, 3, False)
    live: list = []
    for _ in range(400):
        action = rng.random()
        if action < 0.3 and len(live) < 3:
            req = manager.new_request()
            if manager.try_allocate(req, rng.randrange(1, 20)):
                live.append([req, 0])
        elif action < 0.8 and live:
            item = rng.choice(live)
            held = len(item[0].block_tables[0]) * 4
            item[1] = min(held, item[1] + rng.randrange(1, 9))
            manager.release_behind_window(item[0], item[1])
            manager.try_allocate(item[0], held + rng.randrange(0, 9))
            table = item[0].block_tables[0]
            assert NULL_PAGE not in table[:2] and NULL_PAGE not in table[max(0, item[1] - 8) // 4 :]
        elif live:
            manager.free(live.pop(rng.randrange(len(live)))[0])
        manager.check_invariants([item[0] for item in live])


def test_prefix_hits_need_the_kept_pages_too():
    manager = CacheManager([GroupSpec("w", window=4, keep_first=3)], 16, 4, 2, True)
    tokens = list(range(21))
    req = manager.new_request()
    assert manager.try_allocate(req, 21)
    manager.register_computed(req, tokens, 20)
    manager.release_behind_window(req, 20)
    manager.free(req)
    hit = manager.match_prefix(tokens)[0]
    assert len(hit) == 5 and hit[0] != NULL_PAGE and hit[1:4] == [NULL_PAGE] * 3 and hit[4] != NULL_PAGE
