"""Host-side pieces of the Molotar design: its configuration and registry entry, the tensors it declares,
the cache groups and state slots its layers ask for, and the stretched rotary frequencies."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_molotar as plain
from mini_engine_b200.cache.storage import plan_groups
from mini_engine_b200.config import MolotarConfig, load_model_config
from mini_engine_b200.config.qwen3 import ConfigError
from mini_engine_b200.parts.base import PagedCacheSpec
from mini_engine_b200.parts.model import DecoderModel, declared_weights
from mini_engine_b200.parts.rotary import RotaryEncoding
from mini_engine_b200.weights import write_random_model

ROUTED = {"kind": "moe", "expert": {"ff": 24, "limit": 2.0},
          "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}}  # fmt: skip


def attention(window=20, kv_from=None, heads=6, kv_heads=2, dim=16, vdim=24):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.2, "mask": {"size": window},
           "rot": {"dims": 8, "base": 500.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 64}}}  # fmt: skip
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def raw_config():
    return copy.deepcopy(_raw_config())


def _raw_config():
    return {
        "architecture": "Molotar", "vocab": 90, "width": 48, "norm": {"eps": 2e-5}, "postln_alpha": 2.5,
        "embedding": {"scale": 3.0, "bigram": {"buckets": 37, "mul_prev": 11, "mul_cur": 5}},
        "layers": [
            {"type": "rglru", "mixer": {"width": 32, "blocks": 2, "conv": 3}, "mlp": ROUTED},
            {"type": "attention", "mixer": attention(), "mlp": ROUTED},
            {"type": "attention", "mixer": attention(window=33, kv_from=1), "mlp": None},
            {"type": "attention", "mixer": attention(), "mlp": ROUTED},
        ],
    }  # fmt: skip


def test_config_round_trip_and_registry(tmp_path):
    cfg = MolotarConfig.from_dict(raw_config())
    assert MolotarConfig.from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == raw_config()
    assert cfg.layers[2].mixer.kv_from == 1 and cfg.layers[2].mlp is None and cfg.layers[0].mixer.conv == 3
    assert cfg.layers[1].mlp.group_keep == 2 and cfg.bigram_buckets == 37 and cfg.postln_alpha == 2.5
    write_random_model(tmp_path, cfg, seed=1)
    arch, loaded = load_model_config(tmp_path)
    assert arch.name == "Molotar" and loaded == cfg


@pytest.mark.parametrize(
    "path,value,message",
    [
        (("layers", 0, "type"), "conv", "not a mixer"),
        (("layers", 2, "mixer", "kv_from"), 0, "earlier attention layer"),
        (("layers", 2, "mixer", "kv_from"), 2, "earlier attention layer"),
        (("layers", 2, "mixer", "dim"), 32, "do not fit"),
        (("layers", 1, "mixer", "heads"), 5, "multiple of kv_heads"),
        (("layers", 1, "mixer", "rot", "dims"), 18, "rot.dims"),
        (("layers", 0, "mixer", "blocks"), 5, "blocks must divide"),
        (("layers", 0, "mlp", "router", "top"), 5, "exceeds"),
        (("layers", 0, "mlp", "kind"), "dense", "not a feed-forward"),
        (("embedding", "bigram", "buckets"), 0, "positive"),
        (("postln_alpha",), None, "lacks the key"),
    ],
)
def test_config_errors_name_the_key(path, value, message):
    raw = raw_config()
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        MolotarConfig.from_dict(raw)


def test_optional_keys_may_be_absent():
    raw = raw_config()
    del raw["layers"][1]["mixer"]["rot"]["scaling"], raw["layers"][3]["mixer"]["rot"], raw["layers"][3]["mixer"]["mask"]
    del raw["layers"][0]["mlp"]["router"]["groups"]
    cfg = MolotarConfig.from_dict(raw)
    assert cfg.layers[1].mixer.rot_scaling is None and cfg.layers[3].mixer.rot_dims == 0 and cfg.layers[3].mixer.window is None
    assert (cfg.layers[0].mlp.group_count, cfg.layers[0].mlp.group_keep) == (1, 1)


def test_declared_tensors():
    from mini_engine_b200.config.registry import architecture_for

    spec = architecture_for("Molotar").build_spec(MolotarConfig.from_dict(raw_config()))
    declared = {s.name: s for s in declared_weights(spec)}
    assert declared["bigram"].shape == (38, 48) and declared["embed"].shape == (90, 48) and declared["head"].shape == (90, 48)
    assert declared["l1.mix.q.norm"].shape == (96,) and declared["l1.mix.k.norm"].shape == (32,)  # over whole projections
    assert declared["l1.mix.g"].shape == (6, 48) and declared["l1.mix.v"].shape == (48, 48) and declared["l1.mix.o"].shape == (48, 144)
    # a layer that reads another layer's keys and values has none of their tensors
    assert "l2.mix.q" in declared and not any(name in declared for name in ("l2.mix.k", "l2.mix.v", "l2.mix.k.norm"))
    assert declared["l2.norm2"].optional and "l2.mlp.router" not in declared  # no feed-forward
    assert declared["l0.mix.ra"].shape == (2, 16, 16) and declared["l0.mix.conv"].shape == (32, 3) and declared["l0.mix.lam"].shape == (32,)
    assert declared["l0.mlp.e5.down"].shape == (48, 24) and declared["l0.mlp.router"].shape == (6, 48)
    assert declared["l0.mix.ra"].role == "vector" and declared["l0.mlp.router"].role == "vector"  # kept in 32-bit
    assert spec.order[2].cache_of == 1 and spec.order[3].cache_of is None


def test_cache_groups_state_slots_and_a_reader_with_a_wider_window():
    from mini_engine_b200.config.registry import architecture_for

    model = DecoderModel(architecture_for("Molotar").build_spec(MolotarConfig.from_dict(raw_config())))
    needs = model.cache_needs()
    assert needs[0][0] is None and needs[0][1].shape == (3, 32)  # the recurrence: state and the convolution's two inputs
    assert needs[1][0] == PagedCacheSpec(2, 16, 20, 24, 0) and needs[2][0].window == 33 and needs[2][2] == 1
    specs, group_of = plan_groups(needs)
    # layer 1 keeps its pages for the wider window of its reader; layer 3, with the same sizes, gives them back earlier
    assert group_of == [None, 0, 0, 1] and specs[0].window == 33 and specs[1].window == 20
    assert model.embedding_state().shape == (1,) and model.embedding_state().dtype == torch.int32
    no_window = copy.deepcopy(needs)
    no_window[2] = (PagedCacheSpec(2, 16, None, 24, 0), None, 1)
    assert plan_groups(no_window)[0][0].window is None
    wrong = copy.deepcopy(needs)
    wrong[2] = (PagedCacheSpec(2, 8, 33, 24, 0), None, 1)
    with pytest.raises(ValueError, match="reads a cache"):
        plan_groups(wrong)


@pytest.mark.parametrize("dims,base,scaling", [
    (8, 500.0, {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 64}),
    (32, 10000.0, {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 300}),
    (6, 50.0, None),
])  # fmt: skip
def test_stretched_rotary_frequencies(dims, base, scaling):
    part = RotaryEncoding("", 0, head_dim=dims + 4, theta=base, rotary_dim=dims, wavelength_scaling=scaling)
    want = plain.rotary_frequencies({"dims": dims, "base": base, "scaling": scaling})
    got = part.inv_freq().double().tolist()
    assert len(got) == dims // 2 and all(math.isclose(g, w, rel_tol=1e-6) for g, w in zip(got, want))
    if scaling:  # the three regimes are all there: kept, divided, blended
        plainly = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        kinds = {"kept" if math.isclose(w, p) else "divided" if math.isclose(w, p / scaling["factor"]) else "blended"
                 for w, p in zip(want, plainly)}  # fmt: skip
        assert kinds >= {"kept", "divided"}
