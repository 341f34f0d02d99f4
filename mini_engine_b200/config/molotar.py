"""Typed configuration of the Molotar decoder, read from its own ``config.json`` keys.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``postln_alpha`` (what the stream is
multiplied by in front of every sum), ``embedding`` (``scale`` and the ``bigram`` table's ``buckets``, ``mul_prev``,
``mul_cur``) and ``layers``: one entry per layer with its ``type`` (``attention`` or ``rglru``), the mixer's sizes
and constants under ``mixer`` and its feed-forward under ``mlp`` (``null``: the layer has none).  Layers may differ
from one another in every size.  An attention layer with ``kv_from: j`` has no keys and values of its own and reads
layer ``j``'s.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from mini_engine_b200.config.pimezen import _need
from mini_engine_b200.config.qwen3 import ConfigError

NUMBER = (int, float)


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    low: float
    high: float
    original: float

    def to_dict(self) -> dict[str, Any]:
        return {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None  # mask.size: position i sees j when 0 <= i - j < window
    rot_dims: int  # 0: no rotation
    rot_base: float
    rot_scaling: RotaryScaling | None
    kv_from: int | None = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "AttentionMixer":
        mask = raw.get("mask")
        window = None if mask is None else _need(mask, "size", int, where + "mask.")
        rot = raw.get("rot")
        dims, base, scaling = 0, 10000.0, None
        if rot is not None:
            dims = _need(rot, "dims", int, where + "rot.")
            base = float(_need(rot, "base", NUMBER, where + "rot."))
            if rot.get("scaling") is not None:
                sc, at = rot["scaling"], where + "rot.scaling."
                scaling = RotaryScaling(*(float(_need(sc, key, NUMBER, at)) for key in ("factor", "low", "high", "original")))
        kv_from = raw.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
            raise ConfigError(f"config.json key {where}'kv_from' must be a layer's number, got {kv_from!r}")
        out = cls(
            heads=_need(raw, "heads", int, where),
            kv_heads=_need(raw, "kv_heads", int, where),
            dim=_need(raw, "dim", int, where),
            vdim=_need(raw, "vdim", int, where),
            scale=float(_need(raw, "scale", NUMBER, where)),
            window=window,
            rot_dims=dims,
            rot_base=base,
            rot_scaling=scaling,
            kv_from=kv_from,
        )
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or (window is not None and window < 1):
            raise ConfigError(f"{where}: sizes must be positive")
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
        if dims % 2 or not 0 <= dims <= out.dim:
            raise ConfigError(f"{where}rot.dims must be even and at most dim, got {dims}")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
            if self.rot_scaling is not None:
                out["rot"]["scaling"] = self.rot_scaling.to_dict()
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class RecurrentMixer:
    width: int
    blocks: int
    conv: int  # taps of the causal convolution

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "RecurrentMixer":
        out = cls(_need(raw, "width", int, where), _need(raw, "blocks", int, where), _need(raw, "conv", int, where))
        if min(out.width, out.blocks, out.conv) < 1 or out.width % out.blocks:
            raise ConfigError(f"{where}: sizes must be positive and blocks must divide width")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class RoutedFeedForward:
    ff: int
    limit: float
    experts: int
    top: int
    group_count: int
    group_keep: int
    scale: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "RoutedFeedForward":
        if _need(raw, "kind", str, where) != "moe":
            raise ConfigError(f"{where}kind {raw['kind']!r} is not a feed-forward of this design (known: 'moe')")
        unit = _need(raw, "expert", Mapping, where)
        router = _need(raw, "router", Mapping, where)
        groups = router.get("groups")
        out = cls(
            ff=_need(unit, "ff", int, where + "expert."),
            limit=float(_need(unit, "limit", NUMBER, where + "expert.")),
            experts=_need(router, "experts", int, where + "router."),
            top=_need(router, "top", int, where + "router."),
            group_count=1 if groups is None else _need(groups, "count", int, where + "router.groups."),
            group_keep=1 if groups is None else _need(groups, "keep", int, where + "router.groups."),
            scale=float(_need(router, "scale", NUMBER, where + "router.")),
        )
        if min(out.ff, out.experts, out.top, out.group_count, out.group_keep) < 1 or not out.limit > 0:
            raise ConfigError(f"{where}: sizes and limit must be positive")
        if out.experts % out.group_count or out.group_keep > out.group_count:
            raise ConfigError(f"{where}router: {out.experts} experts do not form {out.group_count} equal groups of which {out.group_keep} are kept")
        if out.top > out.group_keep * (out.experts // out.group_count):
            raise ConfigError(f"{where}router.top ({out.top}) exceeds the experts of the kept groups")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {
            "kind": "moe",
            "expert": {"ff": self.ff, "limit": self.limit},
            "router": {"experts": self.experts, "top": self.top, "scale": self.scale,
                       "groups": {"count": self.group_count, "keep": self.group_keep}},
        }  # fmt: skip


@dataclass(frozen=True)
class MolotarLayer:
    type: str  # "attention" or "rglru"
    mixer: AttentionMixer | RecurrentMixer
    mlp: RoutedFeedForward | None

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class MolotarConfig:
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    embedding_scale: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple[MolotarLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Molotar"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MolotarConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"architecture must be {cls.architecture!r}, got {raw.get('architecture')!r}")
        norm = _need(raw, "norm", Mapping, "")
        embedding = _need(raw, "embedding", Mapping, "")
        bigram = _need(embedding, "bigram", Mapping, "embedding.")
        layers: list[MolotarLayer] = []
        for index, entry in enumerate(_need(raw, "layers", list, "")):
            where = f"layers[{index}]."
            kind = _need(entry, "type", str, where)
            mixer_raw = _need(entry, "mixer", Mapping, where)
            if kind == "attention":
                mixer: AttentionMixer | RecurrentMixer = AttentionMixer.from_dict(mixer_raw, where + "mixer.")
                source = mixer.kv_from
                if source is not None:
                    if not 0 <= source < index or layers[source].type != "attention" or layers[source].mixer.kv_from is not None:
                        raise ConfigError(f"{where}mixer.kv_from must name an earlier attention layer with keys and values of its own, got {source}")
                    owner = layers[source].mixer
                    if (owner.kv_heads, owner.dim, owner.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ConfigError(f"{where}mixer: the key and value heads of layer {source} do not fit this layer's")
            elif kind == "rglru":
                mixer = RecurrentMixer.from_dict(mixer_raw, where + "mixer.")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (known: 'attention', 'rglru')")
            mlp_raw = entry.get("mlp")
            mlp = None if mlp_raw is None else RoutedFeedForward.from_dict(mlp_raw, where + "mlp.")
            layers.append(MolotarLayer(kind, mixer, mlp))
        if not layers:
            raise ConfigError("config.json lists no layers")
        eos = raw.get("eos_token_id")
        out = cls(
            vocab=_need(raw, "vocab", int, ""),
            width=_need(raw, "width", int, ""),
            norm_eps=float(_need(norm, "eps", NUMBER, "norm.")),
            postln_alpha=float(_need(raw, "postln_alpha", NUMBER, "")),
            embedding_scale=float(_need(embedding, "scale", NUMBER, "embedding.")),
            bigram_buckets=_need(bigram, "buckets", int, "embedding.bigram."),
            bigram_mul_prev=_need(bigram, "mul_prev", int, "embedding.bigram."),
            bigram_mul_cur=_need(bigram, "mul_cur", int, "embedding.bigram."),
            layers=tuple(layers),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)),
        )
        if out.vocab < 1 or out.width < 1 or not out.norm_eps > 0 or out.bigram_buckets < 1:
            raise ConfigError("vocab, width, norm.eps and embedding.bigram.buckets must be positive")
        if out.bigram_mul_prev < 0 or out.bigram_mul_cur < 0:
            raise ConfigError("embedding.bigram.mul_prev and mul_cur must not be negative")
        return out

    @classmethod
    def from_folder(cls, folder: str | Path) -> "MolotarConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "postln_alpha": self.postln_alpha,
            "embedding": {"scale": self.embedding_scale,
                          "bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev, "mul_cur": self.bigram_mul_cur}},
            "layers": [layer.to_dict() for layer in self.layers],
        }  # fmt: skip
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
