"""Typed configuration of the Pimezen decoder, read from its own ``config.json`` keys.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``norm.eps`` and ``layers``: a list with
one entry per layer, each naming its ``type`` (which mixer the layer has), the mixer's sizes and
constants under ``mixer`` and its feed-forward under ``mlp`` (``null``: the layer has none).  Layers
may differ from one another in every size.  The one mixer type of this design, ``parallel``, runs a
softmax attention (``left``) beside a gated linear attention (``right``); the rank of the decay's
low-rank projection is not a key of the configuration but the shape of its tensor, so it is read
from the checkpoint's header (``decay_ranks``; a configuration made in memory names it).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from mini_engine_b200.config.qwen3 import ConfigError


def _need(raw: Mapping[str, Any], key: str, kind: type | tuple[type, ...], where: str) -> Any:
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks the key {where}{key!r}")
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config.json key {where}{key!r} must be {kind}, got {value!r}")
    return value


@dataclass(frozen=True)
class SoftmaxBranch:
    """The softmax attention of a parallel mixer."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int  # mask.size: position i sees j when i - j < window ...
    keep_first: int  # ... or j < keep_first

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "SoftmaxBranch":
        mask = _need(raw, "mask", Mapping, where)
        out = cls(
            heads=_need(raw, "heads", int, where),
            kv_heads=_need(raw, "kv_heads", int, where),
            dim=_need(raw, "dim", int, where),
            vdim=_need(raw, "vdim", int, where),
            scale=float(_need(raw, "scale", (int, float), where)),
            window=_need(mask, "size", int, where + "mask."),
            keep_first=_need(mask, "keep_first", int, where + "mask."),
        )
        if min(out.heads, out.kv_heads, out.dim, out.vdim, out.window) < 1 or out.keep_first < 0:
            raise ConfigError(f"{where}: sizes must be positive")
        if out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "mask": {"size": self.window, "keep_first": self.keep_first}}  # fmt: skip


@dataclass(frozen=True)
class LinearBranch:
    """The gated linear attention of a parallel mixer."""

    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str, decay_rank: int) -> "LinearBranch":
        out = cls(
            heads=_need(raw, "heads", int, where),
            dim=_need(raw, "dim", int, where),
            vdim=_need(raw, "vdim", int, where),
            tau=float(_need(raw, "tau", (int, float), where)),
            decay_rank=int(decay_rank),
        )
        if min(out.heads, out.dim, out.vdim, out.decay_rank) < 1 or not out.tau > 0:
            raise ConfigError(f"{where}: sizes and tau must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int
    limit: float

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class PimezenLayer:
    left: SoftmaxBranch
    right: LinearBranch
    left_scale: float
    right_scale: float
    mlp: DenseFeedForward | None
    type: str = "parallel"

    def to_dict(self) -> dict[str, Any]:
        return {
            "type": self.type,
            "mixer": {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                      "right_scale": self.right_scale},
            "mlp": None if self.mlp is None else self.mlp.to_dict(),
        }  # fmt: skip


@dataclass(frozen=True)
class PimezenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[PimezenLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Pimezen"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], decay_ranks: Mapping[int, int] | None = None) -> "PimezenConfig":
        """``decay_ranks``: per layer index the rank of the decay's low-rank projection (from the
        checkpoint's tensor shapes); a layer's ``mixer.right.decay_rank`` key is used where present."""
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"architecture must be {cls.architecture!r}, got {raw.get('architecture')!r}")
        norm = _need(raw, "norm", Mapping, "")
        layers = []
        for index, entry in enumerate(_need(raw, "layers", list, "")):
            where = f"layers[{index}]."
            kind = _need(entry, "type", str, where)
            if kind != "parallel":
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (known: 'parallel')")
            mixer = _need(entry, "mixer", Mapping, where)
            right_raw = _need(mixer, "right", Mapping, where + "mixer.")
            rank = right_raw.get("decay_rank", (decay_ranks or {}).get(index))
            if rank is None:
                raise ConfigError(f"{where}mixer.right: the rank of the decay projection is neither given nor found in the checkpoint")
            mlp_raw = entry.get("mlp")
            mlp = None
            if mlp_raw is not None:
                if _need(mlp_raw, "kind", str, where + "mlp.") != "dense":
                    raise ConfigError(f"{where}mlp.kind {mlp_raw['kind']!r} is not a feed-forward of this design (known: 'dense')")
                mlp = DenseFeedForward(_need(mlp_raw, "ff", int, where + "mlp."), float(_need(mlp_raw, "limit", (int, float), where + "mlp.")))
                if mlp.ff < 1 or not mlp.limit > 0:
                    raise ConfigError(f"{where}mlp: ff and limit must be positive")
            layers.append(
                PimezenLayer(
                    left=SoftmaxBranch.from_dict(_need(mixer, "left", Mapping, where + "mixer."), where + "mixer.left."),
                    right=LinearBranch.from_dict(right_raw, where + "mixer.right.", rank),
                    left_scale=float(_need(mixer, "left_scale", (int, float), where + "mixer.")),
                    right_scale=float(_need(mixer, "right_scale", (int, float), where + "mixer.")),
                    mlp=mlp,
                )
            )
        if not layers:
            raise ConfigError("config.json lists no layers")
        eos = raw.get("eos_token_id")
        out = cls(
            vocab=_need(raw, "vocab", int, ""),
            width=_need(raw, "width", int, ""),
            norm_eps=float(_need(norm, "eps", (int, float), "norm.")),
            layers=tuple(layers),
            eos_token_ids=() if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)),
        )
        if out.vocab < 1 or out.width < 1 or not out.norm_eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        return out

    @classmethod
    def from_folder(cls, folder: str | Path) -> "PimezenConfig":
        from mini_engine_b200.weights.safetensors_io import read_folder_index

        folder = Path(folder)
        raw = json.loads((folder / "config.json").read_text())
        ranks: dict[int, int] = {}
        count = len(raw.get("layers") or [])
        index = read_folder_index(folder) if any(folder.glob("*.safetensors")) else {}
        for layer in range(count):
            name = f"l{layer}.mix.right.a1"
            if name in index:
                ranks[layer] = int(index[name].entries[name][1][0])
        return cls.from_dict(raw, ranks)

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for layer in self.layers:
            entry = layer.to_dict()
            entry["mixer"]["right"]["decay_rank"] = layer.right.decay_rank
            layers.append(entry)
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "layers": layers}  # fmt: skip
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
