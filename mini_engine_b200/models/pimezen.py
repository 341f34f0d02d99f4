"""Pimezen laid out as parts.

Every layer is pre-norm with layer scales: ``x += ls1 * mixer(norm1(x))``, then (where the layer has a
feed-forward) ``x += ls2 * ff(norm2(x))``; the norms keep their weights around zero (``(1 + w) * x /
rms(x)``).  The mixer runs two mixers side by side on the same input and adds them with two constants:

* a grouped-query softmax attention with per-head q/k norms, no rotation, value heads of their own
  width, a sliding window that also keeps the sequence's first tokens, a logarithmic distance bias
  per head taken off the scores and the heads' weights mixed by a learned matrix after the softmax;
* a gated linear attention with a decay per key channel and a 32-bit matrix state per head.

The feed-forward is gated: ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``,
``W_down (g * sigmoid(1.702 g) * (u + 1))``.  The head is the embedding matrix.  Every size and every
constant that models of this design may differ in comes from the typed configuration, layer by
layer; 1.702 and the 1 of the gated unit and of the norms are fixed by the design.
"""

from __future__ import annotations

from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from mini_engine_b200.config.pimezen import PimezenConfig, PimezenLayer
from mini_engine_b200.config.registry import Architecture, register_architecture

GATE_SLOPE = 1.702  # sigmoid(1.702 g) of the gated unit
UP_OFFSET = 1.0  # (u + 1)
NORM_OFFSET = 1.0  # (1 + w)


def _mixer(layer: PimezenLayer, eps: float) -> PartSpec:
    left, right = layer.left, layer.right
    softmax = PartSpec(
        "gqa_attention",
        {
            "num_heads": left.heads, "kv_heads": left.kv_heads, "head_dim": left.dim, "value_dim": left.vdim,
            "qk_norm_eps": eps, "position_encoding": None, "window": left.window, "keep_first": left.keep_first,
            "scale": left.scale, "distance_bias": True, "talking_heads": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "r1": "r1",
                      "r2": "r2", "talk": "talk"},
        },
    )  # fmt: skip
    linear = PartSpec(
        "gated_linear_attention",
        {
            "num_heads": right.heads, "head_dim": right.dim, "value_dim": right.vdim, "decay_rank": right.decay_rank,
            "tau": right.tau, "norm_eps": eps,
            "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2",
                      "a2_bias": "a2.b"},
        },
    )  # fmt: skip
    return PartSpec(
        "parallel_mixers",
        {
            "branches": (
                {"mixer": softmax, "factor": layer.left_scale, "prefix": "mix.left."},
                {"mixer": linear, "factor": layer.right_scale, "prefix": "mix.right."},
            )
        },
    )


def pimezen_spec(cfg: PimezenConfig) -> ModelSpec:
    eps = cfg.norm_eps
    layers = []
    for index, layer in enumerate(cfg.layers):
        norm = lambda name: PartSpec("rmsnorm", {"name": name, "eps": eps, "offset": NORM_OFFSET})  # noqa: E731
        if layer.mlp is None:
            layers.append(
                LayerSpec(
                    prefix=f"l{index}.", block="prenorm_scaled_mixer_only", mixer=_mixer(layer, eps), feed_forward=None,
                    mixer_norm=norm("norm1"),
                    block_params={"scale_names": {"mixer": "ls1"}, "unused_names": ("norm2", "ls2")},
                )
            )  # fmt: skip
            continue
        feed_forward = PartSpec(
            "gated_mlp",
            {
                "intermediate_size": layer.mlp.ff, "gate_slope": GATE_SLOPE, "limit": layer.mlp.limit,
                "up_offset": UP_OFFSET, "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"},
            },
        )  # fmt: skip
        layers.append(
            LayerSpec(
                prefix=f"l{index}.", block="prenorm_scaled", mixer=_mixer(layer, eps), feed_forward=feed_forward,
                mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2"),
                block_params={"scale_names": {"mixer": "ls1", "feed_forward": "ls2"}},
            )
        )  # fmt: skip
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", {"weight": "embed"}),
        layers=tuple(layers),
        order=tuple(OrderEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"name": "final.norm", "eps": eps, "offset": NORM_OFFSET}),
        head=PartSpec("linear_head", {"weight": "head.tied", "tied_to": "embed"}),
    )


register_architecture(
    Architecture(
        name=PimezenConfig.architecture,
        read_config=PimezenConfig.from_folder,
        build_spec=pimezen_spec,
        config_type=PimezenConfig,
    )
)
