"""Molotar laid out as parts.

The embedding adds a row of a second table chosen by the pair (previous token, token) to the scaled token row.
In every layer the norm follows the sum: ``x = norm1(alpha * x + mixer(x))``, then (where the layer has a
feed-forward) ``x = norm2(alpha * x + ff(x))``; the sublayers read ``x`` itself.  A layer's mixer is one of

* ``attention``: grouped-query attention with q and k normalised over their whole projections, a rotation of the
  first part of each head with stretched slow frequencies, a sliding window, a softmax with a silent participant
  of score zero, and a sigmoid gate per head; a layer may read an earlier layer's keys and values instead of
  making its own;
* ``rglru``: a gated linear recurrence per channel behind a short causal convolution, gated by a tanh-GELU branch.

The feed-forward is a set of small gated units of which a token uses the few that a sigmoid router with groups
chooses.  Every size and every constant that models of this design may differ in comes from the typed
configuration, layer by layer; the constants below are fixed by the design.
"""

from __future__ import annotations

from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from mini_engine_b200.config.molotar import AttentionMixer, MolotarConfig, RecurrentMixer, RoutedFeedForward
from mini_engine_b200.config.registry import Architecture, register_architecture

GATE_SLOPE = 1.702  # sigmoid(1.702 g) of a unit
UP_OFFSET = 1.0  # (u + 1)
DECAY_SHARPNESS = 8.0  # a = exp(-8 r softplus(lam))


def _attention(mixer: AttentionMixer, eps: float) -> PartSpec:
    position = None
    if mixer.rot_dims:
        params = {"head_dim": mixer.dim, "theta": mixer.rot_base, "rotary_dim": mixer.rot_dims}
        if mixer.rot_scaling is not None:
            params["wavelength_scaling"] = mixer.rot_scaling.to_dict()
        position = PartSpec("rope", params)
    return PartSpec(
        "gqa_attention",
        {
            "num_heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim, "value_dim": mixer.vdim,
            "qk_norm_eps": eps, "qk_norm_scope": "projection", "position_encoding": position, "window": mixer.window,
            "scale": mixer.scale, "softmax_sink": True, "head_gate": True, "reads_shared_cache": mixer.kv_from is not None,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm",
                      "gate": "mix.g"},
        },
    )  # fmt: skip


def _recurrence(mixer: RecurrentMixer) -> PartSpec:
    return PartSpec(
        "gated_linear_recurrence",
        {
            "channels": mixer.width, "blocks": mixer.blocks, "taps": mixer.conv, "sharpness": DECAY_SHARPNESS,
            "names": {"y": "mix.y", "y_bias": "mix.y.b", "x": "mix.x", "x_bias": "mix.x.b", "conv": "mix.conv",
                      "conv_bias": "mix.conv.b", "ra": "mix.ra", "ra_bias": "mix.ra.b", "ri": "mix.ri", "ri_bias": "mix.ri.b",
                      "lam": "mix.lam", "o": "mix.o"},
        },
    )  # fmt: skip


def _feed_forward(mlp: RoutedFeedForward) -> PartSpec:
    return PartSpec(
        "routed_experts",
        {
            "units": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "group_count": mlp.group_count,
            "group_keep": mlp.group_keep, "weight_scale": mlp.scale, "gate_slope": GATE_SLOPE, "limit": mlp.limit,
            "up_offset": UP_OFFSET,
            "names": {"router": "mlp.router", "unit": "mlp.e{index}.", "gate": "gate", "up": "up", "down": "down"},
        },
    )  # fmt: skip


def molotar_spec(cfg: MolotarConfig) -> ModelSpec:
    eps = cfg.norm_eps
    layers, order = [], []
    for index, layer in enumerate(cfg.layers):
        norm = lambda name: PartSpec("rmsnorm", {"name": name, "eps": eps})  # noqa: E731
        mixer = _attention(layer.mixer, eps) if layer.type == "attention" else _recurrence(layer.mixer)
        if layer.mlp is None:
            layers.append(
                LayerSpec(
                    prefix=f"l{index}.", block="postnorm_mixer_only", mixer=mixer, feed_forward=None, mixer_norm=norm("norm1"),
                    block_params={"alpha": cfg.postln_alpha, "unused_names": ("norm2",)},
                )
            )  # fmt: skip
        else:
            layers.append(
                LayerSpec(
                    prefix=f"l{index}.", block="postnorm", mixer=mixer, feed_forward=_feed_forward(layer.mlp),
                    mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2"), block_params={"alpha": cfg.postln_alpha},
                )
            )  # fmt: skip
        order.append(OrderEntry(index, cache_of=getattr(layer.mixer, "kv_from", None)))
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        embedding=PartSpec(
            "pair_hash_embedding",
            {"weight": "embed", "pair_weight": "bigram", "multiplier": cfg.embedding_scale, "buckets": cfg.bigram_buckets,
             "mul_prev": cfg.bigram_mul_prev, "mul_cur": cfg.bigram_mul_cur},
        ),  # fmt: skip
        layers=tuple(layers),
        order=tuple(order),
        final_norm=PartSpec("rmsnorm", {"name": "final.norm", "eps": eps}),
        head=PartSpec("linear_head", {"weight": "head"}),
    )


register_architecture(
    Architecture(
        name=MolotarConfig.architecture,
        read_config=MolotarConfig.from_folder,
        build_spec=molotar_spec,
        config_type=MolotarConfig,
    )
)
