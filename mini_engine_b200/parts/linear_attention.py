"""Gated linear attention as a mixer part: a matrix state per head instead of cached keys.

Per head, with ``q_t = (W_q h_t) * dim^-1/2``, ``k_t = W_k h_t`` (``dim`` channels) and ``v_t = W_v h_t``
(``vdim`` channels)::

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t
    alpha_t = sigmoid(z_t)^(1/tau)                 z_t = W_a2 (W_a1 h_t) + b   (one decay per key channel)

Each head's ``o_t`` is divided by its root mean square over ``vdim`` and multiplied by a weight
``[vdim]`` shared by the heads; the heads are concatenated, multiplied by ``silu(W_g h_t)`` and projected
by ``W_o``.  The state ``[heads, dim, vdim]`` is float32, starts at zero and is carried from token to
token in the request's state slot of the cache manager; the decay (sigmoid, its logarithm, the power),
the recurrence and the unit norm are computed in 32-bit from the 32-bit sums of the projections.

The five projections of the input run as one product on the row-concatenated weight; the second,
small factor of the decay's low-rank projection is applied by the kernel that prepares q, k and the
decays of all tokens for the scan.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import LayerCache, Mixer, StateSpec, StepContext, register
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    capturable = True
    # Prompt steps of a model with this mixer at widths of 4,096 stalled on a B200 when every kernel of the step
    # was launched as a programmatic dependent (after 5 to 12 steps of 2,048 tokens in a row) and ran through in
    # plain stream order; which kernels meet badly is not known, so such a model's steps run in order.
    programmatic_launch = False

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        num_heads: int,
        head_dim: int,
        value_dim: int,
        decay_rank: int,
        tau: float,
        norm_eps: float,
        query_scale: float | None = None,
        names: Mapping[str, str] | None = None,
    ):
        if min(num_heads, head_dim, value_dim, decay_rank) < 1 or not tau > 0:
            raise ValueError("gated_linear_attention: sizes and tau must be positive")
        self.hidden, self.heads, self.dim, self.vdim = hidden_size, num_heads, head_dim, value_dim
        self.rank, self.tau, self.eps = decay_rank, float(tau), float(norm_eps)
        self.q_scale = float(query_scale) if query_scale is not None else head_dim**-0.5
        defaults = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                    "o": "o_proj.weight", "norm": "norm.weight", "a1": "decay_down.weight",
                    "a2": "decay_up.weight", "a2_bias": "decay_up.bias"}  # fmt: skip
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        # Columns of the fused input projection, in this order.
        widths = {"q": num_heads * head_dim, "k": num_heads * head_dim, "v": num_heads * value_dim,
                  "g": num_heads * value_dim, "a": decay_rank}  # fmt: skip
        self.columns, column = {}, 0
        for key, width in widths.items():
            self.columns[key] = column
            column += width
        self.proj: Linear | None = None
        self.out: Linear | None = None
        self.norm_weight = self.a2t = self.a2_bias = None

    def state(self) -> StateSpec:
        return StateSpec((self.heads, self.dim, self.vdim), torch.float32)

    def weight_specs(self) -> list[WeightSpec]:
        n, inner, outer = self.names, self.heads * self.dim, self.heads * self.vdim
        return [
            WeightSpec(n["q"], (inner, self.hidden)),
            WeightSpec(n["k"], (inner, self.hidden)),
            WeightSpec(n["v"], (outer, self.hidden)),
            WeightSpec(n["g"], (outer, self.hidden)),
            WeightSpec(n["o"], (self.hidden, outer)),
            WeightSpec(n["norm"], (self.vdim,), role="vector", init="ones_normal"),
            WeightSpec(n["a1"], (self.rank, self.hidden)),
            # the second factor of the decay enters the recurrence: kept and applied in 32-bit
            WeightSpec(n["a2"], (inner, self.rank), role="vector", init="small_normal"),
            WeightSpec(n["a2_bias"], (inner,), role="vector", init="ones_normal"),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.proj = Linear(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g", "a1")], dim=0).contiguous())
        self.out = Linear(tensors[n["o"]])
        self.norm_weight, self.a2_bias = tensors[n["norm"]], tensors[n["a2_bias"]]
        self.a2t = tensors[n["a2"]].t().contiguous()  # [rank, heads * dim]: the prepare kernel reads it along the channels

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        tokens = h.shape[0]
        proj = self.proj.forward(h, ctx, "gla.proj")
        raw = ctx.buffer("gla.raw", (tokens, self.heads * self.vdim), torch.float32)
        prepared = ctx.buffer("gla.prepared", (tokens, self.heads * 3 * self.dim), torch.float32)
        ops.gla_scan(
            proj=proj, columns=self.columns, a2t=self.a2t, a2_bias=self.a2_bias, ctx=ctx, state=cache.state, out=raw,
            prepared=prepared, q_scale=self.q_scale, tau=self.tau, heads=self.heads, dim=self.dim, vdim=self.vdim,
        )  # fmt: skip
        gated = ctx.buffer("gla.out", (tokens, self.heads * self.vdim), ctx.dtype)
        ops.gla_finish(
            o=raw, proj=proj, gate_column=self.columns["g"], weight=self.norm_weight, eps=self.eps, out=gated,
            heads=self.heads, vdim=self.vdim,
        )  # fmt: skip
        return self.out.forward(gated, ctx, "gla.o")
