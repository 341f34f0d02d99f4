"""A gated linear recurrence per channel as a mixer part (the real-gated linear recurrent unit).

Two branches of ``channels`` columns are projected from the input ``h``::

    y_t = gelu_tanh(W_y h_t + b_y)                    x_t = W_x h_t + b_x
    u_t = b_c + sum_j taps[:, K-1-j] * x_(t-j)        (causal, per channel, zeros before the sequence)
    r_t = sigmoid(Ra u_t + b_ra)    i_t = sigmoid(Ri u_t + b_ri)     (Ra, Ri block-diagonal: ``blocks`` equal blocks)
    a_t = exp(-c * r_t * softplus(lam))               S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t

and the output is ``W_o (S_t * y_t)``.  ``c`` (``sharpness``) is a constant of the model.  The state of a request
is ``S`` and the last ``K - 1`` inputs ``x`` of the convolution, ``[K, channels]`` float32 in the request's state
slot of the cache manager; it starts at zero.  Gates, decay and recurrence are computed in 32-bit from the 32-bit
sums of the projections; the two projections run as one product on the row-concatenated weight.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import LayerCache, Mixer, StateSpec, StepContext, register
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    capturable = True
    # The scan is one long kernel per layer, like the scan of the gated linear attention, with which prompt
    # steps launched as programmatic dependents were seen to stall; this mixer's steps run in plain stream order too.
    programmatic_launch = False

    def __init__(
        self,
        prefix: str,
        hidden_size: int,
        *,
        channels: int,
        blocks: int,
        taps: int,
        sharpness: float,
        names: Mapping[str, str] | None = None,
    ):
        if min(channels, blocks, taps) < 1 or channels % blocks or not sharpness > 0:
            raise ValueError("gated_linear_recurrence: sizes must be positive, blocks must divide channels, sharpness > 0")
        self.hidden, self.channels, self.blocks, self.taps = hidden_size, channels, blocks, taps
        self.sharpness = float(sharpness)
        defaults = {"y": "gate_proj.weight", "y_bias": "gate_proj.bias", "x": "in_proj.weight", "x_bias": "in_proj.bias",
                    "conv": "conv.weight", "conv_bias": "conv.bias", "ra": "recurrence_gate.weight",
                    "ra_bias": "recurrence_gate.bias", "ri": "input_gate.weight", "ri_bias": "input_gate.bias",
                    "lam": "decay", "o": "o_proj.weight"}  # fmt: skip
        self.names = {key: prefix + (names or {}).get(key, value) for key, value in defaults.items()}
        self.proj: Linear | None = None
        self.out: Linear | None = None
        self.held: dict[str, torch.Tensor] = {}

    def state(self) -> StateSpec:
        return StateSpec((self.taps, self.channels), torch.float32)

    def weight_specs(self) -> list[WeightSpec]:
        n, c, width = self.names, self.channels, self.channels // self.blocks
        small = dict(role="vector", init="small_normal")
        return [
            WeightSpec(n["y"], (c, self.hidden)),
            WeightSpec(n["y_bias"], (c,), **small),
            WeightSpec(n["x"], (c, self.hidden)),
            WeightSpec(n["x_bias"], (c,), **small),
            WeightSpec(n["conv"], (c, self.taps), **small),
            WeightSpec(n["conv_bias"], (c,), **small),
            # the gates enter the recurrence: kept and applied in 32-bit
            WeightSpec(n["ra"], (self.blocks, width, width), **small),
            WeightSpec(n["ra_bias"], (self.blocks, width), **small),
            WeightSpec(n["ri"], (self.blocks, width, width), **small),
            WeightSpec(n["ri_bias"], (self.blocks, width), **small),
            WeightSpec(n["lam"], (c,), **small),
            WeightSpec(n["o"], (self.hidden, c)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.proj = Linear(torch.cat((tensors[n["y"]], tensors[n["x"]]), dim=0).contiguous())
        self.out = Linear(tensors[n["o"]])
        self.held = {
            "in_bias": torch.cat((tensors[n["y_bias"]], tensors[n["x_bias"]])).contiguous(),
            "taps": tensors[n["conv"]],
            "conv_bias": tensors[n["conv_bias"]],
            # [blocks, in, out]: the kernel's threads are output channels and read along them
            "ra_t": tensors[n["ra"]].transpose(1, 2).contiguous(),
            "ra_bias": tensors[n["ra_bias"]].reshape(-1).contiguous(),
            "ri_t": tensors[n["ri"]].transpose(1, 2).contiguous(),
            "ri_bias": tensors[n["ri_bias"]].reshape(-1).contiguous(),
            "lam": tensors[n["lam"]],
        }

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        tokens = h.shape[0]
        proj = self.proj.forward(h, ctx, "recurrence.proj")
        decay = ctx.buffer("recurrence.decay", (tokens, self.channels), torch.float32)
        driven = ctx.buffer("recurrence.driven", (tokens, self.channels), torch.float32)
        conv = ctx.buffer("recurrence.conv", (tokens, self.channels), torch.float32)
        out = ctx.buffer("recurrence.out", (tokens, self.channels), ctx.dtype)
        ops.rglru(
            proj=proj, **self.held, ctx=ctx, state=cache.state, decay=decay, driven=driven, conv=conv, out=out,
            sharpness=self.sharpness,
        )  # fmt: skip
        return self.out.forward(out, ctx, "recurrence.o")
