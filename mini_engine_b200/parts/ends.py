"""The two ends of a model as parts: token embedding and output head.

``token_embedding``: ``x = E[token_ids]``, times ``multiplier`` when the model scales its
embeddings (the reference's decoder does not: src/mini_engine/model.py:182 of
YuvGev00/mini-engine).  ``linear_head``: ``logits = rows W^T`` without bias, where ``W`` may be
the embedding matrix itself (``tied_to``; src/mini_engine/model.py:168-170,186-187); a head may
also have a bias, a logit scale and a soft cap ``cap * tanh(logits / cap)``, applied in that
order by one small kernel.  Both are looked up by ``PartSpec.kind`` like every other part, so a
model with another first or last part registers its own and changes nothing here.

``pair_hash_embedding`` adds a row of a second table that is chosen by the pair (previous token, token):
``x = E[id] * multiplier + P[(previous * mul_prev + id * mul_cur) mod buckets]``, and the table's last row
(number ``buckets``) for the first token of a sequence.  The id in front of a step's first token is the
request's state: one int32 in the request's state slot of the cache manager.
"""

from __future__ import annotations

from typing import Mapping

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import Embedding, Head, StateSpec, StepContext, register
from mini_engine_b200.parts.linear import Linear
from mini_engine_b200.weights.loader import WeightSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, *, weight: str, multiplier: float | None = None):
        self.vocab, self.hidden = vocab_size, hidden_size
        self.weight_name = weight
        self.multiplier = 1.0 if multiplier is None else float(multiplier)
        self.table: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.vocab, self.hidden))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.weight_name]

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, out: torch.Tensor) -> None:
        ops.embedding(self.table, token_ids, out, self.multiplier)


@register("embedding", "pair_hash_embedding")
class PairHashEmbedding(Embedding):
    capturable = True

    def __init__(
        self, vocab_size: int, hidden_size: int, *, weight: str, pair_weight: str, buckets: int, mul_prev: int,
        mul_cur: int, multiplier: float | None = None,
    ):  # fmt: skip
        if buckets < 1 or mul_prev < 0 or mul_cur < 0:
            raise ValueError("pair_hash_embedding: buckets must be positive and the multipliers not negative")
        self.vocab, self.hidden = vocab_size, hidden_size
        self.weight_name, self.pair_name = weight, pair_weight
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.multiplier = 1.0 if multiplier is None else float(multiplier)
        self.table: torch.Tensor | None = None
        self.pair_table: torch.Tensor | None = None

    def state(self) -> StateSpec:
        return StateSpec((1,), torch.int32)  # the request's last token

    def weight_specs(self) -> list[WeightSpec]:
        return [
            WeightSpec(self.weight_name, (self.vocab, self.hidden)),
            WeightSpec(self.pair_name, (self.buckets + 1, self.hidden)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table, self.pair_table = tensors[self.weight_name], tensors[self.pair_name]

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, out: torch.Tensor) -> torch.Tensor | None:
        if ctx.embedding_state is None:
            raise RuntimeError("pair_hash_embedding needs the step's embedding state (the requests' last tokens)")
        rounded = None
        if ctx.dtype != torch.float32:
            rounded = ctx.buffer("embedding.rounded", tuple(out.shape), ctx.dtype)
        ops.pair_embedding(
            table=self.table, pair_table=self.pair_table, ctx=ctx, last_token=ctx.embedding_state.view(-1), out=out,
            rounded=rounded, multiplier=self.multiplier, buckets=self.buckets, mul_prev=self.mul_prev, mul_cur=self.mul_cur,
        )  # fmt: skip
        return rounded


@register("head", "linear_head")
class LinearHead(Head):
    capturable = True

    def __init__(
        self,
        vocab_size: int,
        hidden_size: int,
        *,
        weight: str,
        tied_to: str | None = None,
        bias: str | None = None,
        logit_scale: float | None = None,
        soft_cap: float | None = None,
    ):
        self.vocab, self.hidden = vocab_size, hidden_size
        self.weight_name, self.tied_to, self.bias_name = weight, tied_to, bias
        self.logit_scale = 1.0 if logit_scale is None else float(logit_scale)
        self.soft_cap = 0.0 if soft_cap is None else float(soft_cap)
        if self.soft_cap < 0:
            raise ValueError("soft_cap must be positive (or absent)")
        self.linear: Linear | None = None
        self.bias: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        specs = [WeightSpec(self.weight_name, (self.vocab, self.hidden), alias_of=self.tied_to)]
        if self.bias_name:
            specs.append(WeightSpec(self.bias_name, (self.vocab,), role="vector"))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.linear = Linear(tensors[self.weight_name])
        self.bias = tensors[self.bias_name] if self.bias_name else None

    def forward(self, rows: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = self.linear.forward(rows, ctx, "logits", whole=True)[0]
        if self.bias is not None or self.logit_scale != 1.0 or self.soft_cap > 0.0:
            ops.logits_finish(logits, self.bias, self.logit_scale, self.soft_cap)
        return logits
