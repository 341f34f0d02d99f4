"""A plain, slow implementation of the Pimezen decoder, one function per mechanism, written from
the design's equations with whole-sequence tensors (no cache, no state slots, no batching).  It shares
no code with the package and is the oracle of ``test_pimezen_gpu.py``.

Notation: ``T`` tokens at positions ``0..T-1``; weights ``[out, in]`` applied as ``x @ W.T``; everything in
the dtype of the inputs (the tests pass float64).
"""

from __future__ import annotations

import math

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def zero_centred_norm(x, weight, eps):
    """RMS norm whose stored weight lies around zero: ``unit_rms(x) * (1 + w)``."""
    return unit_rms(x, eps) * (1.0 + weight)


def visible(T: int, window: int, keep_first: int) -> torch.Tensor:
    """``[T, T]`` bool: query i sees key j when j <= i and (i - j < window or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def softmax_weights(q, k, scale, r1, r2, window, keep_first):
    """``q [T, H, D]``, ``k [T, H, D]`` (already expanded to query heads) -> ``[H, T, T]`` weights:
    softmax over visible keys of ``q.k * scale - r1_h * ln(1 + r2_h * (i - j))``."""
    T = q.shape[0]
    distance = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0).to(q.dtype)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    scores = scores - r1[:, None, None] * torch.log(1.0 + r2[:, None, None] * distance)
    scores = scores.masked_fill(~visible(T, window, keep_first), -math.inf)
    return torch.softmax(scores, dim=-1)


def mix_heads(weights, talk):
    """``weights [H, T, T]`` -> ``sum_g talk[h, g] * weights[g]``."""
    return torch.einsum("hg,gij->hij", talk, weights)


def softmax_branch(h, w, p, cfg, eps):
    """The softmax attention of a parallel mixer.  ``cfg``: heads, kv_heads, dim, vdim, scale, window, keep_first."""
    T = h.shape[0]
    H, G, D, V = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    kv_of_head = torch.arange(H) // (H // G)
    weights = softmax_weights(q, k[:, kv_of_head], cfg["scale"], w[p + "r1"], w[p + "r2"], cfg["window"], cfg["keep_first"])
    weights = mix_heads(weights, w[p + "talk"])
    out = torch.einsum("hij,jhv->ihv", weights, v[:, kv_of_head])
    return out.reshape(T, H * V) @ w[p + "o"].T


def decays(h, w, p, heads, dim, tau):
    """``alpha [T, heads, dim] = sigmoid(W_a2 (W_a1 h) + b) ** (1 / tau)``."""
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    return torch.sigmoid(z).pow(1.0 / tau).view(h.shape[0], heads, dim)


def recurrence(q, k, v, alpha, state=None):
    """``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head, token by token.
    ``q, k, alpha [T, H, D]``, ``v [T, H, V]``; returns ``o [T, H, V]`` and the last state ``[H, D, V]``."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros(H, D, V, dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


def linear_branch(h, w, p, cfg, eps):
    """The gated linear attention of a parallel mixer.  ``cfg``: heads, dim, vdim, tau."""
    T = h.shape[0]
    H, D, V = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D**-0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    o, _ = recurrence(q, k, v, decays(h, w, p, H, D, cfg["tau"]))
    o = unit_rms(o, eps) * w[p + "norm"]
    gate = torch.nn.functional.silu(h @ w[p + "g"].T)
    return (o.reshape(T, H * V) * gate) @ w[p + "o"].T


def gated_unit(h, w, p, limit):
    """``W_down (g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, +-limit)``."""
    g = (h @ w[p + "gate"].T).clamp(max=limit)
    u = (h @ w[p + "up"].T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def layer(x, w, index, cfg, eps):
    p = f"l{index}."
    h = zero_centred_norm(x, w[p + "norm1"], eps)
    m = cfg["mixer"]
    left = {**{k: m["left"][k] for k in ("heads", "kv_heads", "dim", "vdim", "scale")},
            "window": m["left"]["mask"]["size"], "keep_first": m["left"]["mask"]["keep_first"]}  # fmt: skip
    mixed = m["left_scale"] * softmax_branch(h, w, p + "mix.left.", left, eps)
    mixed = mixed + m["right_scale"] * linear_branch(h, w, p + "mix.right.", m["right"], eps)
    x = x + w[p + "ls1"] * mixed
    if cfg["mlp"] is not None:
        h = zero_centred_norm(x, w[p + "norm2"], eps)
        x = x + w[p + "ls2"] * gated_unit(h, w, p + "mlp.", cfg["mlp"]["limit"])
    return x


def forward_logits(weights, config, token_ids, dtype=torch.float64):
    """Logits ``[T, vocab]`` of one whole sequence; ``config`` is the ``config.json`` dictionary."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(token_ids)]
    for index, cfg in enumerate(config["layers"]):
        x = layer(x, w, index, cfg, eps)
    return zero_centred_norm(x, w["final.norm"], eps) @ w["embed"].T
