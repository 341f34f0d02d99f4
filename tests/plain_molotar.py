"""The Molotar decoder restated plainly: whole sequences, no cache, one function per mechanism.

Everything takes the raw ``config.json`` dictionary and a mapping from tensor names to tensors, and
computes in the dtype of ``h`` (the tests use float64).  Nothing here is shared with the engine.

Notation: ``T`` tokens, ``D`` model width, ``H`` query heads, ``G`` key/value heads, ``d`` key width,
``e`` value width, ``R`` rotated width, ``W`` window, ``C`` recurrent channels, ``B`` gate blocks.
"""

from __future__ import annotations

import math

import torch


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight.to(x.dtype)


# ------------------------------------------------------------------------------------ embedding


def embed(tokens: list[int], cfg: dict, w: dict, dtype=torch.float64) -> torch.Tensor:
    """Token row times a constant, plus a row of a second table chosen by the pair (previous token, token)."""
    e = cfg["embedding"]
    big = e["bigram"]
    rows = []
    for t, token in enumerate(tokens):
        if t == 0:
            pair = big["buckets"]  # the row behind the buckets: a sequence's first token has no pair
        else:
            pair = (tokens[t - 1] * big["mul_prev"] + token * big["mul_cur"]) % big["buckets"]
        rows.append(w["embed"][token].to(dtype) * e["scale"] + w["bigram"][pair].to(dtype))
    return torch.stack(rows)


# ------------------------------------------------------------------------------------- rotation


def rotary_frequencies(rot: dict) -> list[float]:
    """``f_i = base^(-2i/R)``, then stretched by wavelength: short waves stay, long ones are divided by
    ``factor``, and those between are blended linearly in ``original / wavelength``."""
    dims, base, sc = rot["dims"], rot["base"], rot.get("scaling")  # sc may be None: plain frequencies
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc is not None:
            wavelength = 2.0 * math.pi / f
            if wavelength < sc["original"] / sc["high"]:
                pass
            elif wavelength > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate(x: torch.Tensor, positions: list[int], rot: dict) -> torch.Tensor:
    """``x [T, heads, d]``: element i of a head turns with element i + R/2, i < R/2; the rest stays."""
    dims = rot["dims"]
    half = dims // 2
    freqs = torch.tensor(rotary_frequencies(rot), dtype=x.dtype)
    angle = torch.tensor(positions, dtype=x.dtype)[:, None] * freqs[None, :]  # [T, R/2]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., dims:]), dim=-1)


# ------------------------------------------------------------------------------------ attention


def attention_keys_values(h: torch.Tensor, m: dict, w: dict, p: str, eps: float):
    """Keys (normalised over the whole projection, then rotated) and values of a layer that has them."""
    T = h.shape[0]
    G, d, e = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ w[p + "k"].to(h.dtype).T
    k = rms_norm(k, w[p + "k.norm"], eps).view(T, G, d)
    if m.get("rot"):
        k = rotate(k, list(range(T)), m["rot"])
    v = (h @ w[p + "v"].to(h.dtype).T).view(T, G, e)
    return k, v


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int | None) -> torch.Tensor:
    """``q [T, H, d]``, ``k [T, G, d]``, ``v [T, G, e]`` of one sequence -> ``[T, H, e]``.  Query i sees keys j with
    ``0 <= i - j < window``; the weights are ``exp(s_j) / (1 + sum exp(s))``: a silent participant of score zero."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo : i + 1, g] @ q[i, head]) * scale
            weights = torch.exp(s) / (1.0 + torch.exp(s).sum())
            out[i, head] = (weights[:, None] * v[lo : i + 1, g]).sum(dim=0)
    return out


def attention(h: torch.Tensor, m: dict, w: dict, p: str, eps: float, kv=None):
    """Windowed grouped-query attention whose softmax has one more, silent participant of score zero,
    with a sigmoid gate per head on the way out.  ``kv``: keys and values of another layer to use."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    window = m["mask"]["size"] if m.get("mask") else None
    q = h @ w[p + "q"].to(h.dtype).T
    q = rms_norm(q, w[p + "q.norm"], eps).view(T, H, d)
    if m.get("rot"):
        q = rotate(q, list(range(T)), m["rot"])
    k, v = kv if kv is not None else attention_keys_values(h, m, w, p, eps)
    gate = torch.sigmoid(h @ w[p + "g"].to(h.dtype).T)  # [T, H]
    out = attend(q, k, v, m["scale"], window) * gate[:, :, None]
    return out.reshape(T, H * e) @ w[p + "o"].to(h.dtype).T, (k, v)


# ----------------------------------------------------------------------------- gated recurrence


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """Per channel: ``out_t = bias + sum_j taps[:, K-1-j] * x_(t-j)``; nothing before the start."""
    T, K = x.shape[0], taps.shape[1]
    out = bias.to(x.dtype).expand(T, -1).clone()
    for j in range(min(K, T)):
        out[j:] += x[: T - j] * taps[:, K - 1 - j].to(x.dtype)
    return out


def rglru(h: torch.Tensor, m: dict, w: dict, p: str) -> torch.Tensor:
    """Two branches of C channels; one is a gate (tanh-GELU), the other is convolved and run through
    ``S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t`` with ``a_t = exp(-8 r_t softplus(lam))``."""
    T, C, B = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].to(h.dtype).T + w[p + "y.b"].to(h.dtype))
    u = causal_conv(h @ w[p + "x"].to(h.dtype).T + w[p + "x.b"].to(h.dtype), w[p + "conv"], w[p + "conv.b"])
    ub = u.view(T, B, C // B)
    r = torch.sigmoid(torch.einsum("tbj,bkj->tbk", ub, w[p + "ra"].to(h.dtype)) + w[p + "ra.b"].to(h.dtype)).reshape(T, C)
    i = torch.sigmoid(torch.einsum("tbj,bkj->tbk", ub, w[p + "ri"].to(h.dtype)) + w[p + "ri.b"].to(h.dtype)).reshape(T, C)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"].to(h.dtype))
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    state = torch.zeros(C, dtype=h.dtype)
    states = []
    for t in range(T):
        state = a[t] * state + drive[t]
        states.append(state)
    return (torch.stack(states) * y) @ w[p + "o"].to(h.dtype).T


# --------------------------------------------------------------------------- routed feed-forward


def route(h: torch.Tensor, router: dict, weight: torch.Tensor, follow: dict | None = None, close: float = 0.0):
    """Per token: chosen experts, their weights, and how close the choice was.  Sigmoid scores; experts in equal
    groups of neighbours, a group valued by its two best scores, only the best groups eligible; the chosen scores
    normalised.  The third result is the smallest gap by which a group or an expert won its place.

    ``follow`` (token -> experts) is somebody else's choice: where it differs from the one made here it is taken
    instead, provided the decision here was closer than ``close`` (a choice with a tiny gap may fall the other way
    under rounding, and everything behind it then follows the other choice); a differing choice on a clear
    decision is an error."""
    E, top = router["experts"], router["top"]
    count, keep = (router["groups"]["count"], router["groups"]["keep"]) if router.get("groups") else (1, 1)
    scores = torch.sigmoid(h @ weight.to(h.dtype).T)  # [T, E]
    chosen, weights, gaps = [], [], []
    for t, s in enumerate(scores):
        per = E // count
        value = [sum(sorted(s[g * per : (g + 1) * per].tolist(), reverse=True)[:2]) for g in range(count)]
        ranked = sorted(range(count), key=lambda g: (-value[g], g))
        groups = ranked[:keep]
        allowed = sorted((x for g in groups for x in range(g * per, (g + 1) * per)), key=lambda x: (-float(s[x]), x))
        pick = allowed[:top]
        gap = float("inf")
        if keep < count:
            gap = min(gap, value[ranked[keep - 1]] - value[ranked[keep]])
        if top < len(allowed):
            gap = min(gap, float(s[allowed[top - 1]]) - float(s[allowed[top]]))
        if follow is not None and sorted(follow[t]) != sorted(pick):
            assert gap < close, f"token {t}: {sorted(follow[t])} chosen where {sorted(pick)} wins by {gap:.4f}"
            pick = list(follow[t])
        total = sum(float(s[x]) for x in pick) + 1e-20
        chosen.append(pick)
        weights.append([float(s[x]) / total * router["scale"] for x in pick])
        gaps.append(gap)
    return chosen, weights, gaps


def expert(h: torch.Tensor, w: dict, p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].to(h.dtype).T, max=limit)
    u = torch.clamp(h @ w[p + "up"].to(h.dtype).T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].to(h.dtype).T


def moe(h: torch.Tensor, mlp: dict, w: dict, p: str, gaps: list | None = None, follow: dict | None = None, close: float = 0.0) -> torch.Tensor:
    """``gaps`` (optional) collects, per call, every token's closest routing decision; ``follow``, ``close``: see :func:`route`."""
    chosen, weights, closest = route(h, mlp["router"], w[p + "router"], follow, close)
    if gaps is not None:
        gaps.append(closest)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for x, weight in zip(chosen[t], weights[t]):
            out[t] += weight * expert(h[t : t + 1], w, f"{p}e{x}.", mlp["expert"]["limit"])[0]
    return out


# ---------------------------------------------------------------------------------------- model


def forward(tokens: list[int], cfg: dict, w: dict, dtype=torch.float64, gaps: list | None = None, follow: dict | None = None, close: float = 0.0):
    """Logits ``[T, vocab]`` and the stream after every layer ``[layers, T, D]``.  A layer is
    ``x = norm1(alpha x + mixer(x))``, ``x = norm2(alpha x + ff(x))``: the norm follows the sum.
    ``follow``: per routed feed-forward (counted from 0 in layer order) and token, a choice to follow (:func:`route`)."""
    routed = 0
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = embed(tokens, cfg, w, dtype)
    kept, after = {}, []
    for index, layer in enumerate(cfg["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        if layer["type"] == "attention":
            source = m.get("kv_from")
            mixed, kv = attention(x, m, w, p + "mix.", eps, None if source is None else kept[source])
            kept[index] = kv
        elif layer["type"] == "rglru":
            mixed = rglru(x, m, w, p + "mix.")
        else:
            raise ValueError(layer["type"])
        x = rms_norm(alpha * x + mixed, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            chosen = None if follow is None else follow[routed]
            routed += 1
            x = rms_norm(alpha * x + moe(x, layer["mlp"], w, p + "mlp.", gaps, chosen, close), w[p + "norm2"], eps)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].to(dtype).T
    return logits, torch.stack(after)
