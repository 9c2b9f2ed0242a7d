"""A plain, slow restatement of the Mezadra decoder, one function per mechanism.

Everything runs on the CPU in float64 over whole sequences: no cache, no state carried between
calls, no batching.  It shares no code with the package; the tests compare the engine's logits,
and single mechanisms, with it.

Notation: ``x`` is ``[T, width]``, weights are ``[out, in]`` and applied as ``x @ W.T``; ``w`` maps
tensor names (``l0.mix.q`` ...) to float64 tensors; ``layer`` is one entry of the configuration's
``layers``.  A layer is ``x += norm1(mixer(x)); x += norm2(ff(x))``: the sublayers read the stream
itself and the norms sit on their outputs.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


# ------------------------------------------------------------------ small functions
def rms_norm(x: torch.Tensor, eps: float, weight: torch.Tensor | None = None) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """``y[t, c] = sum_j taps[c, j] * u[t - (n - 1) + j, c]`` with zeros before the sequence (``n`` taps)."""
    length, n = u.shape[0], taps.shape[1]
    y = torch.zeros_like(u)
    for j in range(n):
        back = n - 1 - j
        if back < length:
            y[back:] += taps[:, j] * u[: length - back]
    return y


def rotate(x: torch.Tensor, dims: int, base: float, positions: torch.Tensor) -> torch.Tensor:
    """``x [T, heads, dim]``: entry ``i < dims/2`` of a head is paired with entry ``i + dims/2``."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    low, high = x[..., :half], x[..., half:dims]
    return torch.cat([low * cos - high * sin, high * cos + low * sin, x[..., dims:]], dim=-1)


def capped(score: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(score / cap) if cap else score


# ------------------------------------------------------------------ mixers
def attention_values(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """The layer's own values ``[T, kv_heads * vdim]``: projection, then the short convolution."""
    return causal_conv(h @ w[prefix + "v"].T, w[prefix + "v.conv"])


def softmax_attention(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float, first_values, is_first: bool):
    """Causal softmax attention with a sink; returns ``(output, this layer's values before mixing)``.

    q, k, v pass a short convolution; q and k rotate on their first ``rot.dims`` entries and are then
    divided by their root mean square over the head; scores are scaled, squashed by ``cap * tanh(s / cap)``
    and normalised over the keys ``j <= i`` plus one more term ``exp(sink[head])`` that carries no value.
    """
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    rot = mixer.get("rot") or {}
    length = h.shape[0]
    positions = torch.arange(length)
    q = causal_conv(h @ w[prefix + "q"].T, w[prefix + "q.conv"]).view(length, heads, dim)
    k = causal_conv(h @ w[prefix + "k"].T, w[prefix + "k.conv"]).view(length, kv_heads, dim)
    own = attention_values(h, w, prefix)
    v = own
    if mixer.get("v_mix") and not is_first:
        lam = w[prefix + "vmix"]
        v = (1 - lam) * own + lam * first_values
    v = v.view(length, kv_heads, vdim)
    q = rms_norm(rotate(q, int(rot.get("dims", 0)), float(rot.get("base", 1.0)), positions), eps)
    k = rms_norm(rotate(k, int(rot.get("dims", 0)), float(rot.get("base", 1.0)), positions), eps)
    share = heads // kv_heads
    out = torch.zeros(length, heads, vdim, dtype=F)
    causal = positions[None, :] <= positions[:, None]
    for head in range(heads):
        score = capped((q[:, head] @ k[:, head // share].T) * mixer["scale"], float(mixer.get("softcap", 0.0)))
        score = torch.where(causal, score, torch.tensor(-math.inf, dtype=F))
        sink = w[prefix + "sink"][head]
        top = torch.maximum(score.max(-1, keepdim=True).values, sink)
        weight = torch.exp(score - top)
        weight = weight / (weight.sum(-1, keepdim=True) + torch.exp(sink - top))
        out[:, head] = weight @ v[:, head // share]
    return out.reshape(length, heads * vdim) @ w[prefix + "o"].T, own


def lightning(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head: ``S <- decay S + k v^T; o = S^T q``; the heads side by
    side are normed together, gated by ``sigmoid(W_g h)`` and projected."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    q = silu(h @ w[prefix + "q"].T).view(length, heads, dim)
    k = silu(h @ w[prefix + "k"].T).view(length, heads, dim)
    v = silu(h @ w[prefix + "v"].T).view(length, heads, vdim)
    out = torch.zeros(length, heads, vdim, dtype=F)
    for head in range(heads):
        state = torch.zeros(dim, vdim, dtype=F)
        for t in range(length):
            state = float(mixer["decay"][head]) * state + torch.outer(k[t, head], v[t, head])
            out[t, head] = state.T @ q[t, head]
    normed = rms_norm(out.reshape(length, heads * vdim), eps, w[prefix + "norm"])
    return (normed * torch.sigmoid(h @ w[prefix + "g"].T)) @ w[prefix + "o"].T


# ------------------------------------------------------------------ feed-forwards
def clamped_glu(h: torch.Tensor, w: dict, prefix: str, limit: float) -> torch.Tensor:
    """``down(g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(gate h, limit)``, ``u = clamp(up h, +-limit)``."""
    g = torch.clamp(h @ w[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ w[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[prefix + "down"].T


def silu_glu(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def router_scores(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    return torch.sigmoid(h @ w[prefix + "router"].T)


def routed_experts(h: torch.Tensor, w: dict, prefix: str, mlp: dict, margins: list | None = None) -> torch.Tensor:
    """Each token runs its ``top`` best experts on ``score * h`` (the score scales the input, scores are not
    renormalised); a shared expert runs for every token, times ``sigmoid(sg h)``.  ``margins`` receives, per
    token, the gap between the last chosen and the first unchosen router logit over the logits' spread."""
    top = int(mlp["router"]["top"])
    scores = router_scores(h, w, prefix)
    if margins is not None and top < scores.shape[1]:
        logits = torch.sort(h @ w[prefix + "router"].T, dim=-1, descending=True).values
        margins.extend(((logits[:, top - 1] - logits[:, top]) / (logits.std(-1) + 1e-9)).tolist())
    # the largest scores are the largest logits; choosing on the logits keeps large ones apart that the sigmoid,
    # in any float format, rounds to the same 1.0
    chosen = torch.topk(h @ w[prefix + "router"].T, top, dim=-1).indices
    out = torch.zeros(h.shape[0], w[prefix + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += silu_glu((scores[t, e] * h[t])[None], w, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        out = out + silu_glu(h, w, prefix + "shared.") * torch.sigmoid(h @ w[prefix + "shared.sg"].T)
    return out


def feed_forward(h: torch.Tensor, w: dict, prefix: str, mlp: dict, margins: list | None = None) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return clamped_glu(h, w, prefix, float(mlp["limit"]))
    return routed_experts(h, w, prefix, mlp, margins)


# ------------------------------------------------------------------ the model
def forward(config: dict, w: dict, tokens, collect: list | None = None, margins: list | None = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence; ``collect`` receives the stream after every layer, ``margins`` how
    clearly every router decision fell (see :func:`routed_experts`)."""
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    first_values = None
    for index, layer in enumerate(config["layers"]):
        prefix, mixer = f"l{index}.", layer["mixer"]
        if layer["type"] == "attention":
            is_first = bool(mixer.get("v_mix")) and first_values is None
            mixed, own = softmax_attention(x, w, prefix + "mix.", mixer, eps, first_values, is_first)
            if is_first:
                first_values = own
        elif layer["type"] == "lightning":
            mixed = lightning(x, w, prefix + "mix.", mixer, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(mixed, eps, w[prefix + "norm1"])
        if layer.get("mlp") is not None:
            x = x + rms_norm(feed_forward(x, w, prefix + "mlp.", layer["mlp"], margins), eps, w[prefix + "norm2"])
        if collect is not None:
            collect.append(x.clone())
    return rms_norm(x, eps, w["final.norm"]) @ w["head"].T


def greedy(config: dict, w: dict, prompt, steps: int) -> list[int]:
    """The ``steps`` tokens that always taking the largest logit produces after ``prompt``."""
    tokens = list(prompt)
    for _ in range(steps):
        tokens.append(int(forward(config, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]


def clear_margin(config: dict, w: dict, tokens) -> float:
    """The narrowest router decision of the sequence (infinite for a model without routers)."""
    margins: list = []
    forward(config, w, tokens, margins=margins)
    return min(margins) if margins else math.inf
