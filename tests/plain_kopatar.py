"""A plain, slow restatement of the Kopatar decoder, one function per mechanism.

Everything runs token by token on the CPU in float64 over whole sequences: no cache, no
state carried between calls, no batching.  It shares no code with the package; the tests
compare the engine's logits, and single mixers, with it.

Notation: ``x`` is ``[T, width]``, weights are ``[out, in]`` and applied as ``x @ W.T``;
``w`` maps tensor names (``l0.mix.q`` ...) to float64 tensors; ``layer`` is one entry of the
configuration's ``layers``.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``y[t, c] = sum_d taps[c, last - d] * x[t - d, c]`` with zeros before the sequence."""
    length, width = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(length):
        for d in range(width):
            if t - d >= 0:
                y[t] += taps[:, width - 1 - d] * x[t - d]
    if bias is not None:
        y = y + bias
    return y


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    positive = softplus(p) * z * z + z / 2
    negative = (0.5 + softplus(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1 - z) + z / 2
    return torch.where(z > 0, positive, negative)


def dense_feed_forward(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    act = w[prefix + "act"]
    return xielu(h @ w[prefix + "up"].T, act[0], act[1]) @ w[prefix + "down"].T


# ------------------------------------------------------------------ mixers
def channel_delta(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    """Delta rule with one decay per head and key channel."""
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    q = silu(causal_conv(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).view(length, kv_heads, dim)
    k = silu(causal_conv(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).view(length, kv_heads, dim)
    v = silu(causal_conv(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).view(length, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)
    rate = softplus((h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "dt_bias"]).view(length, heads, dim)
    decay = torch.exp(-torch.exp(w[prefix + "A_log"]).view(1, heads, 1) * rate)
    gate = torch.sigmoid((h @ w[prefix + "g1"].T) @ w[prefix + "g2"].T).view(length, heads, vdim)
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    share = heads // kv_heads
    for head in range(heads):
        state = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(length):
            key, query = k[t, head // share], q[t, head // share]
            state = decay[t, head].unsqueeze(1) * state
            update = beta[t, head] * (v[t, head] - state.T @ key)
            state = state + torch.outer(key, update)
            out[t, head] = state.T @ query
    out = unit_rms(out, eps) * w[prefix + "norm"] * gate
    return out.reshape(length, heads * vdim) @ w[prefix + "o"].T


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotation of the first ``dims`` entries of every head, entry i paired with i + dims / 2."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    angle = positions.to(x.dtype).view(-1, 1, 1) * freq
    cos, sin = torch.cos(angle), torch.sin(angle)
    first, second = x[..., :half], x[..., half:dims]
    return torch.cat([first * cos - second * sin, second * cos + first * sin, x[..., dims:]], dim=-1)


def retention(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    positions = torch.arange(length)
    q = (h @ w[prefix + "q"].T).view(length, heads, dim)
    k = (h @ w[prefix + "k"].T).view(length, heads, dim)
    v = (h @ w[prefix + "v"].T).view(length, heads, vdim)
    rot = mixer.get("rot")
    if rot:
        q = rotate_halves(q, positions, rot["dims"], rot["base"])
        k = rotate_halves(k, positions, rot["dims"], rot["base"])
    k = k * dim ** -0.5
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        state = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(length):
            state = mixer["decay"][head] * state + torch.outer(k[t, head], v[t, head])
            out[t, head] = state.T @ q[t, head]
    out = unit_rms(out, eps).reshape(length, heads * vdim) * silu(h @ w[prefix + "g"].T)
    return out @ w[prefix + "o"].T


def windowed_attention(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    """Softmax attention without positions over the last ``mask.size`` tokens, with an output gate."""
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    length = h.shape[0]
    q = unit_rms((h @ w[prefix + "q"].T).view(length, heads, dim), eps) * w[prefix + "q.norm"]
    k = unit_rms((h @ w[prefix + "k"].T).view(length, kv_heads, dim), eps) * w[prefix + "k.norm"]
    v = (h @ w[prefix + "v"].T).view(length, kv_heads, vdim)
    window = mixer["mask"]["size"]
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    share = heads // kv_heads
    for head in range(heads):
        for t in range(length):
            first = max(0, t - window + 1)
            scores = (k[first : t + 1, head // share] @ q[t, head]) * mixer["scale"]
            out[t, head] = torch.softmax(scores, dim=0) @ v[first : t + 1, head // share]
    out = out.reshape(length, heads * vdim) * torch.sigmoid(h @ w[prefix + "g"].T)
    return out @ w[prefix + "o"].T


def state_space(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    """Selective state space with a scalar decay per head (the dual form's recurrence)."""
    heads, vdim, state_size, groups = mixer["heads"], mixer["vdim"], mixer["state"], mixer["groups"]
    inner, length = heads * vdim, h.shape[0]
    projected = h @ w[prefix + "in"].T
    z = projected[:, :inner]
    mixed = projected[:, inner : 2 * inner + 2 * groups * state_size]
    dt = projected[:, 2 * inner + 2 * groups * state_size :]
    mixed = silu(causal_conv(mixed, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = mixed[:, :inner].view(length, heads, vdim)
    b = mixed[:, inner : inner + groups * state_size].view(length, groups, state_size)
    c = mixed[:, inner + groups * state_size :].view(length, groups, state_size)
    dt = softplus(dt + w[prefix + "dt_bias"])
    rate = torch.exp(w[prefix + "A_log"])
    y = torch.zeros(length, heads, vdim, dtype=h.dtype)
    share = heads // groups
    for head in range(heads):
        state = torch.zeros(state_size, vdim, dtype=h.dtype)
        for t in range(length):
            state = torch.exp(-rate[head] * dt[t, head]) * state + dt[t, head] * torch.outer(b[t, head // share], x[t, head])
            y[t, head] = state.T @ c[t, head // share] + w[prefix + "D"][head] * x[t, head]
    y = y.reshape(length, inner) * silu(z)
    parts = mixer["norm_groups"]
    y = unit_rms(y.view(length, parts, inner // parts), eps).reshape(length, inner) * w[prefix + "norm"]
    return y @ w[prefix + "o"].T


def parallel(h: torch.Tensor, w: dict, prefix: str, mixer: dict, eps: float) -> torch.Tensor:
    left = windowed_attention(h, w, prefix + "left.", mixer["left"], eps)
    right = state_space(h, w, prefix + "right.", mixer["right"], eps)
    return mixer["left_scale"] * left + mixer["right_scale"] * right


MIXERS = {"channel_delta": channel_delta, "retention": retention, "parallel": parallel}


# ------------------------------------------------------------------- model
def run_order(config: dict) -> list[tuple[int, int | None]]:
    """``(layer, pass number or None)``; the pass number is given at the first layer of a pass."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    order: list[tuple[int, int | None]] = [(i, None) for i in range(loop["start"])]
    for number in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, number if i == loop["start"] else None))
    order.extend((i, None) for i in range(loop["stop"], count))
    return order


def forward(config: dict, w: dict, tokens: list[int], keep_layers: bool = False):
    """Logits ``[T, vocab]`` of one whole sequence (and the stream after every layer run)."""
    eps = config["norm"]["eps"]
    embedded = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = embedded.clone()
    after = []
    for index, number in run_order(config):
        if number is not None:
            if number > 0:
                x = x + embedded
            x = x + w["loop.step"][number]
        layer, prefix = config["layers"][index], f"l{index}."
        x = x + MIXERS[layer["type"]](unit_rms(x, eps) * w[prefix + "norm1"], w, prefix + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + dense_feed_forward(unit_rms(x, eps) * w[prefix + "norm2"], w, prefix + "mlp.")
        after.append(x)
    logits = (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T
    return (logits, torch.stack(after)) if keep_layers else logits


def greedy(config: dict, w: dict, prompt: list[int], count: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(forward(config, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
