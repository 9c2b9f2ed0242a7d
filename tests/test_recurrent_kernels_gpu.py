"""The kernels of the recurrent mixers, each alone, against plain float64 restatements."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch
from plain_kopatar import causal_conv, rotate_halves, silu, softplus, unit_rms, xielu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _batch(lengths, slots, starts):
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=DEV)
    return SimpleNamespace(
        cu_seqlens=cu, entry_slot=torch.tensor(slots, dtype=torch.int32, device=DEV),
        entry_start=torch.tensor(starts, dtype=torch.int32, device=DEV), num_entries=len(lengths),
        fault=torch.zeros(1, dtype=torch.int32, device=DEV),
    )


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [1, 2, 4])
def test_short_convolution_over_steps_of_any_length(dtype, width):
    """Two requests fed in steps of 1, 2 and more tokens (fewer than the taps reach back, too); the tail kept in the
    slot carries each over; a slot that changes hands starts from zeros whatever it holds."""
    from rapid_llm_b200.ops import kernels

    channels, slots = 10, 3
    generator = torch.Generator().manual_seed(width)
    taps = torch.randn(channels, width, generator=generator)
    bias = torch.randn(channels, generator=generator)
    sequences = [torch.randn(n, channels + 4, generator=generator).to(dtype) for n in (23, 17)]
    want = [silu(causal_conv(s[:, 2 : 2 + channels].double(), taps.double(), bias.double())) for s in sequences]
    tail = torch.full((slots, (width - 1) * channels + 5), 7.0, device=DEV)      # garbage: position 0 must not read it
    cuts = [[1, 2, 1, 5, 3, 1, 1, 9], [2, 1, 1, 1, 6, 4, 2]]
    fed, got = [0, 0], [[], []]
    for step in range(max(len(c) for c in cuts)):
        live = [i for i in (0, 1) if step < len(cuts[i])]
        lengths = [cuts[i][step] for i in live]
        rows = torch.cat([sequences[i][fed[i] : fed[i] + n] for i, n in zip(live, lengths)]).to(DEV)
        out = torch.empty(rows.shape[0], channels, device=DEV)
        batch = _batch(lengths, [2 - i for i in live], [fed[i] for i in live])
        kernels.causal_conv_silu(rows[:, 2 : 2 + channels], taps.to(DEV), bias.to(DEV), tail[:, 5:], out, batch)
        at = 0
        for i, n in zip(live, lengths):
            got[i].append(out[at : at + n].cpu())
            at, fed[i] = at + n, fed[i] + n
        assert int(batch.fault.item()) == 0
    for i in (0, 1):
        torch.testing.assert_close(torch.cat(got[i]).double(), want[i], rtol=1e-5, atol=1e-5)
    assert torch.all(tail[:, :5] == 7.0)


def _plain_scan(q, k, v, decay, beta, v_scale, skip, heads, kv_heads, dim, vdim):
    length = q.shape[0]
    out = torch.zeros(length, heads, vdim, dtype=torch.float64)
    q, k, v = q.view(length, kv_heads, dim), k.view(length, kv_heads, dim), v.view(length, heads, vdim)
    for h in range(heads):
        S = torch.zeros(dim, vdim, dtype=torch.float64)
        for t in range(length):
            kh = h // (heads // kv_heads)
            if decay.dim() == 1:
                S = decay[h] * S
            elif decay.shape[1] == heads:
                S = decay[t, h] * S
            else:
                S = decay[t].view(heads, dim)[h].unsqueeze(1) * S
            if beta is not None:
                u = beta[t, h] * (v[t, h] - S.T @ k[t, kh])
            else:
                u = v[t, h] * (1.0 if v_scale is None else v_scale[t, h])
            S = S + torch.outer(k[t, kh], u)
            out[t, h] = S.T @ q[t, kh] + (0.0 if skip is None else skip[h]) * v[t, h]
    return out.view(length, heads * vdim)


@pytest.mark.parametrize("dim,vdim,heads,kv_heads", [(20, 7, 4, 2), (64, 64, 2, 2), (128, 48, 2, 1), (5, 130, 3, 3), (300, 16, 1, 1)])
@pytest.mark.parametrize("kind", ["fixed", "per_token", "per_row_delta", "per_token_scaled_skip"])
def test_the_recurrence_over_steps_and_slots(kind, dim, vdim, heads, kv_heads):
    from rapid_llm_b200.ops import kernels

    generator = torch.Generator().manual_seed(dim + vdim)
    lengths_total = (37, 12)
    data = []
    fixed = torch.rand(heads, generator=generator) * 0.2 + 0.8
    skips = torch.randn(heads, generator=generator)
    for n in lengths_total:
        q, k = torch.randn(n, kv_heads * dim, generator=generator) / dim ** 0.5, torch.randn(n, kv_heads * dim, generator=generator)
        v = torch.randn(n, heads * vdim, generator=generator)
        beta = v_scale = skip = None
        if kind == "fixed":
            decay = fixed
        elif kind == "per_token":
            decay = torch.rand(n, heads, generator=generator) * 0.5 + 0.5
        elif kind == "per_row_delta":
            decay = torch.rand(n, heads * dim, generator=generator) * 0.3 + 0.7
            beta = torch.rand(n, heads, generator=generator)
            k = k / k.view(n, kv_heads, dim).norm(dim=-1).repeat_interleave(dim, dim=1)
        else:
            decay = torch.rand(n, heads, generator=generator) * 0.5 + 0.5
            v_scale, skip = torch.rand(n, heads, generator=generator), skips
        data.append((q, k, v, decay, beta, v_scale, skip))
    want = [_plain_scan(*(None if t is None else t.double() for t in item), heads, kv_heads, dim, vdim) for item in data]
    state = torch.full((3, heads * dim * vdim + 3), float("nan"), device=DEV)      # position 0 must not read it
    cuts = [[5, 1, 1, 17, 2, 11], [1, 1, 10]]
    fed, got = [0, 0], [[], []]
    for step in range(max(len(c) for c in cuts)):
        live = [i for i in (0, 1) if step < len(cuts[i])]
        lengths = [cuts[i][step] for i in live]
        batch = _batch(lengths, [i + 1 for i in live], [fed[i] for i in live])

        def rows(index):
            if data[0][index] is None:
                return None
            return torch.cat([data[i][index][fed[i] : fed[i] + n] for i, n in zip(live, lengths)]).to(DEV).contiguous()

        q, k, v = rows(0), rows(1), rows(2)
        decay = data[0][3].to(DEV) if kind == "fixed" else rows(3)
        skip = None if data[0][6] is None else data[0][6].to(DEV)
        out = torch.empty(v.shape, device=DEV)
        kernels.linear_scan(q, k, v, decay, out, state[:, 3:], batch, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                            beta=rows(4), v_scale=rows(5), skip=skip)
        assert int(batch.fault.item()) == 0
        at = 0
        for i, n in zip(live, lengths):
            got[i].append(out[at : at + n].cpu())
            at, fed[i] = at + n, fed[i] + n
    for i in (0, 1):
        torch.testing.assert_close(torch.cat(got[i]).double(), want[i], rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_gate_in_their_three_orders(dtype):
    from rapid_llm_b200.ops import kernels

    generator = torch.Generator().manual_seed(0)
    tokens, groups, size = 5, 3, 20
    y = torch.randn(tokens, groups * size, generator=generator)
    gate = torch.randn(tokens, groups * size + 6, generator=generator).to(dtype)
    g = gate[:, 6:].double()
    per_group, whole = torch.randn(size, generator=generator), torch.randn(groups * size, generator=generator)
    yd = y.double().view(tokens, groups, size)
    cases = [
        (dict(act=kernels.GATE_SIGMOID, weight=per_group.to(DEV), eps=1e-5),
         (unit_rms(yd, 1e-5) * per_group.double()).reshape(tokens, -1) * torch.sigmoid(g)),
        (dict(act=kernels.GATE_SILU, eps=1e-6), unit_rms(yd, 1e-6).reshape(tokens, -1) * silu(g)),
        (dict(act=kernels.GATE_SILU, gate_first=True, weight=whole.to(DEV), eps=1e-5),
         unit_rms((y.double() * silu(g)).view(tokens, groups, size), 1e-5).reshape(tokens, -1) * whole.double()),
    ]
    for options, want in cases:
        out = torch.empty(tokens, groups * size, dtype=dtype, device=DEV)
        kernels.gated_norm(y.to(DEV), out, group=size, gate=gate.to(DEV)[:, 6:], **options)
        tolerance = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(out.double().cpu(), want, **tolerance)
    # the gate alone, on rows of the engine's dtype (an attention's output gate)
    rows = y.to(dtype)
    out = torch.empty_like(rows, device=DEV)
    kernels.gated_norm(rows.to(DEV), out, group=groups * size, gate=gate.to(DEV)[:, 6:], act=kernels.GATE_SIGMOID, norm=False)
    torch.testing.assert_close(out.double().cpu(), rows.double() * torch.sigmoid(g), rtol=1e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-6)


def test_activation_decays_unit_heads_and_rotation():
    from rapid_llm_b200.ops import kernels

    generator = torch.Generator().manual_seed(1)
    z = torch.randn(7, 33, generator=generator) * 3
    pq = torch.tensor([0.3, -0.8])
    out = torch.empty_like(z, device=DEV)
    kernels.xielu(z.to(DEV), out, pq.to(DEV))
    torch.testing.assert_close(out.cpu().double(), xielu(z.double(), pq[0].double(), pq[1].double()), rtol=1e-5, atol=1e-6)

    heads, per, tokens = 3, 4, 6
    x = torch.randn(tokens, heads * per + 2, generator=generator) * 2
    a_log, bias = torch.randn(heads, generator=generator), torch.randn(heads * per, generator=generator)
    decay, step = torch.empty(tokens, heads * per, device=DEV), torch.empty(tokens, heads * per, device=DEV)
    kernels.decay_gate(x.to(DEV)[:, 2:], torch.exp(a_log).to(DEV), bias.to(DEV), per, decay, step)
    dt = softplus(x[:, 2:].double() + bias.double())
    torch.testing.assert_close(step.cpu().double(), dt, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(decay.cpu().double(), torch.exp(-torch.exp(a_log.double()).repeat_interleave(per) * dt), rtol=1e-5, atol=1e-6)

    dim = 12
    rows = torch.randn(tokens, 1 + 4 * dim, generator=generator)
    raw = torch.randn(tokens, 5, generator=generator)
    work, gates = rows.to(DEV), torch.empty(tokens, 3, device=DEV)
    kernels.unit_heads(work[:, 1:], heads=4, dim=dim, eps=1e-6, split=2, scale_low=dim ** -0.5, scale_high=1.0,
                       gate_in=raw.to(DEV)[:, 2:], gate_out=gates)
    v = rows[:, 1:].double().view(tokens, 4, dim)
    want = v / torch.sqrt((v * v).sum(-1, keepdim=True) + 1e-6)
    want[:, :2] *= dim ** -0.5
    torch.testing.assert_close(work[:, 1:].cpu().double(), want.reshape(tokens, -1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(gates.cpu().double(), torch.sigmoid(raw[:, 2:].double()), rtol=1e-5, atol=1e-6)
    assert torch.equal(work[:, 0].cpu(), rows[:, 0])

    heads, dim, vdim, rot, base = 2, 10, 6, 6, 50.0
    proj = torch.randn(tokens, 2 * heads * dim + heads * vdim + 3, generator=generator)
    positions = torch.tensor([0, 1, 2, 900, 31, 7], dtype=torch.int32)
    inv_freq = 1.0 / (torch.tensor(base) ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    out = torch.empty(tokens, 2 * heads * dim + heads * vdim, device=DEV)
    on = proj.to(DEV)
    hd = heads * dim
    kernels.rotate_heads(on[:, 3 : 3 + hd], on[:, 3 + hd : 3 + 2 * hd], on[:, 3 + 2 * hd :], out, positions.to(DEV), inv_freq.to(DEV),
                         heads=heads, dim=dim, vdim=vdim, k_scale=0.25)
    q = rotate_halves(proj[:, 3 : 3 + hd].double().view(tokens, heads, dim), positions, rot, base).reshape(tokens, -1)
    k = rotate_halves(proj[:, 3 + hd : 3 + 2 * hd].double().view(tokens, heads, dim), positions, rot, base).reshape(tokens, -1) * 0.25
    torch.testing.assert_close(out.cpu().double(), torch.cat([q, k, proj[:, 3 + 2 * hd :].double()], dim=1), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("hidden", [64, 60])
def test_the_norm_takes_addends_into_the_stream(hidden):
    from rapid_llm_b200.ops import kernels

    generator = torch.Generator().manual_seed(2)
    tokens = 5
    x, residual, rows = (torch.randn(tokens, hidden, generator=generator) for _ in range(3))
    vector, weight = torch.randn(hidden, generator=generator), torch.randn(hidden, generator=generator)
    stream = residual.to(DEV)
    out = torch.empty(tokens, hidden, device=DEV)
    kernels.add_rmsnorm(x.to(DEV), stream, weight.to(DEV), out, 1e-5, mode=1, write_residual=True,
                        extra_rows=rows.to(DEV), extra_vector=vector.to(DEV))
    total = x.double() + residual.double() + rows.double() + vector.double()
    torch.testing.assert_close(stream.cpu().double(), total, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out.cpu().double(), unit_rms(total, 1e-5) * weight.double(), rtol=1e-5, atol=1e-5)
