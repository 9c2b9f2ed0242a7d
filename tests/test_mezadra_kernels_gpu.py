"""The kernels that came with the Mezadra decoder, one by one, against plain PyTorch float32."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"


def _silu(x):
    return x * torch.sigmoid(x)


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,top,hidden,inter", [(300, 40, 3, 64, 24), (37, 5, 2, 50, 22), (1, 3, 3, 32, 8), (200, 1, 1, 40, 16),
                                                             (150, 2, 2, 200, 72)])
def test_products_over_pairs_grouped_by_expert(tokens, experts, top, hidden, inter, dtype, wide):
    """Given choices and weights, plan + gated product + down product + sum equal the experts run pair by pair; on the
    plain tiles and on the pipelined bfloat16 ones (``wide``; inner sizes that are no multiples of their chunk too)."""
    from rapid_llm_b200.ops import kernels

    if wide and not kernels.moe_wide_takes(dtype, hidden, inter):
        pytest.skip("the pipelined tiles take bfloat16 with 16-byte rows")

    g = torch.Generator().manual_seed(tokens + experts)
    x = torch.randn(tokens, hidden, generator=g).to(dtype).to(DEVICE)
    gate_up = (torch.randn(experts, 2 * inter, hidden, generator=g) / hidden ** 0.5).to(dtype).to(DEVICE)
    down = (torch.randn(experts, hidden, inter, generator=g) / inter ** 0.5).to(dtype).to(DEVICE)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).to(torch.int32).to(DEVICE)
    weights = torch.rand(tokens, top, generator=g).to(DEVICE)
    shared = torch.randn(tokens, hidden, generator=g).to(dtype).to(DEVICE)
    gate = torch.rand(tokens, 1, generator=g).to(DEVICE)
    fault = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    pairs = tokens * top
    order = torch.empty(pairs, dtype=torch.int32, device=DEVICE)
    place = torch.empty(pairs, dtype=torch.int32, device=DEVICE)
    meta = torch.zeros(1 + 3 * kernels.moe_max_tiles(pairs, experts, wide), dtype=torch.int32, device=DEVICE)
    max_tiles = kernels.moe_plan(ids, experts, order, place, meta, fault, wide=wide)
    act = torch.empty(pairs, inter, dtype=dtype, device=DEVICE)
    kernels.grouped_linear(x, gate_up, order, meta, top=top, by_token=True, max_tiles=max_tiles, pair_weight=weights.view(-1), out_act=act, wide=wide)
    each = torch.full((pairs, hidden), float("nan"), device=DEVICE)
    kernels.grouped_linear(act, down, order, meta, top=top, by_token=False, max_tiles=max_tiles, out_y=each, wide=wide)
    out = torch.empty(tokens, hidden, dtype=dtype, device=DEVICE)
    kernels.moe_combine(each, top, out, shared=shared, gate=gate)
    assert int(fault.item()) == 0
    # every pair has one place, and the places of an expert are consecutive
    assert sorted(order.tolist()) == list(range(pairs))
    assert torch.equal(order[place.long()].cpu(), torch.arange(pairs, dtype=torch.int32))
    by_place = ids.view(-1)[order.long()].tolist()
    assert by_place == sorted(by_place)
    want = torch.zeros(tokens, hidden, device=DEVICE)
    xf, wf, df = x.float(), gate_up.float(), down.float()
    for t in range(tokens):
        for j in range(top):
            e, w = int(ids[t, j]), weights[t, j]
            wide = wf[e] @ xf[t]
            a = _silu(w * wide[:inter]) * (w * wide[inter:])
            if dtype == torch.bfloat16:
                a = a.to(dtype).float()
            want[t] += df[e] @ a
    want += gate * shared.float()
    bound = {"rtol": 1e-4, "atol": 1e-5} if dtype == torch.float32 else {"rtol": 2e-2, "atol": 2e-2}
    torch.testing.assert_close(out.float(), want, **bound)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,gates,hidden", [(12, 1, 1, 64), (40, 3, 0, 50), (2, 2, 2, 33), (70, 8, 1, 128)])
def test_router_scores_choices_and_gates(experts, top, gates, hidden, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(experts)
    tokens = 45
    x = (4 * torch.randn(tokens, hidden, generator=g)).to(dtype).to(DEVICE)
    w = torch.randn(experts + gates, hidden, generator=g).to(DEVICE)
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEVICE)
    weights = torch.empty(tokens, top, device=DEVICE)
    gate_out = torch.empty(tokens, gates, device=DEVICE) if gates else None
    scores = torch.empty(tokens, experts, device=DEVICE)
    kernels.router_topk(x, w, experts=experts, top=top, ids=ids, weights=weights, gates=gate_out, scores=scores)
    logits = x.double() @ w.double().T
    want = torch.topk(logits[:, :experts], top, dim=-1)
    assert torch.equal(ids.long().cpu(), want.indices.cpu())       # large logits: sigmoid saturates, the order must not
    torch.testing.assert_close(weights.double(), torch.sigmoid(want.values), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(scores.double(), torch.sigmoid(logits[:, :experts]), rtol=1e-5, atol=1e-6)
    if gates:
        torch.testing.assert_close(gate_out.double(), torch.sigmoid(logits[:, experts:]), rtol=1e-5, atol=1e-6)


def test_equal_logits_go_to_the_lower_index():
    from rapid_llm_b200.ops import kernels

    x = torch.ones(3, 8, device=DEVICE)
    w = torch.zeros(6, 8, device=DEVICE)
    w[4], w[1] = 0.5, 0.5
    ids = torch.empty(3, 3, dtype=torch.int32, device=DEVICE)
    weights = torch.empty(3, 3, device=DEVICE)
    kernels.router_topk(x, w, experts=6, top=3, ids=ids, weights=weights)
    assert ids.tolist() == [[1, 4, 0]] * 3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [64, 50, 1032])
def test_a_norm_that_joins_the_stream_and_the_norm_of_the_stream(hidden, dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(hidden)
    y = torch.randn(9, hidden, generator=g).to(dtype).to(DEVICE)
    stream = (5 * torch.randn(9, hidden, generator=g)).to(DEVICE)
    weight = (1 + 0.2 * torch.randn(hidden, generator=g)).to(DEVICE)
    before = stream.clone()
    out = torch.empty(9, hidden, dtype=dtype, device=DEVICE)
    kernels.join_rmsnorm(y, stream, weight, out, 1e-5)
    yf = y.float()
    want = before + yf * torch.rsqrt((yf * yf).mean(-1, keepdim=True) + 1e-5) * weight
    torch.testing.assert_close(stream, want, rtol=1e-5, atol=1e-5)
    assert torch.equal(out, stream.to(dtype))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEVICE)
    normed = torch.empty(3, hidden, dtype=dtype, device=DEVICE)
    kernels.stream_rmsnorm(stream, weight, normed, 1e-5, rows)
    picked = stream[rows.long()]
    want = picked * torch.rsqrt((picked * picked).mean(-1, keepdim=True) + 1e-5) * weight
    torch.testing.assert_close(normed.float(), want, **({"rtol": 1e-5, "atol": 1e-5} if dtype == torch.float32 else {"rtol": 1e-2, "atol": 1e-2}))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_clamped_gated_unit_and_the_scaled_embedding(dtype):
    from rapid_llm_b200.ops import kernels

    g = torch.Generator().manual_seed(2)
    wide = (2 * torch.randn(11, 2 * 37, generator=g)).to(dtype).to(DEVICE)
    out = torch.empty(11, 37, dtype=dtype, device=DEVICE)
    kernels.clamped_glu(wide, out, 0.8, 1.702)
    gate, up = wide.float()[:, :37].clamp(max=0.8), wide.float()[:, 37:].clamp(-0.8, 0.8)
    want = gate * torch.sigmoid(1.702 * gate) * (up + 1)
    torch.testing.assert_close(out.float(), want, **({"rtol": 1e-5, "atol": 1e-6} if dtype == torch.float32 else {"rtol": 1e-2, "atol": 1e-2}))
    table = torch.randn(20, 24, generator=g).to(dtype).to(DEVICE)
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32, device=DEVICE)
    rows = torch.empty(4, 24, dtype=dtype, device=DEVICE)
    stream = torch.empty(4, 24, device=DEVICE)
    fault = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    kernels.embedding(rows, table, ids, fault, scale=13.5, stream=stream)
    assert torch.equal(stream, table[ids.long()].float() * 13.5) and torch.equal(rows, stream.to(dtype)) and int(fault.item()) == 0


@pytest.mark.parametrize("tokens", [5, 64, 300, 1100])
def test_the_clamped_unit_rides_on_the_gate_up_product(tokens):
    """Small steps: the streaming tcgen05 product's epilogue; a thousand tokens and more: the pair kernel's; between
    them the library product and the unit's own kernel.  All against float32 arithmetic on the same bfloat16 operands."""
    from rapid_llm_b200.engine.batch import Workspace
    from rapid_llm_b200.ops import gemm

    g = torch.Generator().manual_seed(tokens)
    hidden, inter, limit, alpha = 256, 384, 0.8, 1.702
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(DEVICE)
    w = (2 * torch.randn(2 * inter, hidden, generator=g) / hidden ** 0.5).to(torch.bfloat16).to(DEVICE)
    fault = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    act = torch.empty(tokens, inter, dtype=torch.bfloat16, device=DEVICE)
    gemm.gated_linear(x, w, act, Workspace(tokens, torch.device(DEVICE)), fault, clamp=(limit, alpha))
    wide = x.float() @ w.float().T
    gate, up = wide[:, :inter].clamp(max=limit), wide[:, inter:].clamp(-limit, limit)
    want = gate * torch.sigmoid(alpha * gate) * (up + 1)
    assert int(fault.item()) == 0
    assert float((gate == limit).float().mean()) > 0.05 and float((up.abs() == limit).float().mean()) > 0.05      # the limits bite
    torch.testing.assert_close(act.float(), want, rtol=2e-2, atol=2e-2)
