"""Prefill and decode throughput of Mezadra models at layer sizes of real models, beside Qwen3 of equal size, and
the kernels that came with the design alone against their rooflines.

    python bench.py --workload mezadra [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.mezadra_compare [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.mezadra_compare --alone --sizes 2048      # the kernels a few times each, for ncu

Random weights, bfloat16, one GPU.  A model of width ``W`` has six layers, ``lightning, attention, lightning,
lightning, attention, lightning`` with the feed-forwards ``dense, experts, dense, experts, dense, experts``: heads of
128 (attention: a kv head per four heads, four taps, 32 rotated entries, a cap of 30), a dense
feed-forward of ``8 W / 3`` (rounded to 256), 16 experts of ``W / 4`` of which a token takes two, and a shared expert
of ``W / 2``.  The Qwen3 beside it has six layers.  Prefill is one 2,048-token step (best of three, CUDA events around
the step function); decode is batch 8 behind 1,024-token prompts, replayed from the captured graph (median of 32
steps).  Kernels are timed alone with CUDA events, L2 flushed between runs (a write of 256 MB), on one 2,048-token
prompt and on 64 single tokens behind 1,024 cached ones; ``frac`` is (bytes the kernel must move) / time / measured
copy bandwidth, ``tflops`` the products' arithmetic over the same time.
"""

from __future__ import annotations

import argparse
import json
import statistics
from types import SimpleNamespace

import torch

from .recurrent_compare import PREFILL, _events, model_figures, qwen3_raw

EXPERTS, TOP = 16, 2


def mezadra_raw(width: int) -> dict:
    heads = width // 128
    lightning = {"heads": heads, "dim": 128, "vdim": 128,
                 "decay": [1.0 - 2.0 ** (-3 - 7 * h / max(heads - 1, 1)) for h in range(heads)]}
    attention = {"heads": heads, "kv_heads": max(heads // 4, 1), "dim": 128, "vdim": 128, "conv": 4,
                 "rot": {"dims": 32, "base": 1.0e6}, "scale": 128 ** -0.5, "softcap": 30.0, "v_mix": True}
    dense = {"kind": "dense", "ff": (8 * width // 3 + 255) // 256 * 256, "limit": 7.0}
    experts = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP}, "expert": {"ff": width // 4},
               "shared": {"ff": width // 2}}
    order = [("lightning", lightning, dense), ("attention", attention, experts), ("lightning", lightning, dense),
             ("lightning", lightning, experts), ("attention", attention, dense), ("lightning", lightning, experts)]
    return {"architecture": "Mezadra", "vocab": 32000, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"scale": float(width) ** 0.5},
            "layers": [{"type": kind, "mixer": dict(mixer), "mlp": dict(mlp)} for kind, mixer, mlp in order]}


def kernel_figures(width: int, hbm_gbs: float) -> dict:
    """The design's own kernels alone, on a 2,048-token prompt and on 64 single tokens."""
    from . import kernels

    device = "cuda:0"
    heads, kv_heads, d, inter = width // 128, max(width // 512, 1), 128, width // 4
    flush = torch.empty(64 << 20, dtype=torch.float32, device=device)
    out = {}

    def timed(label, tokens, entries, moved, run, flops=0.0):
        times = []
        for _ in range(5):
            flush.zero_()
            begin, end = _events()
            begin.record()
            run()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1e3)
        us = statistics.median(times[1:])
        row = {"us": round(us, 1), "mb": round(moved / 1e6, 2), "frac": round(moved / (us * 1e-6) / (hbm_gbs * 1e9), 3)}
        if flops:
            row["tflops"] = round(flops / (us * 1e-6) / 1e12, 1)
        out[f"{label} ({'prompt of ' + str(tokens) if entries == 1 else str(entries) + ' single tokens'})"] = row

    bf = lambda *shape: torch.randn(*shape, device=device).to(torch.bfloat16)      # noqa: E731
    f32 = lambda *shape: torch.randn(*shape, device=device)                        # noqa: E731
    fault = torch.zeros(1, dtype=torch.int32, device=device)
    page, context = 16, 1024
    for tokens, entries in ((PREFILL, 1), (64, 64)):
        per = tokens // entries
        start = 0 if entries == 1 else context
        batch = SimpleNamespace(
            cu_seqlens=torch.arange(0, tokens + 1, per, dtype=torch.int32, device=device),
            entry_slot=torch.arange(entries, dtype=torch.int32, device=device),
            entry_start=torch.full((entries,), start, dtype=torch.int32, device=device), num_entries=entries, fault=fault)
        # -- routed feed-forward
        x = bf(tokens, width)
        router = f32(EXPERTS + 1, width)
        ids = torch.empty(tokens, TOP, dtype=torch.int32, device=device)
        weights, gates = torch.empty(tokens, TOP, device=device), torch.empty(tokens, 1, device=device)
        timed("router_topk", tokens, entries, tokens * width * 2 + router.numel() * 4,
              lambda: kernels.router_topk(x, router, experts=EXPERTS, top=TOP, ids=ids, weights=weights, gates=gates))
        pairs = tokens * TOP
        order, place = (torch.empty(pairs, dtype=torch.int32, device=device) for _ in range(2))
        meta = torch.zeros(1 + 3 * kernels.moe_max_tiles(pairs, EXPERTS, True), dtype=torch.int32, device=device)
        timed("moe_plan", tokens, entries, pairs * 16, lambda: kernels.moe_plan(ids, EXPERTS, order, place, meta, fault, wide=True))
        max_tiles = kernels.moe_max_tiles(pairs, EXPERTS, True)
        gate_up, down = bf(EXPERTS, 2 * inter, width), bf(EXPERTS, width, inter)
        act, each = torch.empty(pairs, inter, dtype=torch.bfloat16, device=device), torch.empty(pairs, width, device=device)
        touched = min(EXPERTS, pairs)          # experts whose weights a step streams
        timed("grouped_linear, gate and up with the activation", tokens, entries,
              touched * 2 * inter * width * 2 + tokens * width * 2 + pairs * inter * 2,
              lambda: kernels.grouped_linear(x, gate_up, order, meta, top=TOP, by_token=True, max_tiles=max_tiles,
                                             pair_weight=weights.view(-1), out_act=act, wide=True),
              flops=2.0 * pairs * 2 * inter * width)
        timed("grouped_linear, down", tokens, entries, touched * inter * width * 2 + pairs * inter * 2 + pairs * width * 4,
              lambda: kernels.grouped_linear(act, down, order, meta, top=TOP, by_token=False, max_tiles=max_tiles, out_y=each, wide=True),
              flops=2.0 * pairs * inter * width)
        shared, combined = bf(tokens, width), torch.empty(tokens, width, dtype=torch.bfloat16, device=device)
        timed("moe_combine", tokens, entries, pairs * width * 4 + tokens * width * 4,
              lambda: kernels.moe_combine(each, TOP, combined, shared=shared, gate=gates))
        # -- the layer's norms and the dense unit
        stream, weight = f32(tokens, width), f32(width)
        timed("join_rmsnorm", tokens, entries, tokens * width * 12, lambda: kernels.join_rmsnorm(x, stream, weight, combined, 1e-6))
        ff = (8 * width // 3 + 255) // 256 * 256
        wide, unit = bf(tokens, 2 * ff), torch.empty(tokens, ff, dtype=torch.bfloat16, device=device)
        timed("clamped_glu", tokens, entries, tokens * ff * 6, lambda: kernels.clamped_glu(wide, unit, 7.0, 1.702))
        # -- attention: convolution, rotation and norm into the cache, the tiles with a cap and a sink
        channels = (heads + 2 * kv_heads) * d
        proj, conv = bf(tokens, channels), torch.empty(tokens, channels, device=device)
        taps, tail = f32(channels, 4), torch.zeros(entries, 3 * channels, device=device)
        timed("causal_conv (no activation), 4 taps", tokens, entries, tokens * channels * 6 + 2 * tail.numel() * 4,
              lambda: kernels.causal_conv_silu(proj, taps, None, tail, conv, batch, act=False))
        pages_per = -(-(start + per) // page)
        cache = torch.zeros(entries * pages_per + 1, 2, kv_heads, page, d, dtype=torch.bfloat16, device=device)
        cache.normal_()
        table = (1 + torch.arange(entries * pages_per, dtype=torch.int32, device=device)).view(entries, pages_per)
        positions = (start + torch.arange(per, dtype=torch.int32, device=device)).repeat(entries)
        slot_of = torch.arange(entries, dtype=torch.int32, device=device).repeat_interleave(per)
        dest = (table[slot_of.long(), (positions // page).long()] * page + positions % page).to(torch.int32)
        q = torch.empty(tokens, heads * d, dtype=torch.bfloat16, device=device)
        inv_freq, mix, first = torch.rand(16, device=device), torch.rand(1, device=device), f32(tokens, kv_heads * d)
        timed("rope_unit_write", tokens, entries, tokens * channels * 6 + tokens * kv_heads * d * 4,
              lambda: kernels.rope_unit_write(conv, q, num_heads=heads, num_kv_heads=kv_heads, head_dim=d, inv_freq=inv_freq,
                                              positions=positions, kv_dest=dest, cache=cache, page_size=page, norm_size=d,
                                              unit=True, eps=1e-6, fault=fault, first=first, first_mode=2, mix=mix))
        from ..parts.attention import AttentionItems
        from ..parts.base import StepShape
        import numpy as np

        for capped in (True, False):
            planner = AttentionItems(heads // kv_heads, kv_heads, d, decode_tensor_core=not capped)
            plan = planner.plan(StepShape(lengths=np.full(entries, per, dtype=np.int32), starts=np.full(entries, start, dtype=np.int32),
                                          decode_only=per == 1, page_size=page))
            chunk = torch.from_numpy(plan["chunk_items"]).to(device)
            decode = torch.from_numpy(plan["decode_items"]).to(device)
            splits = plan["splits"]
            rows = tokens * heads * splits
            part_out = torch.empty(rows, d, device=device) if splits > 1 else None
            part_lse = torch.empty(rows, 1, device=device) if splits > 1 else None
            attended = torch.empty_like(q)
            sink = f32(heads) if capped else None
            keys = sum(range(start + 1, start + per + 1)) * entries
            label = "attention tiles, cap and sink" if capped else "attention tiles, plain scores"
            timed(label, tokens, entries, entries * (start + per) * kv_heads * d * 4 + tokens * heads * d * 4,
                  lambda: kernels.attention_mma(
                      q, cache, attended, chunk_items=chunk, decode_items=decode, splits=splits, part_out=part_out,
                      part_lse=part_lse, cu_seqlens=batch.cu_seqlens, entry_start=batch.entry_start, entry_slot=batch.entry_slot,
                      block_table=table, num_heads=heads, num_kv_heads=kv_heads, head_dim=d, window=0, scale=d ** -0.5,
                      fault=fault, decode_rows=plan["decode_rows"], chunk_rows=plan["chunk_rows"],
                      decode_splits=plan["decode_splits"], softcap=30.0 if capped else 0.0, sink=sink),
                  flops=4.0 * keys * heads * d)
    assert int(fault.item()) == 0, "a kernel reported a fault"
    return out


def alone(width: int = 2048) -> None:
    """Every kernel of :func:`kernel_figures` a few times and nothing else: the case a profiler captures, picking its
    kernel by name."""
    kernel_figures(width, 6650.0)
    torch.cuda.synchronize()


def run(sizes: list[int], hbm_gbs: float) -> dict:
    from ..config import MezadraConfig, Qwen3Config

    result = {"workload": "mezadra beside qwen3, equal sizes", "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": PREFILL, "decode_batch": 8, "decode_context": 1024, "sizes": {}}
    for width in sizes:
        result["sizes"][str(width)] = {
            "mezadra": model_figures(MezadraConfig.from_dict(mezadra_raw(width))),
            "qwen3": model_figures(Qwen3Config.from_dict(qwen3_raw(width, layers=6))),
            "kernels": kernel_figures(width, hbm_gbs),
        }
    return result


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--sizes", default="2048,4096")
    parser.add_argument("--hbm-gbs", type=float, default=6650.0)
    parser.add_argument("--alone", action="store_true", help="only launch the kernels a few times (for a profiler)")
    args = parser.parse_args()
    if args.alone:
        alone(int(args.sizes.split(",")[0]))
        return 0
    print(json.dumps(run([int(s) for s in args.sizes.split(",") if s], args.hbm_gbs)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
