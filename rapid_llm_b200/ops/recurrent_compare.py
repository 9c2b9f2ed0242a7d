"""Prefill and decode throughput of Kopatar models at layer sizes of real models, beside Qwen3 of equal size,
and every kernel of the recurrent mixers alone against the memory roofline.

    python bench.py --workload kopatar [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.recurrent_compare [--sizes 2048,4096]
    python -m rapid_llm_b200.ops.recurrent_compare --scan fixed|delta      # three launches of the recurrence, for ncu

Random weights, bfloat16, one GPU.  A model of width ``W`` has heads of 128, a feed-forward of ``4 W`` (Qwen3's
gated one gets ``8 W / 3`` rounded to 256, the same number of weights) and the layers
``parallel, channel_delta, retention, retention`` with the last three run twice (seven layer runs); the Qwen3
beside it has seven layers.  Prefill is one 2,048-token step (best of three, CUDA events around the step
function); decode is batch 8 behind 1,024-token prompts, replayed from the captured graph (median of 32 steps).
Kernels are timed alone with CUDA events, L2 flushed between runs (a write of 256 MB), on one 2,048-token
prompt and on 64 single tokens; ``frac`` is (bytes the kernel must move) / time / measured copy bandwidth.
"""

from __future__ import annotations

import argparse
import json
import statistics
from types import SimpleNamespace

import torch

PREFILL, PROMPT, BATCH, STEPS, PAGE = 2048, 1024, 8, 32, 16


def kopatar_raw(width: int) -> dict:
    heads, ff = width // 128, 4 * width
    mlp = {"kind": "dense", "ff": ff}
    retention = {"type": "retention", "mlp": mlp, "mixer": {
        "heads": heads, "dim": 128, "vdim": 128, "rot": {"dims": 128, "base": 1.0e6},
        "decay": [1.0 - 2.0 ** (-5 - 5 * h / max(heads - 1, 1)) for h in range(heads)]}}
    return {
        "architecture": "Kopatar", "vocab": 32000, "width": width, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "parallel", "mlp": mlp, "mixer": {
                "left": {"heads": heads // 2, "kv_heads": max(heads // 8, 1), "dim": 128, "vdim": 128,
                         "mask": {"size": 1024}, "scale": 128 ** -0.5},
                "right": {"heads": width // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8},
                "left_scale": 0.7, "right_scale": 0.7}},
            {"type": "channel_delta", "mlp": mlp,
             "mixer": {"heads": heads, "kv_heads": heads, "dim": 128, "vdim": 128, "conv": 4}},
            retention, retention,
        ],
        "loop": {"start": 1, "stop": 4, "times": 2},
        "ranks": {"1": [width // 16, width // 16]},
    }


def qwen3_raw(width: int, layers: int = 7) -> dict:
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 32000, "hidden_size": width,
        "intermediate_size": (8 * width // 3 + 255) // 256 * 256, "num_hidden_layers": layers,
        "num_attention_heads": width // 128, "num_key_value_heads": max(width // 512, 1), "head_dim": 128,
        "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "rope_theta": 1.0e6, "tie_word_embeddings": True,
        "torch_dtype": "bfloat16",
    }


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def model_figures(config) -> dict:
    """Prefill and decode of one model through the step function."""
    from ..config import EngineConfig
    from ..engine.runner import ModelRunner, StepEntry
    from . import kernels

    longest = PROMPT + STEPS + 16
    engine = EngineConfig(dtype=torch.bfloat16, max_seq_len=PREFILL + 64, page_size=PAGE,
                          num_pages=(BATCH + 1) * (-(-max(longest, PREFILL) // PAGE)) + 8, max_num_seqs=BATCH + 1,
                          max_num_batched_tokens=PREFILL, max_chunk_size=PREFILL, use_cuda_graph=True)
    runner = ModelRunner.from_random(config, seed=0, config=engine)
    vocab = runner.model.spec.vocab_size
    generator = torch.Generator().manual_seed(0)
    draw = lambda n: torch.randint(0, vocab, (n,), generator=generator).tolist()      # noqa: E731
    prefill = []
    for _ in range(5):
        tokens = draw(PREFILL)
        runner.admit("p")
        begin, end = _events()
        torch.cuda.synchronize()
        before = kernels.LAUNCHES.count
        begin.record()
        runner.step([StepEntry("p", tokens, [PREFILL - 1])])
        end.record()
        torch.cuda.synchronize()
        launches = kernels.LAUNCHES.count - before
        runner.release("p")
        prefill.append(begin.elapsed_time(end))
    for index in range(BATCH):
        runner.admit(index)
        runner.step([StepEntry(index, draw(PROMPT), [])])
    decode = []
    for step in range(STEPS + 4):
        entries = [StepEntry(index, draw(1), [0]) for index in range(BATCH)]
        begin, end = _events()
        begin.record()
        runner.step_decode(entries)
        end.record()
        torch.cuda.synchronize()
        if step >= 4:
            decode.append(begin.elapsed_time(end))
    runner.check_fault()
    ms = statistics.median(decode)
    figures = {
        "weights_gb": round(runner.model.parameter_bytes() / 1e9, 3),
        "prefill_ms": round(min(prefill[2:]), 3), "prefill_tok_s": round(PREFILL / (min(prefill[2:]) / 1e3), 1),
        "prefill_launches": launches,
        "decode_ms_per_step": round(ms, 4), "decode_tok_s": round(BATCH / (ms / 1e3), 1),
    }
    del runner
    torch.cuda.empty_cache()
    return figures


def kernel_figures(width: int, hbm_gbs: float) -> dict:
    """Every kernel of the recurrent mixers alone, on a 2,048-token prompt and on 64 single tokens."""
    from . import kernels

    device, heads, dim = "cuda:0", width // 128, 128
    flush = torch.empty(64 << 20, dtype=torch.float32, device=device)
    out = {}

    def timed(label, tokens, entries, moved, run):
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
        out[f"{label} ({'prompt of ' + str(tokens) if entries == 1 else str(entries) + ' single tokens'})"] = {
            "us": round(us, 1), "mb": round(moved / 1e6, 2), "frac": round(moved / (us * 1e-6) / (hbm_gbs * 1e9), 3)}

    for tokens, entries in ((PREFILL, 1), (64, 64)):
        per = tokens // entries
        batch = SimpleNamespace(
            cu_seqlens=torch.arange(0, tokens + 1, per, dtype=torch.int32, device=device),
            entry_slot=torch.arange(entries, dtype=torch.int32, device=device),
            entry_start=torch.full((entries,), 512, dtype=torch.int32, device=device), num_entries=entries,
            fault=torch.zeros(1, dtype=torch.int32, device=device))
        bf = lambda *shape: torch.randn(*shape, device=device).to(torch.bfloat16)      # noqa: E731
        f32 = lambda *shape: torch.randn(*shape, device=device)                        # noqa: E731
        c = heads * dim
        state = torch.zeros(entries, heads * dim * dim, device=device)
        state_bytes = 2 * state.numel() * 4
        q, k, v, read = f32(tokens, c), f32(tokens, c), f32(tokens, c), f32(tokens, c)
        fixed, per_token = torch.rand(heads, device=device), torch.rand(tokens, heads, device=device)
        per_row, beta = torch.rand(tokens, c, device=device), torch.rand(tokens, heads, device=device)
        io = 4 * tokens * c * 4
        timed("linear_scan, fixed decay", tokens, entries, state_bytes + io,
              lambda: kernels.linear_scan(q, k, v, fixed, read, state, batch, heads=heads, kv_heads=heads, dim=dim, vdim=dim))
        timed("linear_scan, decay per token", tokens, entries, state_bytes + io,
              lambda: kernels.linear_scan(q, k, v, per_token, read, state, batch, heads=heads, kv_heads=heads, dim=dim,
                                          vdim=dim, v_scale=beta))
        timed("linear_scan, delta rule with row decays", tokens, entries, state_bytes + io + tokens * c * 4,
              lambda: kernels.linear_scan(q, k, v, per_row, read, state, batch, heads=heads, kv_heads=heads, dim=dim,
                                          vdim=dim, beta=beta))
        proj, conv = bf(tokens, 3 * c), torch.empty(tokens, 3 * c, device=device)
        taps, tail = f32(3 * c, 4), torch.zeros(entries, 3 * 3 * c, device=device)
        timed("causal_conv_silu, 4 taps", tokens, entries, tokens * 3 * c * 6 + 2 * tail.numel() * 4,
              lambda: kernels.causal_conv_silu(proj, taps, None, tail, conv, batch))
        timed("decay_gate", tokens, entries, tokens * c * 6,
              lambda: kernels.decay_gate(proj[:, :c], fixed, None, dim, per_row))
        timed("unit_heads", tokens, entries, tokens * 2 * c * 8,
              lambda: kernels.unit_heads(conv[:, : 2 * c], heads=2 * heads, dim=dim, eps=1e-6, split=heads, scale_low=1.0, scale_high=1.0))
        positions = torch.arange(tokens, dtype=torch.int32, device=device)
        inv_freq = torch.rand(dim // 2, device=device)
        timed("rotate_heads", tokens, entries, tokens * 3 * c * 6,
              lambda: kernels.rotate_heads(proj[:, :c], proj[:, c : 2 * c], proj[:, 2 * c :], conv, positions, inv_freq,
                                           heads=heads, dim=dim, vdim=dim, k_scale=1.0))
        normed, weight = torch.empty(tokens, c, dtype=torch.bfloat16, device=device), f32(dim)
        timed("gated_norm", tokens, entries, tokens * c * 8,
              lambda: kernels.gated_norm(read, normed, group=dim, gate=proj[:, :c], act=kernels.GATE_SIGMOID, weight=weight, eps=1e-6))
        wide, act, pq = bf(tokens, 4 * width), torch.empty(tokens, 4 * width, dtype=torch.bfloat16, device=device), f32(2)
        timed("xielu", tokens, entries, tokens * 4 * width * 4, lambda: kernels.xielu(wide, act, pq))
    return out


def scan_alone(kind: str, width: int = 2048, launches: int = 3) -> None:
    """A few launches of the recurrence kernel over one 2,048-token prompt and nothing else: the case a profiler
    captures (``--scan fixed`` or ``--scan delta``)."""
    from . import kernels

    device, heads, dim, tokens = "cuda:0", width // 128, 128, PREFILL
    c = heads * dim
    batch = SimpleNamespace(
        cu_seqlens=torch.tensor([0, tokens], dtype=torch.int32, device=device),
        entry_slot=torch.zeros(1, dtype=torch.int32, device=device),
        entry_start=torch.full((1,), 512, dtype=torch.int32, device=device), num_entries=1,
        fault=torch.zeros(1, dtype=torch.int32, device=device))
    q, k, v, read = (torch.randn(tokens, c, device=device) for _ in range(4))
    state = torch.zeros(1, heads * dim * dim, device=device)
    for _ in range(launches):
        if kind == "delta":
            kernels.linear_scan(q, k, v, torch.rand(tokens, c, device=device), read, state, batch, heads=heads,
                                kv_heads=heads, dim=dim, vdim=dim, beta=torch.rand(tokens, heads, device=device))
        else:
            kernels.linear_scan(q, k, v, torch.rand(heads, device=device), read, state, batch, heads=heads,
                                kv_heads=heads, dim=dim, vdim=dim)
    torch.cuda.synchronize()


def run(sizes: list[int], hbm_gbs: float) -> dict:
    from ..config import KopatarConfig, Qwen3Config

    result = {"workload": "kopatar beside qwen3, equal sizes", "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": PREFILL, "decode_batch": BATCH, "decode_context": PROMPT, "sizes": {}}
    for width in sizes:
        result["sizes"][str(width)] = {
            "kopatar": model_figures(KopatarConfig.from_dict(kopatar_raw(width))),
            "qwen3": model_figures(Qwen3Config.from_dict(qwen3_raw(width))),
            "kernels": kernel_figures(width, hbm_gbs),
        }
    return result


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--sizes", default="2048,4096")
    parser.add_argument("--hbm-gbs", type=float, default=6650.0)
    parser.add_argument("--scan", choices=["fixed", "delta"], default=None,
                        help="only launch the recurrence kernel a few times (for a profiler)")
    args = parser.parse_args()
    if args.scan:
        scan_alone(args.scan)
        return 0
    print(json.dumps(run([int(s) for s in args.sizes.split(",") if s], args.hbm_gbs)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
