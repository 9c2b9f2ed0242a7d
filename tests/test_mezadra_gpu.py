"""The Mezadra decoder in the engine against the plain implementation (``plain_mezadra.py``).

Every configuration of ``mezadra_models.CONFIGS`` runs whole, with its tail decoded token by token, in portions of
changing size down to two tokens, and mixed with other requests on pages and state slots that are used again; then
the edges: a far token whose key stands out among hundreds, the first tokens of a sequence (where the convolutions
read zeros and the sink outweighs the keys), a far token under a slow decay, long decoding from captured graphs,
greedy generation through ``LLM.generate``, the command line and the trace runner.
"""

from __future__ import annotations

import pytest
import torch
from mezadra_models import CONFIGS, as_double, attention_layer, dense, lightning_layer, make_config, make_weights, moe, write_folder
from plain_mezadra import clear_margin, forward, greedy
from test_kopatar_gpu import DTYPES, _compare, _replay, _runner
from tolerances import assert_rows_close_by_size
from trace_tools import mixed, portions, tail_one_by_one, whole

pytestmark = pytest.mark.gpu

# how clearly every router decision of a test sequence must fall, in units of the router logits' spread: bfloat16
# rounds the stream the router reads, and a decision narrower than that rounding is no test of the engine
MARGIN = {"float32": 1e-4, "bfloat16": 0.04}


def _sequences(config, weights, lengths, seed, dtype):
    """Token sequences drawn by seed, each redrawn until no router decision in it is a close call."""
    generator = torch.Generator().manual_seed(seed)
    double, out = as_double(weights), {}
    for index, length in enumerate(lengths):
        for _ in range(200):
            tokens = torch.randint(0, config["vocab"], (length,), generator=generator).tolist()
            if clear_margin(config, double, tokens) > MARGIN[dtype]:
                break
        else:
            raise AssertionError("no sequence without a close router decision was drawn")
        out[f"r{index}"] = tokens
    return out


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_decoded_and_in_portions(name, dtype, tmp_path):
    config = CONFIGS[name]
    weights = make_weights(config, seed=11)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    tokens = _sequences(config, weights, [61], seed=3, dtype=dtype)["r0"]
    plain = {"a": forward(config, as_double(weights), tokens)}
    runner = _runner(folder, config, dtype, 160)
    for label, records in (
        ("whole", whole("a", tokens)),
        ("tail one by one", tail_one_by_one("a", tokens, tail=40)),
        ("portions", portions("a", tokens, [2, 3, 16, 2, 7, 8, 1, 5])),
        ("portions of two", portions("a", tokens, [2])),
        ("token by token", portions("a", tokens, [1])),
    ):
        _compare(_replay(runner, records), plain, dtype, f"{name} {dtype} ({label})")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["blend", "narrow"])
def test_mixed_batches_on_reused_pages_and_slots(name, dtype, tmp_path):
    config = CONFIGS[name]
    weights = make_weights(config, seed=5)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    lengths = [37, 90, 18, 75, 131, 52, 9] if dtype == "float32" else [21, 40, 12, 33, 48, 9]
    sequences = _sequences(config, weights, lengths, seed=8, dtype=dtype)
    plain = {rid: forward(config, as_double(weights), tokens) for rid, tokens in sequences.items()}
    records, peak = mixed(sequences, seed=2, max_live=3, page=8)
    runner = _runner(folder, config, dtype, peak, page=8, slots=3)
    mixed_rows = _replay(runner, records)
    _compare(mixed_rows, plain, dtype, f"{name} {dtype} (mixed)")
    # the same requests alone: what else is in the batch, and which slot and pages serve, changes nothing but rounding
    if dtype == "float32":
        for rid in ("r1", "r4"):
            alone = _replay(runner, whole(rid, sequences[rid]))[rid]
            for position, row in mixed_rows[rid].items():
                torch.testing.assert_close(row, alone[position], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_a_far_key_stands_out_among_hundreds(dtype, tmp_path):
    """One attention layer with sharp scores: the token at position 2 is the only one of its kind, and the last
    query is the same token, so its key is the one that matters among 400.  Changing that far token must change
    the last logits as the plain implementation says, in a prompt and while decoding, across page borders."""
    config = make_config([attention_layer(heads=2, kv_heads=1, dim=32, vdim=32, conv=2, rot_dims=0, scale=0.5, softcap=30.0,
                                          mlp=None)], width=32, vocab=40, scale=2.0)
    weights = make_weights(config, seed=31)
    # queries and keys share their projection and see the current token only: a token's query points at its own key
    # (the values keep their taps, so the far token's value differs from the query's own)
    weights["l0.mix.q"] = torch.cat([weights["l0.mix.k"], weights["l0.mix.k"]])
    for name in ("l0.mix.q.conv", "l0.mix.k.conv"):
        weights[name] = torch.zeros_like(weights[name])
        weights[name][:, -1] = 1.0
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    generator = torch.Generator().manual_seed(1)
    base = torch.randint(2, config["vocab"], (400,), generator=generator).tolist()
    base[2], base[-1] = 0, 0                      # token 0 nowhere else
    other = list(base)
    other[2] = 1
    last = len(base) - 1
    want = [forward(config, as_double(weights), tokens)[last].float() for tokens in (base, other)]
    effect = float((want[0] - want[1]).abs().max())
    assert effect > 0.5, "the test's weights do not make the far key count"
    runner = _runner(folder, config, dtype, 416, page=16)
    for records_of in (lambda t: whole("a", t), lambda t: tail_one_by_one("a", t, tail=20), lambda t: portions("a", t, [150, 2, 99, 17])):
        got = [_replay(runner, records_of(tokens))["a"][last] for tokens in (base, other)]
        error = float(((got[0] - got[1]) - (want[0] - want[1])).abs().max())
        assert error < (2e-3 if dtype == "float32" else 0.15) * effect


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_heads_of_128_on_the_tensor_core_tiles(dtype, tmp_path):
    """Heads of 128 take the tcgen05 chunk tiles in bfloat16, where the cap and the sink are computed by other
    instructions than in the other kernels: a low cap and large sinks, so that both decide the result; prompts long
    enough for several blocks of keys, portions behind cached keys, single tokens beside them."""
    config = make_config([
        attention_layer(heads=4, kv_heads=2, dim=128, vdim=96, conv=3, rot_dims=32, scale=0.3, softcap=3.0, v_mix=True, mlp=dense()),
        lightning_layer(heads=1, dim=128, vdim=128, decay=(0.97,), mlp=None),
        attention_layer(heads=2, kv_heads=2, dim=128, vdim=96, conv=2, rot_dims=128, scale=0.1, softcap=25.0, v_mix=True, mlp=None),
    ], width=128, vocab=150, scale=2.0)
    weights = make_weights(config, seed=61)
    weights["l0.mix.sink"] = torch.tensor([4.0, 0.5, -2.0, 7.0])
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, weights, [300, 45, 170], seed=5, dtype=dtype)
    plain = {rid: forward(config, as_double(weights), tokens) for rid, tokens in sequences.items()}
    runner = _runner(folder, config, dtype, 320, page=16)
    tokens = sequences["r0"]
    _compare(_replay(runner, whole("r0", tokens)), plain, dtype, f"heads of 128 {dtype} (whole)")
    _compare(_replay(runner, portions("r0", tokens, [130, 2, 90, 1, 40])), plain, dtype, f"heads of 128 {dtype} (portions)")
    _compare(_replay(runner, tail_one_by_one("r0", tokens, tail=12)), plain, dtype, f"heads of 128 {dtype} (tail)")
    records, peak = mixed(sequences, seed=3, max_live=3, page=16)
    _compare(_replay(_runner(folder, config, dtype, peak, page=16, slots=3), records), plain, dtype, f"heads of 128 {dtype} (mixed)")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_the_first_tokens_of_a_sequence(dtype, tmp_path):
    """Positions 0 to 5 alone: the convolutions reach before the sequence's start (zeros, whatever the slot's tail
    held from its last owner), a position sees few keys and the sink weighs most.  Every slot is used twice."""
    config = make_config([attention_layer(conv=5, heads=2, kv_heads=2, mlp=dense()), lightning_layer(mlp=None)], width=48)
    weights = make_weights(config, seed=41)
    weights["l0.mix.sink"] = torch.tensor([3.0, -3.0])
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, weights, [6, 1, 3, 2, 5, 4], seed=9, dtype=dtype)
    plain = {rid: forward(config, as_double(weights), tokens) for rid, tokens in sequences.items()}
    runner = _runner(folder, config, dtype, 32, page=8, slots=2)
    for rid, tokens in sequences.items():
        _compare(_replay(runner, portions(rid, tokens, [1, 2])), plain, dtype, f"first tokens {dtype}")
    records, peak = mixed(sequences, seed=4, max_live=2, page=8)
    _compare(_replay(_runner(folder, config, dtype, peak, page=8, slots=2), records), plain, dtype, f"first tokens {dtype} (mixed)")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_a_far_token_under_a_slow_decay(dtype, tmp_path):
    """With decays of 0.9995 and 1 the first token still weighs at position 300: what changing it does to the last
    logits must match the plain implementation (a state that was lost or restarted on the way would show here)."""
    config = make_config([lightning_layer(heads=2, dim=16, vdim=16, decay=(0.9995, 1.0), mlp=None)], width=32, vocab=50)
    weights = make_weights(config, seed=9)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    generator = torch.Generator().manual_seed(6)
    base = torch.randint(0, config["vocab"], (300,), generator=generator).tolist()
    other = [(base[0] + 7) % config["vocab"]] + base[1:]
    runner = _runner(folder, config, dtype, 320, page=16)
    last = len(base) - 1
    got = [_replay(runner, portions("a", tokens, [64, 2, 31, 1, 90]))["a"][last] for tokens in (base, other)]
    want = [forward(config, as_double(weights), tokens)[last].float() for tokens in (base, other)]
    effect = float((want[0] - want[1]).abs().max())
    assert effect > 5e-3, "the test's weights do not make the far token count"
    tolerance = 1e-2 if dtype == "float32" else 0.25
    assert float(((got[0] - got[1]) - (want[0] - want[1])).abs().max()) < tolerance * effect + (0 if dtype == "float32" else 0.05)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_decoding_from_captured_graphs(dtype, tmp_path):
    from rapid_llm_b200.engine.runner import StepEntry

    config = CONFIGS["blend"]
    weights = make_weights(config, seed=13)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    lengths = [150, 171, 160] if dtype == "float32" else [60, 75, 66]
    sequences = _sequences(config, weights, lengths, seed=12, dtype=dtype)
    plain = {rid: forward(config, as_double(weights), tokens) for rid, tokens in sequences.items()}
    runner = _runner(folder, config, dtype, 3 * 176, page=16, slots=4, graphs=True)
    heads = {"r0": 5, "r1": 40, "r2": 2}
    fed = {}
    for rid, head in heads.items():
        assert runner.admit(rid)
        runner.step([StepEntry(rid, sequences[rid][:head], [])])
        fed[rid] = head
    rows = {rid: {} for rid in sequences}
    while any(fed[rid] < len(sequences[rid]) for rid in sequences):
        live = [rid for rid in sequences if fed[rid] < len(sequences[rid])]
        logits = runner.step_decode([StepEntry(rid, [sequences[rid][fed[rid]]], [0]) for rid in live]).float().cpu()
        for row, rid in enumerate(live):
            rows[rid][fed[rid]] = logits[row].clone()
            fed[rid] += 1
    runner.check_fault()
    _compare(rows, plain, dtype, f"long decoding {dtype}")


def test_greedy_generation_through_the_entry_point(tmp_path):
    """More prompts than slots, so requests wait, and slots and pages change hands; float32 picks the same tokens."""
    from rapid_llm_b200 import LLM, SamplingParams

    config = CONFIGS["blend"]
    weights = make_weights(config, seed=17)
    folder = write_folder(tmp_path / "model", config, weights, torch.float32)
    prompts = list(_sequences(config, weights, [5, 23, 2, 41, 12], seed=14, dtype="float32").values())
    llm = LLM(folder, dtype="float32", max_seq_len=96, max_gpu_num_blocks=24, page_size=8, max_num_seqs=2, max_chunk_size=16)
    outputs = llm.generate(prompts, SamplingParams.greedy(max_gen_len=12))
    for prompt, output in zip(prompts, outputs):
        assert output.outputs[0].token_ids == greedy(config, as_double(weights), prompt, 12)


def test_many_experts_and_long_portions(tmp_path):
    """More pairs of one expert than a tile of the grouped products holds, more experts than a warp has lanes, and
    a portion of hundreds of tokens (float32; in bfloat16 a sequence of this length always holds a router decision
    that rounding settles, so there the kernels are compared one by one in ``test_mezadra_kernels_gpu.py`` and the
    two-expert layer alone runs through the engine)."""
    config = make_config([lightning_layer(heads=2, dim=16, vdim=16, decay=(0.9, 0.99), mlp=moe(experts=40, top=3, ff=24, shared=8)),
                          attention_layer(mlp=moe(experts=2, top=1, ff=40, shared=0))], width=64, vocab=90)
    weights = make_weights(config, seed=51)
    folder = write_folder(tmp_path / "float32", config, weights, torch.float32)
    tokens = _sequences(config, weights, [300], seed=2, dtype="float32")["r0"]
    plain = {"a": forward(config, as_double(weights), tokens)}
    runner = _runner(folder, config, "float32", 320, page=16)
    _compare(_replay(runner, whole("a", tokens)), plain, "float32", "many experts float32")
    _compare(_replay(runner, portions("a", tokens, [70, 2, 33])), plain, "float32", "many experts float32 (portions)")
    config = make_config([attention_layer(mlp=moe(experts=2, top=1, ff=40, shared=0))], width=64, vocab=90)
    weights = make_weights(config, seed=52)
    folder = write_folder(tmp_path / "bfloat16", config, weights, torch.bfloat16)
    tokens = _sequences(config, weights, [90], seed=2, dtype="bfloat16")["r0"]
    plain = {"a": forward(config, as_double(weights), tokens)}
    runner = _runner(folder, config, "bfloat16", 96, page=16)
    _compare(_replay(runner, whole("a", tokens)), plain, "bfloat16", "two experts bfloat16")


def test_the_command_line_and_the_trace_runner_take_a_mezadra_folder(tmp_path):
    """``batch`` generates from token-id prompts; ``bin/trace_run`` replays steps and writes the same logits as the
    plain implementation computes."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    root = Path(__file__).resolve().parents[1]
    config = CONFIGS["blend"]
    weights = make_weights(config, seed=23)
    folder = write_folder(tmp_path / "model", config, weights, torch.float32)
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("5 9 12 80 3\n7 7 1\n")
    done = subprocess.run([sys.executable, "-m", "rapid_llm_b200.cli", "batch", "--model-dir", str(folder), "--dtype", "float32",
                           "--prompt-ids-file", str(prompts), "--max-gen-len", "6", "--temperature", "0", "--repetition-penalty", "1.0", "--max-seq-len", "64",
                           "--max-gpu-num-blocks", "16"], cwd=root, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    lines = [line for line in done.stdout.splitlines() if line and not line.startswith("---")]
    assert [int(t) for t in lines[0].split()] == greedy(config, as_double(weights), [5, 9, 12, 80, 3], 6)

    tokens = _sequences(config, weights, [30], seed=2, dtype="float32")["r0"]
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tokens[:17], "want": [16]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": tokens[17:], "want": [0, 12]}], "end": ["x"]}]
    out = tmp_path / "out"
    done = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), cwd=tmp_path,
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
    plain = forward(config, as_double(weights), tokens).float()
    got = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1).copy())
    assert_rows_close_by_size(got, plain[[17, 29]], "float32")
