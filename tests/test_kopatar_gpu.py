"""The Kopatar decoder in the engine against the plain implementation (``plain_kopatar.py``).

Every configuration of ``kopatar_models.CONFIGS`` runs whole, with its tail decoded token by token, in
portions of changing size down to two tokens, and mixed with other requests on pages and state slots that
are used again; then the edges: the sliding window's first key outside and last key inside (in a prompt and
while decoding), a far token under a slow decay, long decoding from captured graphs, greedy generation
through ``LLM.generate``.
"""

from __future__ import annotations

import dataclasses

import pytest
import torch
from kopatar_models import CONFIGS, as_double, make_config, make_weights, parallel_layer, retention_layer, write_folder
from plain_kopatar import forward, greedy
from tolerances import assert_rows_close_by_size
from trace_tools import collect, mixed, portions, tail_one_by_one, whole

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _runner(folder, config, dtype, tokens, page=8, slots=4, graphs=False):
    from rapid_llm_b200.config import load_config
    from rapid_llm_b200.engine.runner import ModelRunner
    from rapid_llm_b200.replay import engine_config_for

    engine = dataclasses.replace(engine_config_for(load_config(folder), dtype, tokens, page, slots), use_cuda_graph=graphs)
    return ModelRunner.from_folder(folder, engine)


def _replay(runner, records):
    from rapid_llm_b200.replay import Replayer

    replayer, outputs = Replayer(runner), {}
    for record in records:
        out = replayer.run_step(record)
        if out is not None:
            outputs[record["step"]] = torch.from_numpy(out.copy())
        runner.cache.check()
    return collect(records, outputs)


WORST: dict[str, float] = {}      # label -> largest root-mean-square error of a row, as a share of the row's size


def _spread(got, want):
    size = (want - want.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt()
    error = got.float() - want
    return float(((error - error.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / size).max())


def _compare(rows, plain, dtype, label):
    for request_id, by_position in rows.items():
        positions = sorted(by_position)
        got = torch.stack([by_position[p] for p in positions])
        want = plain[request_id][positions].float()
        try:
            assert_rows_close_by_size(got, want, dtype)
        except AssertionError as exc:
            raise AssertionError(f"{label}: request {request_id!r}: {exc}") from None
        WORST[label] = max(WORST.get(label, 0.0), _spread(got, want))


def _sequences(config, lengths, seed):
    generator = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=generator).tolist() for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_decoded_and_in_portions(name, dtype, tmp_path):
    config = CONFIGS[name]
    weights = make_weights(config, seed=11)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    tokens = _sequences(config, [77], seed=3)["r0"]
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
@pytest.mark.parametrize("name", ["odd", "loop_inside", "loop_from_start"])
def test_mixed_batches_on_reused_pages_and_slots(name, dtype, tmp_path):
    config = CONFIGS[name]
    weights = make_weights(config, seed=5)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, [37, 90, 18, 75, 131, 52, 9], seed=8)
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


def test_the_low_rank_sizes_come_from_the_file(tmp_path):
    config = dict(CONFIGS["odd"])
    weights = make_weights(config, seed=1)
    bare = {key: value for key, value in config.items() if key != "ranks"}
    folder = write_folder(tmp_path / "model", bare, weights, torch.float32)
    tokens = _sequences(config, [20], seed=1)["r0"]
    runner = _runner(folder, bare, "float32", 64)
    _compare(_replay(runner, whole("a", tokens)), {"a": forward(config, as_double(weights), tokens)}, "float32", "ranks")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_the_window_ends_where_it_should(dtype, tmp_path):
    """One layer, the attention side alone (the other side's scale is 0): a token just outside the window must
    not reach a position's logits at all, the one just inside must; in a prompt, and at a decoded token."""
    window = 13
    config = make_config([parallel_layer(window=window, left_scale=1.0, right_scale=0.0, scale=1.5, ff=None)], width=64)
    weights = make_weights(config, seed=21)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    base = _sequences(config, [60], seed=4)["r0"]
    at = 47                                   # the position whose logits are read
    runner = _runner(folder, config, dtype, 64)

    def logits_at(tokens, decode):
        records = tail_one_by_one("a", tokens, tail=len(tokens) - at + 5) if decode else whole("a", tokens)
        return _replay(runner, records)["a"][at]

    for decode in (False, True):
        reference = logits_at(base, decode)
        outside, inside = list(base), list(base)
        outside[at - window] = (base[at - window] + 1) % config["vocab"]
        inside[at - window + 1] = (base[at - window + 1] + 1) % config["vocab"]
        assert torch.equal(logits_at(outside, decode), reference), "a token outside the window changed the logits"
        moved = (logits_at(inside, decode) - reference).abs().max()
        expected = (forward(config, as_double(weights), inside)[at] - forward(config, as_double(weights), base)[at]).abs().max()
        assert float(moved) > 0.3 * float(expected) > 0, "the last token inside the window did not reach the logits"


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_a_far_token_under_a_slow_decay(dtype, tmp_path):
    """With a decay of 0.9995 the first token still weighs at position 300: what changing it does to the last logits
    must match the plain implementation (a state that was lost or restarted on the way would show here)."""
    config = make_config([retention_layer(heads=2, dim=16, vdim=16, decay=(0.9995, 1.0), rot_dims=4, ff=None)], width=32, vocab=50)
    weights = make_weights(config, seed=9)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    base = _sequences(config, [300], seed=6)["r0"]
    other = [(base[0] + 7) % config["vocab"]] + base[1:]
    runner = _runner(folder, config, dtype, 320, page=16)
    last = len(base) - 1
    got = [_replay(runner, portions("a", tokens, [64, 2, 31, 1, 90]))["a"][last] for tokens in (base, other)]
    want = [forward(config, as_double(weights), tokens)[last].float() for tokens in (base, other)]
    effect = float((want[0] - want[1]).abs().max())
    assert effect > 1e-2, "the test's weights do not make the far token count"
    tolerance = 2e-3 if dtype == "float32" else 0.25
    assert float(((got[0] - got[1]) - (want[0] - want[1])).abs().max()) < tolerance * effect + (0 if dtype == "float32" else 0.05)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_decoding_from_captured_graphs(dtype, tmp_path):
    from rapid_llm_b200.engine.runner import StepEntry

    config = CONFIGS["loop_inside"]
    weights = make_weights(config, seed=13)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    sequences = _sequences(config, [150, 171, 160], seed=12)
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

    config = CONFIGS["loop_inside"]
    weights = make_weights(config, seed=17)
    folder = write_folder(tmp_path / "model", config, weights, torch.float32)
    prompts = list(_sequences(config, [5, 23, 2, 41, 12], seed=14).values())
    llm = LLM(folder, dtype="float32", max_seq_len=96, max_gpu_num_blocks=24, page_size=8, max_num_seqs=2, max_chunk_size=16)
    outputs = llm.generate(prompts, SamplingParams.greedy(max_gen_len=12))
    for prompt, output in zip(prompts, outputs):
        assert output.outputs[0].token_ids == greedy(config, as_double(weights), prompt, 12)


def test_zz_report_the_errors_seen():
    """Not a check: prints the largest bfloat16 row error of every comparison above (shown with ``pytest -s``)."""
    for label, worst in sorted(WORST.items()):
        if "bfloat16" in label:
            print(f"  {label}: {worst:.4f}")


def test_the_command_line_and_the_trace_runner_take_a_kopatar_folder(tmp_path):
    """``batch`` generates from token-id prompts; ``bin/trace_run`` replays steps and writes the same logits as the
    plain implementation computes."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    root = Path(__file__).resolve().parents[1]
    config = CONFIGS["loop_inside"]
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

    tokens = _sequences(config, [30], seed=2)["r0"]
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
