"""Kopatar's configuration on the CPU: the run order a loop becomes, the tensors a model expects, refusals."""

from __future__ import annotations

import pytest
import torch
from kopatar_models import CONFIGS, make_config, make_weights, retention_layer, tensor_shapes, write_folder
from plain_kopatar import causal_conv, run_order

from rapid_llm_b200.config import KopatarConfig, load_config, resolve_architecture
from rapid_llm_b200.models.causal_lm import CausalLM


def test_the_registry_knows_the_architecture_by_its_key():
    assert resolve_architecture({"architecture": "Kopatar"}) is KopatarConfig
    with pytest.raises(ValueError, match="unsupported architecture"):
        resolve_architecture({"architecture": "Kopatar2"})


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_run_order_of_a_loop(name):
    raw = CONFIGS[name]
    spec = KopatarConfig.from_dict(raw).to_spec()
    assert [(entry.layer, entry.pass_index) for entry in spec.schedule] == run_order(raw)
    for entry in spec.schedule:
        assert entry.add_embedding == bool(entry.pass_index)      # every pass but the first
    if raw.get("loop"):
        start, stop, times = (raw["loop"][key] for key in ("start", "stop", "times"))
        assert len(spec.schedule) == len(raw["layers"]) + (times - 1) * (stop - start)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_model_expects_exactly_the_designs_tensors(name):
    raw = CONFIGS[name]
    model = CausalLM(KopatarConfig.from_dict(raw).to_spec(), torch.float32, "meta")
    expected = {key: spec for key, spec in model.tensor_specs().items() if not spec.optional}
    assert {key: tuple(spec.shape) for key, spec in expected.items()} == tensor_shapes(raw)
    # every entry of the run order has a state of its own, also where a layer runs several times
    assert len(model.state_needs()) == len(model.spec.schedule) and all(need is not None for need in model.state_needs())
    pages = [need for need in model.cache_needs() if need is not None]
    parallel_runs = sum(raw["layers"][entry.layer]["type"] == "parallel" for entry in model.spec.schedule)
    assert len(pages) == parallel_runs and all(need.kind == "window" for need in pages)


def test_low_rank_sizes_are_read_from_the_file_when_the_configuration_is_silent(tmp_path):
    raw = {key: value for key, value in CONFIGS["odd"].items() if key != "ranks"}
    with pytest.raises(ValueError, match="low-rank"):
        KopatarConfig.from_dict(raw)
    folder = write_folder(tmp_path / "m", raw, make_weights(CONFIGS["odd"], 0), torch.bfloat16)
    assert load_config(folder).ranks == {2: (3, 4)}
    assert KopatarConfig.from_dict(load_config(folder).to_dict()).ranks == {2: (3, 4)}


def test_refusals():
    with pytest.raises(ValueError, match="unknown mixer type"):
        KopatarConfig.from_dict(make_config([{"type": "conv", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError, match="loop"):
        KopatarConfig.from_dict(make_config([retention_layer()], loop=(0, 2, 2)))
    with pytest.raises(ValueError, match="one decay per head"):
        CausalLM(KopatarConfig.from_dict(make_config([retention_layer(heads=3)])).to_spec(), torch.float32, "meta")


def test_a_model_without_pages_still_has_state_rows_for_every_slot():
    from rapid_llm_b200.cache import CacheManager, plan_groups

    model = CausalLM(KopatarConfig.from_dict(CONFIGS["retention"]).to_spec(), torch.float32, "meta")
    groups, entry_group = plan_groups(model.cache_needs())
    assert groups == [] and entry_group == [None]
    manager = CacheManager(groups, page_size=8, num_pages=4, max_num_seqs=3, max_seq_len=64, extra_table_rows=1)
    assert manager.num_rows == 4
    assert manager.admit("a") is not None and manager.reserve("a", 40) and manager.num_tokens("a") == 40
    manager.release("a")
    manager.check()


def test_the_plain_convolution_is_the_librarys():
    x, taps = torch.randn(9, 5, dtype=torch.float64), torch.randn(5, 3, dtype=torch.float64)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T.unsqueeze(0), (2, 0)), taps.unsqueeze(1), groups=5)[0].T
    torch.testing.assert_close(causal_conv(x, taps), want)


def test_random_init_writes_a_kopatar_folder_from_the_command_line(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS["loop_inside"]))
    done = subprocess.run([sys.executable, "-m", "rapid_llm_b200.cli", "random-init", "--config", str(config), "--out",
                           str(tmp_path / "model"), "--seed", "4"], cwd=root, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    loaded = load_config(tmp_path / "model")
    assert isinstance(loaded, KopatarConfig) and loaded.loop == CONFIGS["loop_inside"]["loop"]
    from rapid_llm_b200.weights import SafetensorsFile

    with SafetensorsFile(tmp_path / "model" / "model.safetensors") as handle:
        assert set(handle.keys()) == set(tensor_shapes(CONFIGS["loop_inside"]))
