"""Mezadra configurations drawn by seed against the plain implementation: layer kinds in any order, head counts,
key and value sizes, taps, rotated sizes, caps, experts and how many a token takes, with and without a shared
expert, layers without a feed-forward.  Each draw replays a mixed trace (portions of prompts beside decoded tokens
on few pages and three state slots) in float32 and bfloat16."""

from __future__ import annotations

import random

import pytest
from mezadra_models import as_double, attention_layer, dense, lightning_layer, make_config, make_weights, moe, write_folder
from plain_mezadra import forward
from test_kopatar_gpu import DTYPES, _compare, _replay, _runner
from test_mezadra_gpu import _sequences
from tolerances import BF16_ROW_RMS
from trace_tools import mixed

DRAWS = 8


def draw_config(seed: int) -> dict:
    rng = random.Random(7000 + seed)
    kv_heads, dim, vdim = rng.choice([1, 2]), rng.choice([16, 24, 32, 64]), rng.choice([8, 16, 32, 48])      # of the layers that blend
    layers = []
    for _ in range(rng.randint(2, 5)):
        pick = rng.random()
        if pick < 0.25:
            mlp = None
        elif pick < 0.6:
            mlp = dense(ff=rng.choice([20, 33, 48, 64]), limit=rng.choice([0.5, 1.0, 7.0]))
        else:
            experts = rng.randint(1, 9)
            mlp = moe(experts=experts, top=rng.randint(1, min(experts, 3)), ff=rng.choice([8, 12, 32]), shared=rng.choice([0, 8, 20]))
        if rng.random() < 0.45:
            heads = rng.randint(1, 4)
            layers.append(lightning_layer(heads=heads, dim=rng.choice([8, 16, 32]), vdim=rng.choice([8, 16, 24]),
                                          decay=[1.0 - 0.5 * rng.random() ** 3 for _ in range(heads)], mlp=mlp))
            continue
        blends = rng.random() < 0.6
        own_kv, own_dim, own_vdim = (kv_heads, dim, vdim) if blends else (rng.choice([1, 2, 3]), rng.choice([16, 32, 40]), rng.choice([16, 32, 40]))
        layers.append(attention_layer(heads=own_kv * rng.choice([1, 2, 4]), kv_heads=own_kv, dim=own_dim, vdim=own_vdim,
                                      conv=rng.randint(1, 5), rot_dims=rng.choice([0, 2, 8, own_dim]), base=rng.choice([50.0, 1.0e4, 5.0e5]),
                                      scale=rng.uniform(0.1, 1.0), softcap=rng.choice([1.5, 10.0, 50.0]), v_mix=blends, mlp=mlp))
    return make_config(layers, width=rng.choice([32, 40, 48, 64, 72, 96]), vocab=rng.randint(50, 200),
                       eps=rng.choice([1e-6, 1e-5]), scale=rng.choice([1.0, 4.0, 9.5]))


def test_the_draws_differ():
    drawn = [draw_config(seed) for seed in range(DRAWS)]
    kinds = [tuple((layer["type"], (layer["mlp"] or {}).get("kind")) for layer in config["layers"]) for config in drawn]
    assert len(set(kinds)) >= DRAWS - 2
    assert {"attention", "lightning"} <= {k for order in kinds for k, _ in order}
    assert {"dense", "moe", None} <= {m for order in kinds for _, m in order}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("seed", range(DRAWS))
def test_a_drawn_configuration_in_mixed_batches(seed, dtype, tmp_path):
    config = draw_config(seed)
    weights = make_weights(config, seed=100 + seed)
    folder = write_folder(tmp_path / "model", config, weights, DTYPES[dtype])
    lengths = [33, 70, 12, 58, 91, 6] if dtype == "float32" else [17, 30, 12, 25, 36, 6]
    sequences = _sequences(config, weights, lengths, seed=seed, dtype=dtype)
    plain = {rid: forward(config, as_double(weights), tokens) for rid, tokens in sequences.items()}
    records, peak = mixed(sequences, seed=seed, max_live=3, page=8)
    runner = _runner(folder, config, dtype, peak, page=8, slots=3)
    rows = _replay(runner, records)
    if dtype == "float32":
        return _compare(rows, plain, dtype, f"seed {seed} {dtype}: {config}")
    # bfloat16: the stream a router reads has been through every layer before it in 16-bit products, and a drawn
    # model has decisions that this rounding settles although the sequences were drawn clear of the closest calls.
    # So the bound by the row's size is asked of 19 rows in 20, and no row may be off by more than a quarter of its
    # size; the float32 run of the same draw holds the element-wise bound at every position.
    spreads = []
    for request_id, by_position in rows.items():
        for position, got in by_position.items():
            want = plain[request_id][position].float()
            error = got.float() - want
            size = (want - want.mean()).pow(2).mean().sqrt()
            spreads.append(float((error - error.mean()).pow(2).mean().sqrt() / size))
    spreads.sort()
    assert spreads[int(0.95 * len(spreads))] <= BF16_ROW_RMS, f"seed {seed}: 95th percentile {spreads[int(0.95 * len(spreads))]:.4f}: {config}"
    assert spreads[-1] <= 0.25, f"seed {seed}: worst row {spreads[-1]:.4f}: {config}"
