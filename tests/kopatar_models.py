"""Small Kopatar configurations and seeded weights for the tests.

The weights are drawn so that every mechanism carries weight: decays between about 0.7 and 0.999,
peaked attention, activations on both branches.  Every value is rounded to bfloat16 once, so a folder
written in either precision and the float64 plain implementation hold the same numbers.
"""

from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def parallel_layer(*, heads=4, kv_heads=2, dim=16, vdim=32, window=9, scale=0.3, left_scale=0.7, right_scale=1.3,
                   ssm_heads=3, ssm_vdim=16, state=8, groups=1, conv=2, norm_groups=3, ff=72):
    return {
        "type": "parallel",
        "mixer": {
            "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale},
            "right": {"heads": ssm_heads, "vdim": ssm_vdim, "state": state, "groups": groups, "conv": conv,
                      "norm_groups": norm_groups},
            "left_scale": left_scale, "right_scale": right_scale,
        },
        "mlp": None if ff is None else {"kind": "dense", "ff": ff},
    }


def delta_layer(*, heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def retention_layer(*, heads=2, dim=32, vdim=16, decay=(0.9, 0.999), rot_dims=8, base=100.0, ff=40):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "retention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def make_config(layers, *, width=64, vocab=97, eps=1e-5, loop=None, ranks=(5, 7)) -> dict:
    config = {"architecture": "Kopatar", "vocab": vocab, "width": width, "norm": {"eps": eps},
              "layers": copy.deepcopy(list(layers))}
    if loop:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
    config["ranks"] = {str(i): list(ranks) for i, layer in enumerate(layers) if layer["type"] == "channel_delta"}
    return config


CONFIGS = {
    # one mixer kind each, with sizes that differ wherever they may: heads from kv heads, dim from vdim
    "delta": make_config([delta_layer()], width=64),
    "retention": make_config([retention_layer()], width=48, vocab=61),
    "parallel": make_config([parallel_layer()], width=64),
    # a width, a feed-forward and ranks that are no multiples of 8; one group norm; whole head rotated; window of 1
    "odd": make_config([
        parallel_layer(heads=3, kv_heads=3, dim=24, vdim=8, window=1, ssm_heads=4, ssm_vdim=12, state=5, groups=2,
                       conv=4, norm_groups=1, ff=50),
        retention_layer(heads=3, dim=8, vdim=20, decay=(0.5, 0.97, 1.0), rot_dims=8, ff=None),
        delta_layer(heads=2, kv_heads=1, dim=40, vdim=8, conv=2, ff=36),
    ], width=60, vocab=130, ranks=(3, 4)),
    # nothing is a multiple of 4: every kernel's element-by-element path; a convolution of one tap; no rotation
    "narrow": make_config([
        delta_layer(heads=3, kv_heads=3, dim=10, vdim=6, conv=2, ff=30),
        parallel_layer(heads=2, kv_heads=1, dim=10, vdim=14, window=7, ssm_heads=3, ssm_vdim=5, state=7, groups=3,
                       conv=1, norm_groups=1, ff=None),
        retention_layer(heads=3, dim=6, vdim=9, decay=(0.8, 0.9, 0.99), rot_dims=0, ff=22),
    ], width=50, vocab=83, ranks=(3, 3), loop=(2, 3, 2)),
    # a loop that starts at the first layer and runs three times, layers before and after none
    "loop_from_start": make_config([retention_layer(decay=(0.95, 0.99)), delta_layer(ff=40)], loop=(0, 2, 3)),
    # a loop in the middle, a parallel layer inside it (pages per pass), layers on both sides
    "loop_inside": make_config([
        delta_layer(heads=2, kv_heads=2, dim=32, vdim=16, ff=48),
        parallel_layer(window=20, conv=3, norm_groups=1, groups=3),
        retention_layer(ff=None),
        parallel_layer(heads=2, kv_heads=1, dim=32, vdim=32, window=33, ssm_heads=2, ssm_vdim=8, state=16, groups=2,
                       conv=4, norm_groups=2, ff=40),
    ], loop=(1, 3, 2)),
}


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    width, shapes = config["width"], {"embed": (config["vocab"], config["width"]), "final.norm": (config["width"],)}
    if config.get("loop"):
        shapes["loop.step"] = (config["loop"]["times"], width)
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        shapes[p + "norm1"] = (width,)
        if layer["type"] == "channel_delta":
            ra, rg = config["ranks"][str(index)]
            hk, h = m["kv_heads"] * m["dim"], m["heads"]
            shapes.update({
                p + "mix.q": (hk, width), p + "mix.q.conv": (hk, m["conv"]), p + "mix.k": (hk, width),
                p + "mix.k.conv": (hk, m["conv"]), p + "mix.v": (h * m["vdim"], width),
                p + "mix.v.conv": (h * m["vdim"], m["conv"]), p + "mix.b": (h, width), p + "mix.A_log": (h,),
                p + "mix.norm": (m["vdim"],), p + "mix.a1": (ra, width), p + "mix.a2": (h * m["dim"], ra),
                p + "mix.dt_bias": (h * m["dim"],), p + "mix.g1": (rg, width), p + "mix.g2": (h * m["vdim"], rg),
                p + "mix.o": (width, h * m["vdim"]),
            })
        elif layer["type"] == "retention":
            h = m["heads"]
            shapes.update({p + "mix.q": (h * m["dim"], width), p + "mix.k": (h * m["dim"], width),
                           p + "mix.v": (h * m["vdim"], width), p + "mix.g": (h * m["vdim"], width),
                           p + "mix.o": (width, h * m["vdim"])})
        else:
            left, right = m["left"], m["right"]
            inner, gn = right["heads"] * right["vdim"], right["groups"] * right["state"]
            shapes.update({
                p + "mix.left.q": (left["heads"] * left["dim"], width), p + "mix.left.k": (left["kv_heads"] * left["dim"], width),
                p + "mix.left.v": (left["kv_heads"] * left["vdim"], width), p + "mix.left.q.norm": (left["dim"],),
                p + "mix.left.k.norm": (left["dim"],), p + "mix.left.g": (left["heads"] * left["vdim"], width),
                p + "mix.left.o": (width, left["heads"] * left["vdim"]),
                p + "mix.right.in": (2 * inner + 2 * gn + right["heads"], width),
                p + "mix.right.conv": (inner + 2 * gn, right["conv"]), p + "mix.right.conv.b": (inner + 2 * gn,),
                p + "mix.right.dt_bias": (right["heads"],), p + "mix.right.A_log": (right["heads"],),
                p + "mix.right.D": (right["heads"],), p + "mix.right.norm": (inner,), p + "mix.right.o": (width, inner),
            })
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            shapes.update({p + "norm2": (width,), p + "mlp.up": (ff, width), p + "mlp.down": (width, ff), p + "mlp.act": (2,)})
    return shapes


def make_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors whose values are exact in bfloat16."""
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in tensor_shapes(config).items():
        draw = torch.randn(shape, generator=generator)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            value = draw
        elif last in ("norm", "norm1", "norm2", "D") or name.endswith("q.norm") or name.endswith("k.norm"):
            value = 1.0 + 0.2 * draw
        elif last == "conv":
            value = 0.6 * draw
        elif last == "A_log":
            value = 0.5 * draw
        elif last == "dt_bias":
            value = -3.0 + draw
        elif last in ("b", "act", "step"):
            value = (0.1 if name.endswith("conv.b") else 0.7) * draw
        else:
            value = draw / math.sqrt(shape[-1]) * (2.0 if last in ("q", "k") else 1.0)
        weights[name] = value.to(torch.bfloat16).to(torch.float32)
    return weights


def write_folder(folder: Path, config: dict, weights: dict[str, torch.Tensor], dtype: torch.dtype) -> Path:
    from rapid_llm_b200.weights.safetensors_io import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", {name: value.to(dtype) for name, value in weights.items()})
    return folder


def as_double(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {name: value.double() for name, value in weights.items()}
