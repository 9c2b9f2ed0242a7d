"""Small Mezadra configurations and seeded weights for the tests.

The weights are drawn so that every mechanism carries weight: sinks of the scores' size, blending weights
between 0.2 and 0.8, peaked attention (scores reach the cap), gate and up products on both sides of their
limit.  Every value is rounded to bfloat16 once, so a folder written in either precision and the float64
plain implementation hold the same numbers.
"""

from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def dense(ff=40, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=5, top=2, ff=24, shared=16):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def attention_layer(*, heads=4, kv_heads=2, dim=32, vdim=16, conv=3, rot_dims=8, base=100.0, scale=0.4, softcap=6.0,
                    v_mix=False, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
             "rot": {"dims": rot_dims, "base": base}, "scale": scale, "softcap": softcap, "v_mix": v_mix}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def lightning_layer(*, heads=3, dim=16, vdim=24, decay=(0.8, 0.95, 0.999), mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def make_config(layers, *, width=64, vocab=97, eps=1e-5, scale=3.0) -> dict:
    return {"architecture": "Mezadra", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "layers": copy.deepcopy(list(layers))}


CONFIGS = {
    # one mechanism a model
    "attention": make_config([attention_layer(mlp=dense())], width=64),
    "lightning": make_config([lightning_layer(mlp=dense(ff=36, limit=0.7))], width=48, vocab=61),
    "experts": make_config([lightning_layer(heads=2, dim=8, vdim=8, decay=(0.9, 0.5), mlp=moe())], width=40, vocab=70),
    # values blended over three layers (the first leaves them, two read them), other layers between them; heads of
    # 48 with values of 64; one tap; the whole head rotated, and none of it; a layer without a feed-forward
    "blend": make_config([
        attention_layer(heads=2, kv_heads=1, dim=48, vdim=64, conv=2, rot_dims=48, v_mix=True, mlp=moe(experts=3, top=1, ff=16, shared=0)),
        lightning_layer(mlp=None),
        attention_layer(heads=3, kv_heads=1, dim=48, vdim=64, conv=1, rot_dims=0, softcap=2.0, v_mix=True, mlp=dense(ff=24)),
        attention_layer(heads=4, kv_heads=4, dim=16, vdim=16, conv=4, rot_dims=4, scale=1.0, softcap=30.0, mlp=None),
        attention_layer(heads=1, kv_heads=1, dim=48, vdim=64, conv=5, rot_dims=16, base=1.0e6, v_mix=True, mlp=moe(experts=4, top=4, ff=8, shared=8)),
    ], width=72, vocab=130),
    # nothing is a multiple of 4: every kernel's element-by-element path
    "narrow": make_config([
        lightning_layer(heads=3, dim=6, vdim=10, decay=(1.0, 0.97, 0.3), mlp=moe(experts=7, top=3, ff=10, shared=6)),
        attention_layer(heads=3, kv_heads=3, dim=10, vdim=6, conv=2, rot_dims=6, scale=0.7, softcap=4.0, mlp=dense(ff=22, limit=0.9)),
        attention_layer(heads=2, kv_heads=1, dim=14, vdim=22, conv=3, rot_dims=2, v_mix=True, mlp=moe(experts=1, top=1, ff=14, shared=0)),
    ], width=50, vocab=83, eps=1e-6, scale=1.0),
}


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    width = config["width"]
    shapes = {"embed": (config["vocab"], width), "final.norm": (width,), "head": (config["vocab"], width)}
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        shapes[p + "norm1"] = (width,)
        if layer["type"] == "attention":
            hq, hk, hv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            shapes.update({p + "mix.q": (hq, width), p + "mix.k": (hk, width), p + "mix.v": (hv, width),
                           p + "mix.q.conv": (hq, m["conv"]), p + "mix.k.conv": (hk, m["conv"]), p + "mix.v.conv": (hv, m["conv"]),
                           p + "mix.sink": (m["heads"],), p + "mix.o": (width, m["heads"] * m["vdim"])})
            if m.get("v_mix"):
                shapes[p + "mix.vmix"] = ()
        else:
            hk, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            shapes.update({p + "mix.q": (hk, width), p + "mix.k": (hk, width), p + "mix.v": (hv, width), p + "mix.g": (hv, width),
                           p + "mix.o": (width, hv), p + "mix.norm": (hv,)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = (width,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], width), p + "mlp.up": (mlp["ff"], width), p + "mlp.down": (width, mlp["ff"])})
            continue
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            shapes.update({f"{p}mlp.e{e}.gate": (ff, width), f"{p}mlp.e{e}.up": (ff, width), f"{p}mlp.e{e}.down": (width, ff)})
        shapes[p + "mlp.router"] = (mlp["router"]["experts"], width)
        if mlp.get("shared"):
            ff = mlp["shared"]["ff"]
            shapes.update({p + "mlp.shared.gate": (ff, width), p + "mlp.shared.up": (ff, width),
                           p + "mlp.shared.down": (width, ff), p + "mlp.shared.sg": (1, width)})
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
        elif last in ("norm", "norm1", "norm2"):
            value = 1.0 + 0.2 * draw
        elif last == "conv":
            value = 0.6 * draw
        elif last == "sink":
            value = 1.5 * draw
        elif last == "vmix":
            value = 0.2 + 0.6 * torch.rand((), generator=generator)
        else:
            value = draw / math.sqrt(shape[-1])
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
