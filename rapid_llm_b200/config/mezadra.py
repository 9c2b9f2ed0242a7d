"""Configuration of the Mezadra decoder: a list of layers, each a softmax-attention or a linear-attention mixer
with a dense or a routed feed-forward (or none).

``config.json`` gives ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``: one entry a layer,
``type`` names the mixer (``attention`` or ``lightning``), ``mixer`` its sizes and constants, ``mlp`` the
feed-forward (``kind`` ``dense`` or ``moe``) or ``null``.  Layer ``i``'s tensors start with ``l<i>.``.

What the parts are built from:

* every layer is the arrangement ``outnorm``: ``x += norm1(mixer(x)); x += norm2(ff(x))``, weighted RMS norms on
  the sublayers' outputs, the float32 stream opened by the scaled embedding;
* ``attention`` -> ``gqa_attention`` on its convolution path: short convolutions on q, k, v behind the
  projections, rotation of the first ``rot.dims`` entries from frequencies ``rot.base^(-2i / dims)``, a weightless
  norm of q and k after it, ``scale`` and ``softcap`` on the scores, a sink per head, and, in layers with
  ``v_mix``, values blended with those of the first such layer;
* ``lightning`` -> ``lightning`` (a fixed ``decay`` per head);
* ``dense`` -> ``clamped_glu`` (``ff``, ``limit``); ``moe`` -> ``routed_experts`` (``router.experts``,
  ``router.top``, ``expert.ff``, an optional ``shared.ff`` with a sigmoid gate per token).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20     # nothing tabulated bounds a sequence; the engine's max_seq_len does

MIXER_TYPES = ("attention", "lightning")
MLP_KINDS = ("dense", "moe")


@dataclass
class MezadraConfig:
    architecture = "Mezadra"
    model_type = "mezadra"

    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: list[dict[str, Any]]
    raw: dict[str, Any] = field(default_factory=dict)

    # -------------------------------------------------------------- reading #
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], overrides: Mapping[str, Any] | None = None) -> "MezadraConfig":
        raw = copy.deepcopy(dict(raw))
        raw.update(copy.deepcopy(dict(overrides or {})))
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ValueError(f"config.json of a Mezadra model lacks {key!r}")
        config = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                     embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                     layers=list(raw["layers"]), raw=raw)
        config.validate()
        return config

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a Mezadra model needs at least one layer")
        mixed_widths = set()
        for index, layer in enumerate(self.layers):
            if layer.get("type") not in MIXER_TYPES:
                raise ValueError(f"layer {index}: unknown mixer type {layer.get('type')!r}")
            mixer = layer.get("mixer") or {}
            if layer["type"] == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim", "scale"):
                    if key not in mixer:
                        raise ValueError(f"layer {index}: the attention mixer lacks {key!r}")
                if mixer.get("v_mix"):
                    mixed_widths.add((int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])))
            else:
                for key in ("heads", "dim", "vdim", "decay"):
                    if key not in mixer:
                        raise ValueError(f"layer {index}: the lightning mixer lacks {key!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in MLP_KINDS:
                raise ValueError(f"layer {index}: unknown feed-forward kind {mlp.get('kind')!r}")
        if len(mixed_widths) > 1:
            raise ValueError(f"layers that blend their values must agree on kv heads and head sizes, got {sorted(mixed_widths)}")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                "layers": copy.deepcopy(self.layers)}

    # ----------------------------------------------------------------- spec #
    def _mixer(self, layer: Mapping[str, Any], first_mixing: bool) -> PartSpec:
        sizes = layer["mixer"]
        if layer["type"] == "lightning":
            return PartSpec("lightning", {
                "hidden_size": self.width, "num_heads": int(sizes["heads"]), "key_dim": int(sizes["dim"]),
                "value_dim": int(sizes["vdim"]), "decay": tuple(float(d) for d in sizes["decay"]), "norm_eps": self.norm_eps,
            })
        rot = sizes.get("rot") or {}
        value_mix = None
        if sizes.get("v_mix"):
            value_mix = "first" if first_mixing else "later"
        return PartSpec("gqa_attention", {
            "hidden_size": self.width, "num_heads": int(sizes["heads"]), "num_kv_heads": int(sizes["kv_heads"]),
            "head_dim": int(sizes["dim"]), "value_dim": int(sizes["vdim"]), "scale": float(sizes["scale"]),
            "qk_norm": False, "qk_norm_eps": self.norm_eps, "unit_after_rotation": True,
            "conv_width": int(sizes.get("conv", 0)), "softcap": float(sizes.get("softcap") or 0.0), "sink": True,
            "value_mix": value_mix,
            "position": PartSpec("rotary_frequencies", {
                "rotary_dim": int(rot.get("dims", 0)), "theta": float(rot.get("base", 10000.0)), "max_positions": MAX_POSITIONS}),
            "names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                      "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "sink": "sink", "value_mix": "vmix"},
        })

    def _feed_forward(self, mlp: Mapping[str, Any] | None) -> PartSpec | None:
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return PartSpec("clamped_glu", {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                                            "limit": float(mlp["limit"])})
        shared = mlp.get("shared") or None
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "num_experts": int(mlp["router"]["experts"]), "top_k": int(mlp["router"]["top"]),
            "expert_size": int(mlp["expert"]["ff"]), "shared_size": None if shared is None else int(shared["ff"]),
            "shared_gate": shared is not None, "scale_input": True,
        })

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": ""})
        names = {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."}
        layers, mixing_seen = [], False
        for index, layer in enumerate(self.layers):
            mixes = layer["type"] == "attention" and bool(layer["mixer"].get("v_mix"))
            layers.append(LayerSpec(arrangement="outnorm", mixer=self._mixer(layer, mixes and not mixing_seen),
                                    feed_forward=self._feed_forward(layer.get("mlp")), norm=norm, prefix=f"l{index}.",
                                    names=names))
            mixing_seen = mixing_seen or mixes
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "",
                                                   "scale": self.embedding_scale, "opens_stream": True}),
            layers=tuple(layers), schedule=tuple(ScheduleEntry(index) for index in range(len(layers))), final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False, "name": ""}),
            final_norm_prefix="final.norm", embedding_prefix="embed", head_prefix="head",
        )
        spec.validate()
        return spec
