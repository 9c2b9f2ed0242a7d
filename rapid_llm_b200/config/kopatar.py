"""Configuration of the Kopatar decoder: a list of layers of three mixer kinds, part of it run in a loop.

``config.json`` gives ``vocab``, ``width``, ``norm.eps``, ``layers`` (one entry a layer: ``type`` names the
mixer, ``mixer`` its sizes, ``mlp`` the feed-forward or ``null``) and ``loop`` (layers ``start .. stop - 1``
run ``times`` times in a row with the same weights; every pass has a cache and state of its own; before every
pass but the first the embedding's output joins the stream, and before every pass row ``t`` of ``loop.step``).
Low-rank sizes that the file does not name are read from the tensors' shapes.

Mixer types and the parts they become: ``channel_delta`` -> ``gated_delta_rule``; ``retention`` ->
``retention``; ``parallel`` -> ``parallel`` of a windowed ``gqa_attention`` without rotation, with q/k norm
and a sigmoid output gate (left), and a ``state_space_dual`` (right).  Layers are pre-norm blocks; the head is
the embedding table.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping

from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20     # no learned or tabulated positions bound a sequence; the engine's max_seq_len does


@dataclass
class KopatarConfig:
    architecture = "Kopatar"
    model_type = "kopatar"

    vocab: int
    width: int
    norm_eps: float
    layers: list[dict[str, Any]]
    loop: dict[str, int] | None = None
    ranks: dict[int, tuple[int, int]] = field(default_factory=dict)   # layer -> (decay rank, gate rank)
    raw: dict[str, Any] = field(default_factory=dict)

    # -------------------------------------------------------------- reading #
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], overrides: Mapping[str, Any] | None = None) -> "KopatarConfig":
        raw = copy.deepcopy(dict(raw))
        raw.update(copy.deepcopy(dict(overrides or {})))
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ValueError(f"config.json of a Kopatar model lacks {key!r}")
        ranks = {int(layer): (int(pair[0]), int(pair[1])) for layer, pair in (raw.get("ranks") or {}).items()}
        config = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                     layers=list(raw["layers"]), loop=raw.get("loop") or None, ranks=ranks, raw=raw)
        config.validate()
        return config

    @classmethod
    def from_folder(cls, model_dir: str | Path, raw: Mapping[str, Any], overrides=None) -> "KopatarConfig":
        """As :meth:`from_dict`, with the low-rank sizes of ``channel_delta`` layers read from the header of
        the folder's ``model.safetensors`` (the file's JSON gives every tensor's shape)."""
        raw = dict(raw)
        if "ranks" not in raw:
            shapes = _tensor_shapes(Path(model_dir))
            ranks = {}
            for index, layer in enumerate(raw.get("layers", [])):
                if layer.get("type") == "channel_delta":
                    a1, g1 = shapes.get(f"l{index}.mix.a1"), shapes.get(f"l{index}.mix.g1")
                    if a1 is None or g1 is None:
                        raise ValueError(f"model.safetensors lacks l{index}.mix.a1 / g1, which give the layer's low-rank sizes")
                    ranks[str(index)] = [int(a1[0]), int(g1[0])]
            raw["ranks"] = ranks
        return cls.from_dict(raw, overrides)

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a Kopatar model needs at least one layer")
        for index, layer in enumerate(self.layers):
            if layer.get("type") not in ("channel_delta", "retention", "parallel"):
                raise ValueError(f"layer {index}: unknown mixer type {layer.get('type')!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ValueError(f"layer {index}: unknown feed-forward kind {mlp.get('kind')!r}")
            if layer["type"] == "channel_delta" and index not in self.ranks:
                raise ValueError(f"layer {index}: the low-rank sizes of its decay and gate are not known "
                                 "(config key 'ranks': {layer: [decay rank, gate rank]})")
        if self.loop:
            start, stop, times = (int(self.loop[key]) for key in ("start", "stop", "times"))
            if not 0 <= start < stop <= len(self.layers) or times < 1:
                raise ValueError(f"loop {self.loop} does not fit {len(self.layers)} layers")

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.loop:
            out["loop"] = dict(self.loop)
        out["ranks"] = {str(layer): list(pair) for layer, pair in self.ranks.items()}
        return out

    # ----------------------------------------------------------------- spec #
    def _mixer(self, index: int, layer: Mapping[str, Any]) -> PartSpec:
        kind, sizes = layer["type"], layer["mixer"]
        if kind == "channel_delta":
            return PartSpec("gated_delta_rule", {
                "hidden_size": self.width, "num_heads": sizes["heads"], "num_kv_heads": sizes["kv_heads"],
                "key_dim": sizes["dim"], "value_dim": sizes["vdim"], "conv_width": sizes["conv"],
                "decay_rank": self.ranks[index][0], "gate_rank": self.ranks[index][1], "norm_eps": self.norm_eps,
            })
        if kind == "retention":
            rot = sizes.get("rot") or {}
            return PartSpec("retention", {
                "hidden_size": self.width, "num_heads": sizes["heads"], "key_dim": sizes["dim"],
                "value_dim": sizes["vdim"], "decay": tuple(sizes["decay"]), "rotary_dims": int(rot.get("dims", 0)),
                "rotary_base": float(rot.get("base", 10000.0)), "norm_eps": self.norm_eps,
            })
        left, right = sizes["left"], sizes["right"]
        attention = PartSpec("gqa_attention", {
            "hidden_size": self.width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"],
            "head_dim": left["dim"], "value_dim": left["vdim"], "qk_norm": True, "qk_norm_eps": self.norm_eps,
            "window": int((left.get("mask") or {}).get("size", 0)), "scale": float(left["scale"]), "gate": "sigmoid",
            "position": PartSpec("none", {"max_positions": MAX_POSITIONS}),
            "names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                      "q_norm.weight": "q.norm", "k_norm.weight": "k.norm", "g_proj.weight": "g"},
        })
        state_space = PartSpec("state_space_dual", {
            "hidden_size": self.width, "num_heads": right["heads"], "head_dim": right["vdim"],
            "state_size": right["state"], "groups": right["groups"], "conv_width": right["conv"],
            "norm_groups": right["norm_groups"], "norm_eps": self.norm_eps,
        })
        return PartSpec("parallel", {
            "left": attention, "right": state_space, "left_scale": float(sizes["left_scale"]),
            "right_scale": float(sizes["right_scale"]), "hidden_size": self.width,
        })

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": ""})
        names = {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."}
        layers = []
        for index, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            feed_forward = None if mlp is None else PartSpec("dense", {
                "hidden_size": self.width, "intermediate_size": int(mlp["ff"]), "activation": "xielu"})
            layers.append(LayerSpec(arrangement="prenorm", mixer=self._mixer(index, layer), feed_forward=feed_forward,
                                    norm=norm, prefix=f"l{index}.", names=names))
        count = len(layers)
        if self.loop:
            start, stop, times = (int(self.loop[key]) for key in ("start", "stop", "times"))
            schedule = [ScheduleEntry(index) for index in range(start)]
            for number in range(times):
                schedule.append(ScheduleEntry(start, pass_index=number, add_embedding=number > 0))
                schedule.extend(ScheduleEntry(index) for index in range(start + 1, stop))
            schedule.extend(ScheduleEntry(index) for index in range(stop, count))
            offsets = PartSpec("pass_offset", {"passes": times, "hidden_size": self.width, "name": "step"})
        else:
            schedule, offsets = [ScheduleEntry(index) for index in range(count)], None
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": ""}),
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": True}),
            final_norm_prefix="final.norm", embedding_prefix="embed", head_prefix="head.",
            pass_offset=offsets, pass_offset_prefix="loop.",
        )
        spec.validate()
        return spec


def _tensor_shapes(model_dir: Path) -> dict[str, list[int]]:
    """Name -> shape from the header of ``model.safetensors`` (8 bytes of length, then that much JSON)."""
    path = model_dir / "model.safetensors"
    if not path.is_file():
        raise FileNotFoundError(f"no model.safetensors in {model_dir}")
    with open(path, "rb") as handle:
        length = int.from_bytes(handle.read(8), "little")
        header = json.loads(handle.read(length))
    return {name: entry["shape"] for name, entry in header.items() if name != "__metadata__"}
