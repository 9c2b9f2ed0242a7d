"""Two mixers side by side on the same input: ``y = left_scale * Left(x) + right_scale * Right(x)``.

Either side is any registered mixer (given as a nested :class:`PartSpec`); their tensors live under the
sub-prefixes ``left.`` and ``right.``.  What they need from the engine is combined: at most one side may ask
for cache pages (the layer has one cache group), the sides' state rows lie one behind the other in the
layer's state row, and at most one side may plan work on the host.
"""

from __future__ import annotations

import dataclasses

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from .base import MIXERS, Mixer, StateNeed, TensorSpec


@MIXERS.register("parallel")
class ParallelMixers(Mixer):
    def __init__(self, *, left: PartSpec, right: PartSpec, left_scale: float, right_scale: float, hidden_size: int,
                 left_prefix: str = "left.", right_prefix: str = "right.", dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.hidden = int(hidden_size)
        self.scales = (float(left_scale), float(right_scale))
        self.sides = (
            (left_prefix, MIXERS.build(left, dtype=dtype, device=device)),
            (right_prefix, MIXERS.build(right, dtype=dtype, device=device)),
        )
        if sum(part.cache_need() is not None for _, part in self.sides) > 1:
            raise ValueError("only one of two parallel mixers may keep cache pages")
        if sum(part.step_planner() is not None for _, part in self.sides) > 1:
            raise ValueError("only one of two parallel mixers may plan work on the host")
        needs = [part.state_need() for _, part in self.sides]
        if any(need is not None and (need.dtype != torch.float32 or len(need.shape) != 1) for need in needs):
            raise ValueError("parallel mixers share a state row of float32 numbers")
        self.state_sizes = [0 if need is None else int(need.shape[0]) for need in needs]

    # -- needs ----------------------------------------------------------------- #
    def cache_need(self):
        for _, part in self.sides:
            if part.cache_need() is not None:
                return part.cache_need()
        return None

    def state_need(self):
        total = sum(self.state_sizes)
        return StateNeed((total,), torch.float32) if total else None

    def step_planner(self):
        for _, part in self.sides:
            if part.step_planner() is not None:
                return part.step_planner()
        return None

    def uses_libraries(self) -> set[str]:
        return {"recurrent"} | self.sides[0][1].uses_libraries() | self.sides[1][1].uses_libraries()

    # -- weights --------------------------------------------------------------- #
    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {prefix + name: spec for prefix, part in self.sides for name, spec in part.tensor_specs().items()}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        for prefix, part in self.sides:
            if name.startswith(prefix):
                part.load_tensor(name[len(prefix):], tensor)
                return
        raise KeyError(name)

    def finalize(self, loaded: set[str]) -> None:
        for prefix, part in self.sides:
            part.finalize({name[len(prefix):] for name in loaded if name.startswith(prefix)})

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for _, part in self.sides)

    def workspace_elements_per_token(self) -> int:
        return sum(part.workspace_elements_per_token() for _, part in self.sides) + self.hidden

    # -- forward --------------------------------------------------------------- #
    def forward(self, x, batch, cache):
        results, at = [], 0
        for (_, part), size in zip(self.sides, self.state_sizes):
            state = None if not size else cache.state[:, at : at + size]
            at += size
            results.append(part.forward(x, batch, dataclasses.replace(cache, state=state)))
        out = batch.workspace.get("parallel_out", x.shape[0], self.hidden, x.dtype)
        return kernels.scaled_sum(results[0], results[1], self.scales[0], self.scales[1], out)
