"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``.

Gate and up share one product over a fused ``[2I, H]`` weight, gate rows first
(``rapid_llm/modules/mlp.py:52-68``, ``rapid_llm/modules/linear.py:157-172``);
``silu(z) = z * sigmoid(z)`` in float32 (``rapid_llm/kernels/ops/activation/swiglu.py:91-121``).
No biases.
"""

from __future__ import annotations

import torch

from ..ops import gemm, kernels
from .base import FEED_FORWARDS, MATRIX, VECTOR, FeedForward, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    rides_norms = True

    def __init__(self, *, hidden_size: int, intermediate_size: int, dtype, device,
                 gate_name: str = "gate_proj", up_name: str = "up_proj", down_name: str = "down_proj",
                 suffix: str = ".weight") -> None:
        super().__init__(dtype=dtype, device=device)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.names = (gate_name + suffix, up_name + suffix, down_name + suffix)     # the tensors' names after the prefix
        self.gate_up = self.new_storage((2 * self.inter, self.hidden), MATRIX)
        self.down = self.new_storage((self.hidden, self.inter), MATRIX)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        gate, up, down = self.names
        return {
            gate: TensorSpec((self.inter, self.hidden)),
            up: TensorSpec((self.inter, self.hidden)),
            down: TensorSpec((self.hidden, self.inter)),
        }

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        gate, up, down = self.names
        if name == gate:
            self.gate_up[: self.inter].copy_(tensor)
        elif name == up:
            self.gate_up[self.inter :].copy_(tensor)
        elif name == down:
            self.down.copy_(tensor)
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        return (self.gate_up.numel() + self.down.numel()) * self.gate_up.element_size()

    def workspace_elements_per_token(self) -> int:
        return 3 * self.inter + self.hidden          # gate and up of a library-product step, act, out

    def forward(self, x, batch, then_norm=None):
        rows = x.shape[0]
        act = batch.workspace.get("ffn_act", rows, self.inter, x.dtype)
        gemm.gated_linear(x, self.gate_up, act, batch.workspace, batch.fault, defer=batch.defer_products)
        out = batch.workspace.get("ffn_out", rows, self.hidden, x.dtype)
        return gemm.linear(act, self.down, out, batch.fault, then_norm=then_norm, defer=batch.defer_products)


    def uses_libraries(self) -> set[str]:
        return {"gemm"} if self.dtype == torch.bfloat16 else set()


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(SwiGLU):
    """``down(g * sigmoid(alpha g) * (u + 1))`` with ``g = min(gate(x), limit)`` and ``u = clamp(up(x), -limit, limit)``:
    a gated unit whose branches are bounded before they meet, the linear branch shifted by one.  Gate and up
    share one product as in :class:`SwiGLU`, and the unit rides in its epilogue where :class:`SwiGLU`'s does (float32
    arithmetic on the accumulators); elsewhere it is a kernel on the product's result."""

    rides_norms = False

    def __init__(self, *, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702, dtype, device,
                 gate_name: str = "gate", up_name: str = "up", down_name: str = "down", suffix: str = "") -> None:
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, dtype=dtype, device=device,
                         gate_name=gate_name, up_name=up_name, down_name=down_name, suffix=suffix)
        self.limit, self.alpha = float(limit), float(alpha)

    def forward(self, x, batch):
        rows = x.shape[0]
        act = batch.workspace.get("ffn_act", rows, self.inter, x.dtype)
        gemm.gated_linear(x, self.gate_up, act, batch.workspace, batch.fault, clamp=(self.limit, self.alpha))
        return gemm.linear(act, self.down, batch.workspace.get("ffn_out", rows, self.hidden, x.dtype), batch.fault)


# activation name -> (number of learned scalars, kernel over [T, I] rows)
ACTIVATIONS = {"xielu": (2, kernels.xielu)}


@FEED_FORWARDS.register("dense")
class DenseFeedForward(FeedForward):
    """``down(act(up(x)))`` without gate and biases; the activation may have learned scalars of its own.

    ``xielu``: with the two scalars ``p, q`` of the activation's tensor, ``z > 0: softplus(p) z^2 + z / 2`` and
    ``z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` (float32 arithmetic on the product's result).
    """

    def __init__(self, *, hidden_size: int, intermediate_size: int, activation: str, dtype, device,
                 up_name: str = "up", down_name: str = "down", act_name: str = "act") -> None:
        super().__init__(dtype=dtype, device=device)
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ACTIVATIONS)}")
        self.hidden, self.inter, self.activation = int(hidden_size), int(intermediate_size), activation
        self.names = (up_name, down_name, act_name)
        self.up = self.new_storage((self.inter, self.hidden), MATRIX)
        self.down = self.new_storage((self.hidden, self.inter), MATRIX)
        self.scalars = self.new_storage((ACTIVATIONS[activation][0],), VECTOR)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        up, down, act = self.names
        return {
            up: TensorSpec((self.inter, self.hidden)),
            down: TensorSpec((self.hidden, self.inter)),
            act: TensorSpec(tuple(self.scalars.shape), VECTOR),
        }

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        up, down, act = self.names
        if name == up:
            self.up.copy_(tensor)
        elif name == down:
            self.down.copy_(tensor)
        elif name == act:
            self.scalars.copy_(tensor.to(torch.float32))
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        return (self.up.numel() + self.down.numel()) * self.up.element_size() + self.scalars.numel() * 4

    def workspace_elements_per_token(self) -> int:
        return 2 * self.inter + self.hidden

    def uses_libraries(self) -> set[str]:
        return {"recurrent"} | ({"gemm"} if self.dtype == torch.bfloat16 else set())

    def forward(self, x, batch):
        rows = x.shape[0]
        wide = batch.workspace.get("ffn_up", rows, self.inter, x.dtype)
        gemm.linear(x, self.up, wide, batch.fault)
        act = batch.workspace.get("ffn_act", rows, self.inter, x.dtype)
        ACTIVATIONS[self.activation][1](wide, act, self.scalars)
        out = batch.workspace.get("ffn_out", rows, self.hidden, x.dtype)
        return gemm.linear(act, self.down, out, batch.fault)
