"""A dense feed-forward without a gate: down(act(up x)), act(z) = relu(z)^2.  No biases.

The gated forms are ``parts.swiglu``; this one has a single input matrix, and its activation acts on every column by
itself.  On the tensor cores the activation is the epilogue of the up product where that kernel has it (steps of many
tokens), else a kernel of its own between the two products.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FeedForward, Runtime, WeightSpec
from .linear import Linear

ACTIVATIONS = ("relu2",)


class PlainMLP(FeedForward):
    capture_safe = True
    kernels_only = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "relu2",
                 names: Optional[Dict[str, str]] = None, out_dtype: Optional[torch.dtype] = None):
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {ACTIVATIONS}")
        n = {"up": "up_proj.weight", "down": "down_proj.weight"}
        n.update(names or {})
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.out_dtype = out_dtype  # of the result (default: the runtime's)
        self.up = Linear([(prefix + n["up"], intermediate_size)], hidden_size)
        self.down = Linear([(prefix + n["down"], hidden_size)], intermediate_size)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {**self.up.weight_specs(), **self.down.weight_specs()}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.up.load(weights, rt)
        self.down.load(weights, rt)

    def forward(self, x, batch=None) -> torch.Tensor:
        ops = self.rt.ops
        fused = getattr(ops, "linear_relu2", None)
        if fused is not None and self.up.on_tensor_cores() and ops.linear_relu2_takes(x, self.up.weight):
            hidden = fused(x, self.up.weight)
        else:
            hidden = ops.relu2_(self.up.forward(x))
        return self.down.forward(hidden, self.out_dtype)
