"""A state-space mixer in the manner of Mamba-2: a short causal convolution, then a recurrence whose state is a matrix
per head, S_t = a_t S_{t-1} + dt_t B_t x_t^T, read out as y_t = S_t^T C_t + D x_t.

One input product gives, side by side, the gate z [H P], the convolution's input [x: H P | B: G N | C: G N] and the
step sizes dt [H] (H heads of P columns, G groups of N state rows; head h uses group h // (H / G)).  x, B and C pass
a causal convolution per channel over ``conv_taps`` tokens (bias, then silu; the stored taps' last column weighs the
token itself, zeros lie before a sequence's start).  dt <- softplus(dt + dt_bias) without a clamp,
a = exp(-exp(A_log_h) dt).  y (heads side by side) times silu(z) is divided by its root mean square in
``norm_groups`` equal parts of the row (eps inside the root), multiplied by a weight per column and projected out:
the gate comes before the norm.

What a request keeps between steps is one slot row in 32-bit: the convolution's last ``conv_taps - 1`` input rows,
then the heads' states [H, N, P]; both start at zero.  The product's result, the convolution, the step sizes, decays
and the recurrence are 32-bit; only what the output product reads is rounded to the runtime dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Mixer, Runtime, StateNeed, WeightSpec
from .linear import Linear


class StateSpaceMixer(Mixer):
    capture_safe = True  # slots and row boundaries are read on the device; a step of single tokens walks one token
    kernels_only = True

    def __init__(self, prefix: str, hidden_size: int, heads: int, head_dim: int, state_size: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float, names: Optional[Dict[str, str]] = None, out_dtype: Optional[torch.dtype] = None):
        if heads % groups:
            raise ValueError(f"{heads} heads are not a multiple of {groups} groups")
        inner = heads * head_dim
        if inner % norm_groups:
            raise ValueError(f"{inner} columns do not split into {norm_groups} equal parts for the norm")
        if conv_taps < 1:
            raise ValueError("the convolution has at least one tap")
        n = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D", "norm": "norm",
             "o": "o"}
        n.update(names or {})
        self.hidden_size, self.heads, self.head_dim, self.state_size, self.groups = hidden_size, heads, head_dim, state_size, groups
        self.conv_taps, self.norm_groups, self.eps, self.out_dtype = conv_taps, norm_groups, float(eps), out_dtype
        self.inner = inner
        self.channels = inner + 2 * groups * state_size
        self.inputs = Linear([(prefix + n["in"], 2 * inner + 2 * groups * state_size + heads)], hidden_size)
        self.out = Linear([(prefix + n["o"], hidden_size)], inner)
        self.names = {key: prefix + value for key, value in n.items()}
        self.conv_len = (conv_taps - 1) * self.channels
        self.conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm = None

    def cache_need(self) -> StateNeed:
        return StateNeed((self.conv_len + self.heads * self.state_size * self.head_dim,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        return {**self.inputs.weight_specs(), **self.out.weight_specs(),
                n["conv"]: WeightSpec((self.channels, self.conv_taps), "linear"), n["conv_bias"]: WeightSpec((self.channels,), "bias"),
                n["dt_bias"]: WeightSpec((self.heads,), "bias"), n["a_log"]: WeightSpec((self.heads,), "bias"),
                n["skip"]: WeightSpec((self.heads,), "norm"), n["norm"]: WeightSpec((self.inner,), "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.inputs.load(weights, rt)
        self.out.load(weights, rt)
        for key in ("conv", "conv_bias", "dt_bias", "a_log", "skip", "norm"):
            setattr(self, key, weights.on_device(self.names[key], torch.float32))

    def forward(self, x, batch, cache, write_cache: bool = True) -> torch.Tensor:
        ops = self.rt.ops
        rows = self.inputs.forward(x, torch.float32)  # [T, z | x B C | dt]
        gate = rows[:, : self.inner]
        mixed = ops.conv_silu(rows[:, self.inner : self.inner + self.channels], self.conv, self.conv_bias, cache.state, 0, batch)
        y = ops.ssm_walk(mixed, rows[:, self.inner + self.channels :], self.dt_bias, self.a_log, self.skip, cache.state,
                         self.conv_len, batch, self.heads, self.groups, self.state_size, self.head_dim)
        normed = ops.gated_group_norm(y, gate, self.norm, self.eps, self.norm_groups, True, self.rt.dtype)
        return self.out.forward(normed, self.out_dtype)
