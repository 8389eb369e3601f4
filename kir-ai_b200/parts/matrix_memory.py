"""A matrix memory with exponential gates (the mLSTM cell of xLSTM).

Per head, with q = W_q h * d^(-1/2), k = W_k h (d columns) and v = W_v h (dv columns): a log input gate
i = c tanh((W_i h + b_i) / c) and a log forget gate f = logsigmoid(c tanh((W_f h + b_f) / c)), c = ``gate_cap``; a
running maximum m_t = max(f + m_{t-1}, i), which starts at 0; the memory S_t = exp(f + m_{t-1} - m_t) S_{t-1} +
exp(i - m_t) k v^T and a normaliser n_t, the same with k alone; the read-out o = S_t^T q / (max(|n_t . q|, exp(-m_t))
+ 1e-6).  Each head's o is divided by its root mean square (eps inside the root); the heads side by side are
multiplied by a weight per column and by sigmoid(W_g h), then projected out.

One stacked product gives q, k, v, the two gates' pre-activations and the output gate's, in 32-bit.  What a request
keeps between steps is one slot row in 32-bit: S [H, d, dv], n [H, d], m [H], all zero at a sequence's start.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Mixer, Runtime, StateNeed, WeightSpec
from .linear import Linear


class MatrixMemory(Mixer):
    capture_safe = True  # slots and row boundaries are read on the device; a step of single tokens walks one token
    kernels_only = True

    def __init__(self, prefix: str, hidden_size: int, heads: int, key_dim: int, value_dim: int, gate_cap: float, eps: float,
                 names: Optional[Dict[str, str]] = None, out_dtype: Optional[torch.dtype] = None):
        if not gate_cap > 0.0:
            raise ValueError(f"the cap on the gates must be positive, got {gate_cap}")
        n = {"q": "q", "k": "k", "v": "v", "i": "i", "f": "f", "g": "g", "o": "o", "i_bias": "i.b", "f_bias": "f.b", "norm": "norm"}
        n.update(names or {})
        self.hidden_size, self.heads, self.key_dim, self.value_dim = hidden_size, heads, key_dim, value_dim
        self.gate_cap, self.eps, self.out_dtype = float(gate_cap), float(eps), out_dtype
        self.inputs = Linear([(prefix + n["q"], heads * key_dim), (prefix + n["k"], heads * key_dim), (prefix + n["v"], heads * value_dim),
                              (prefix + n["i"], heads), (prefix + n["f"], heads), (prefix + n["g"], heads * value_dim)], hidden_size)
        self.out = Linear([(prefix + n["o"], hidden_size)], heads * value_dim)
        self.names = {key: prefix + value for key, value in n.items()}
        self.gate_at = heads * (2 * key_dim + value_dim + 2)
        self.i_bias = self.f_bias = self.norm = None

    def cache_need(self) -> StateNeed:
        return StateNeed((self.heads * (self.key_dim * self.value_dim + self.key_dim + 1),), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        return {**self.inputs.weight_specs(), **self.out.weight_specs(), n["i_bias"]: WeightSpec((self.heads,), "bias"),
                n["f_bias"]: WeightSpec((self.heads,), "bias"), n["norm"]: WeightSpec((self.heads * self.value_dim,), "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.inputs.load(weights, rt)
        self.out.load(weights, rt)
        self.i_bias = weights.on_device(self.names["i_bias"], torch.float32)
        self.f_bias = weights.on_device(self.names["f_bias"], torch.float32)
        self.norm = weights.on_device(self.names["norm"], torch.float32)

    def forward(self, x, batch, cache, write_cache: bool = True) -> torch.Tensor:
        ops = self.rt.ops
        rows = self.inputs.forward(x, torch.float32)
        o = ops.matrix_memory_walk(rows, self.i_bias, self.f_bias, self.gate_cap, self.key_dim ** -0.5, cache.state, batch,
                                   self.heads, self.key_dim, self.value_dim)
        normed = ops.gated_group_norm(o, rows[:, self.gate_at :], self.norm, self.eps, self.heads, False, self.rt.dtype)
        return self.out.forward(normed, self.out_dtype)
