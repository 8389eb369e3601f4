"""RMSNorm and layer norm with the residual add fused in.

y = x * 1/sqrt(mean(x^2) + eps) * w, statistics in 32-bit, the scale 0 when
mean + eps is 0 (crates/llm-backend/src/core/math.rs:73-113 of the reference; the
dense model uses the plain weight, crates/llm-backend/src/core/qwen/ops/norm.rs:119-133).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from .base import FusedNormSpec, Norm, NormedSum, Runtime, ScaledSum, WeightSpec


class RMSNorm(Norm):
    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, width: int, eps: float, centre: float = 0.0):
        """``centre`` c: the stored tensor w is the weight's distance from c, y = x / rms(x) * (c + w); a tensor that holds
        the weight minus one has c = 1.  The sum is formed once, in 32-bit, at load."""
        self.weight_name = weight_name
        self.width = width
        self.eps = float(eps)
        self.centre = float(centre)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), "bias" if self.centre else "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = weights.on_device(self.weight_name, torch.float32)
        if self.centre:
            self.weight = (self.weight + self.centre).contiguous()

    takes_normed_sum = True  # add_forward and add_forward_rows take a ``NormedSum`` (base.py)

    def add_forward(self, resid: torch.Tensor, delta) -> torch.Tensor:
        if isinstance(delta, NormedSum):
            # the stream takes the sub-layer's normed output and leaves under this norm in one pass over the row
            return self.rt.ops.norm_add_norm(resid, delta.rows, delta.weight, delta.eps, self.weight, self.eps, self.rt.dtype)
        return self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, self.rt.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.rt.ops.add_rmsnorm(x, None, self.weight, self.eps, self.rt.dtype)

    def add_normed(self, resid: torch.Tensor, y: torch.Tensor) -> Optional[torch.Tensor]:
        if y.dtype != torch.float32:
            y = y.float()
        return self.rt.ops.norm_add(resid, y, self.weight, self.eps, None if self.rt.dtype == torch.float32 else self.rt.dtype)

    def fused_spec(self) -> Optional[FusedNormSpec]:
        # the tensor-core products read and write rows in 16-byte units; KIRAI_FUSE_NORMS=0 keeps every norm a
        # kernel of its own (for comparing the two paths)
        if self.rt.dtype != torch.bfloat16 or self.width % 8 or os.environ.get("KIRAI_FUSE_NORMS", "1") == "0":
            return None
        return FusedNormSpec(self.weight, self.eps, self.width)

    def add_forward_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """The norm of ``resid[rows] + delta[rows]`` only; the stream is left untouched."""
        if isinstance(delta, NormedSum):
            return self.rt.ops.norm_add_norm(resid, delta.rows, delta.weight, delta.eps, self.weight, self.eps, self.rt.dtype,
                                             row_index=rows)
        out, _ = self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, self.rt.dtype, row_index=rows)
        return out

    def normed_sum(self, y: torch.Tensor) -> "NormedSum":
        """What is left to add when this norm stands on a sub-layer's OUTPUT ``y`` (32-bit rows) and whoever reads the
        stream next adds it."""
        return NormedSum(y if y.dtype == torch.float32 else y.float(), self.weight, self.eps)


class LayerNorm(Norm):
    """Layer norm with a weight and no bias: y = (x - mean) / sqrt(var + eps) * w, var the mean of the squared
    deviations from the mean, statistics in 32-bit.  ``add_forward`` may also take a bias [width] of the sub-layer
    whose output it adds (``takes_delta_bias``), and can leave its rows in 32-bit for a step that goes on in 32-bit
    (``wide``: a token shift).  It is a kernel of its own: no product takes it over."""

    capture_safe = True
    kernels_only = True
    takes_delta_bias = True
    fuses_shift = True  # add_forward(shift=...) runs a token shift of single-token steps inside the norm's kernel

    def __init__(self, weight_name: str, width: int, eps: float):
        self.weight_name = weight_name
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = weights.on_device(self.weight_name, torch.float32)

    def add_forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], delta_bias: Optional[torch.Tensor] = None,
                    wide: bool = False, shift: Optional[tuple] = None) -> torch.Tensor:
        return self.rt.ops.add_layernorm(resid, delta, self.weight, self.eps, self.rt.dtype, delta_bias=delta_bias, wide=wide,
                                         shift=shift)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.rt.ops.add_layernorm(x, None, self.weight, self.eps, self.rt.dtype)

    def add_forward_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """The norm of ``resid[rows] + delta[rows]`` only; the stream is left untouched."""
        return self.rt.ops.add_layernorm(resid, delta, self.weight, self.eps, self.rt.dtype, row_index=rows)


class DynamicTanh(Norm):
    """Dynamic Tanh in the place of a norm: y = tanh(alpha * x) * weight + bias, element by element, with a learned
    scalar ``alpha``; no mean or variance of the row is taken.  The tensors are ``<name>`` (weight), ``<name>.alpha``
    (a scalar) and ``<name>.b``.  ``add_forward`` adds what the sub-layer before left (a tensor, or a ``ScaledSum``)
    into the 32-bit stream in the same pass.  A kernel of its own: there is no 1 / rms factor a product could take
    over."""

    capture_safe = True
    kernels_only = True
    takes_scaled_sum = True

    def __init__(self, weight_name: str, width: int, alpha_name: Optional[str] = None, bias_name: Optional[str] = None):
        self.weight_name, self.width = weight_name, width
        self.alpha_name = alpha_name or weight_name + ".alpha"
        self.bias_name = bias_name or weight_name + ".b"
        self.weight = self.alpha = self.bias = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), "norm"), self.alpha_name: WeightSpec((), "norm"),
                self.bias_name: WeightSpec((self.width,), "bias")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = weights.on_device(self.weight_name, torch.float32)
        self.alpha = weights.on_device(self.alpha_name, torch.float32).reshape(1).contiguous()
        self.bias = weights.on_device(self.bias_name, torch.float32)

    @staticmethod
    def _terms(delta):
        if delta is None:
            return [], 1.0
        if isinstance(delta, ScaledSum):
            return list(delta.rows), float(delta.factor)
        return [delta if delta.dtype == torch.float32 else delta.float()], 1.0

    def add_forward(self, resid: torch.Tensor, delta=None) -> torch.Tensor:
        rows, factor = self._terms(delta)
        return self.rt.ops.add_dyt(resid, rows, factor, self.alpha, self.weight, self.bias, self.rt.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.rt.ops.add_dyt(x, [], 1.0, self.alpha, self.weight, self.bias, self.rt.dtype)

    def add_forward_rows(self, resid: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        """The rows ``rows`` of the stream plus what is left to add, through the form; the stream is left untouched."""
        terms, factor = self._terms(delta)
        return self.rt.ops.add_dyt(resid, terms, factor, self.alpha, self.weight, self.bias, self.rt.dtype, row_index=rows)
