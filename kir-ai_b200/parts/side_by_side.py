"""Two mixers side by side on the same rows: out = (rms(left(h)) * w_left + rms(right(h)) * w_right) / 2, each output
divided by its root mean square over the model width (eps inside the root) and multiplied by a plain weight of its own.

Each side keeps what it needs (pages for attention, a state slot for a recurrence): ``cache_need()`` is the tuple of
both needs, the layer call names a cache layer for each, and ``forward`` gets the tuple of views.  Both sides are built
to leave 32-bit rows; the mean is 32-bit.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import Mixer, Runtime, WeightSpec


class SideBySideMixer(Mixer):
    def __init__(self, left: Mixer, right: Mixer, hidden_size: int, left_weight: str, right_weight: str, eps: float):
        self.left, self.right, self.hidden_size, self.eps = left, right, hidden_size, float(eps)
        self.left_weight_name, self.right_weight_name = left_weight, right_weight
        self.left_weight = self.right_weight = None
        if left.cache_need() is None or right.cache_need() is None:
            raise ValueError("both sides keep something between steps in this arrangement")

    @property
    def capture_safe(self) -> bool:
        return bool(self.left.capture_safe) and bool(self.right.capture_safe)

    @property
    def kernels_only(self) -> bool:
        return bool(self.left.kernels_only) and bool(self.right.kernels_only)

    def cache_need(self):
        return (self.left.cache_need(), self.right.cache_need())

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {**self.left.weight_specs(), **self.right.weight_specs(),
                self.left_weight_name: WeightSpec((self.hidden_size,), "norm"),
                self.right_weight_name: WeightSpec((self.hidden_size,), "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.left.load(weights, rt)
        self.right.load(weights, rt)
        self.left_weight = weights.on_device(self.left_weight_name, torch.float32)
        self.right_weight = weights.on_device(self.right_weight_name, torch.float32)

    def forward(self, x, batch, cache, write_cache: bool = True) -> torch.Tensor:
        left_view, right_view = cache
        a = self.left.forward(x, batch, left_view, write_cache)
        b = self.right.forward(x, batch, right_view, write_cache)
        a = a if a.dtype == torch.float32 else a.float()
        b = b if b.dtype == torch.float32 else b.float()
        return self.rt.ops.rms_pair_mean(a, b, self.left_weight, self.right_weight, self.eps)
