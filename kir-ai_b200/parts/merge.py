"""Where a stream starts over from itself and its origin: x <- W [x; x0] + b.

``StreamMerge`` stands between blocks, ahead of a run of layers (a pass of a looped stretch).  x is the residual
stream as the blocks before left it, x0 the stream as the embedding made it; W [width, 2 width] reads x in its first
``width`` columns and x0 in the others, and b is one row of a stored table [rows, width], chosen by the caller (the
number of the pass).  The result IS the new stream (32-bit: the product's 32-bit output, plus b in 32-bit).

How it runs: the two streams lie side by side in one buffer [T, 2 width] in the runtime dtype, which one product
reads; the origin's half is written once a step and serves every pass, the stream's half is written by the kernel that
also settles what the block before left to be added (a ``NormedSum``), so the stream is read once.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NormedSum, Part, Runtime, ScaledSum, StreamCopy, UnscaledNorm, WeightSpec
from .linear import Linear


class StreamMerge(Part):
    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, width: int, bias_name: Optional[str] = None, bias_rows: int = 1):
        self.width, self.bias_name, self.bias_rows = width, bias_name, bias_rows
        self.product = Linear([(weight_name, width)], 2 * width)
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = dict(self.product.weight_specs())
        if self.bias_name:
            specs[self.bias_name] = WeightSpec((self.bias_rows, self.width), "bias")
        return specs

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.product.load(weights, rt)
        if self.bias_name:
            self.bias = weights.on_device(self.bias_name, torch.float32)

    def begin(self, origin: torch.Tensor) -> torch.Tensor:
        """The buffer of a step, [T, 2 width] in the runtime dtype, with the origin in its second half."""
        pair = torch.empty((origin.shape[0], 2 * self.width), dtype=self.rt.dtype, device=origin.device)
        self.rt.ops.stream_copy(origin, pair[:, self.width :])
        return pair

    def forward(self, resid: torch.Tensor, delta, pair: torch.Tensor, bias_row: int = 0):
        """The new stream, and nothing left to add.  ``delta`` is what the block before left (None, a ``StreamCopy``,
        a ``NormedSum``, or rows to be added); ``pair`` comes from ``begin``."""
        ops = self.rt.ops
        if isinstance(delta, UnscaledNorm):
            raise ValueError("a merge of streams cannot follow a block that folded a norm into its product")
        left = pair[:, : self.width]
        if isinstance(delta, NormedSum):
            ops.stream_copy(resid, left, delta.rows, delta.weight, delta.eps)
        else:
            if isinstance(delta, ScaledSum):
                ops.add_scaled_into_residual(resid, delta.rows, delta.factor)
            elif delta is not None and not isinstance(delta, StreamCopy):
                ops.add_into_residual(resid, delta)
            ops.stream_copy(resid, left)
        stream = self.product.forward(pair, torch.float32)
        if self.bias is not None:
            ops.add_bias_(stream, self.bias[bias_row])
        return stream, None
