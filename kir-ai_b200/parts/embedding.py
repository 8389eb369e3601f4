"""Token embedding (row gather; optionally times a constant and plus a sinusoidal position vector) and the output head.

crates/llm-backend/src/core/qwen/ops/embedding.rs:26-36 (gather, error for an id outside
the vocabulary) and crates/llm-backend/src/core/qwen/ops/lm_head.rs:68-86 of the
reference; a tied head names the embedding table (crates/llm-models/src/qwen.rs:282-288),
and both then share one device buffer.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Part, Runtime, WeightSpec


def _table(weights, rt: Runtime, name: str, hidden_size: int):
    """The table [V, H] on the device, one copy per stored tensor: in the tensor-core product's box layout
    where that kernel takes it (bfloat16, H a multiple of 8; the embedding gathers rows from the boxes), else
    row-major."""
    if rt.dtype == torch.bfloat16 and hidden_size % 8 == 0:
        def make():
            return rt.ops.tile_weight(weights.stored(name).to(device=rt.device, dtype=rt.dtype))
        return weights.shared((name, "boxes"), make)
    return weights.on_device(name, rt.dtype)


def sinusoid_frequencies(width: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i / width) for the column pairs (2i, 2i + 1) of a row of ``width`` columns, worked out in 64-bit
    and kept in 32-bit."""
    pairs = torch.arange((width + 1) // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * pairs / float(width)).to(torch.float32)


class Embedding(Part):
    """``scale`` multiplies the gathered rows; ``sinusoid_base`` b adds to the token at position p the vector whose
    column 2i is sin(p b^(-2i/H)) and whose column 2i + 1 is the cosine of the same angle (angles in 32-bit).  With
    neither, the rows are gathered as they are."""

    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, vocab_size: int, hidden_size: int, *, scale: float = 1.0,
                 sinusoid_base: Optional[float] = None):
        self.weight_name, self.vocab_size, self.hidden_size = weight_name, vocab_size, hidden_size
        self.scale, self.sinusoid_base = float(scale), sinusoid_base
        self.uses_positions = sinusoid_base is not None
        self.plain = self.scale == 1.0 and sinusoid_base is None
        self.frequencies: Optional[torch.Tensor] = None
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size), "embedding")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        if self.plain:
            self.table = _table(weights, rt, self.weight_name, self.hidden_size)
            return
        self.table = weights.on_device(self.weight_name, rt.dtype)
        if self.sinusoid_base is not None:
            self.frequencies = sinusoid_frequencies(self.hidden_size, self.sinusoid_base).to(rt.device)

    def forward(self, token_ids: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The 32-bit residual stream [T, H] that the blocks add into."""
        if self.plain:
            return self.rt.ops.embedding(self.table, token_ids)
        stream, _ = self.rt.ops.embedding_scaled(self.table, token_ids, self.scale, positions, self.frequencies)
        return stream

    def forward_with_copy(self, token_ids: torch.Tensor, positions: Optional[torch.Tensor] = None):
        """(stream, its copy in the runtime dtype or None when that is 32-bit): for a first block that reads the stream
        itself, written in the same pass."""
        if self.plain:
            return self.forward(token_ids), None
        return self.rt.ops.embedding_scaled(self.table, token_ids, self.scale, positions, self.frequencies,
                                            copy_dtype=None if self.rt.dtype == torch.float32 else self.rt.dtype)


class OutputHead(Part):
    """Logits = W x in 32-bit, W [V, H] (its own tensor, or the embedding table when tied).  ``softcap`` c turns a
    logit z into c tanh(z / c)."""

    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, vocab_size: int, hidden_size: int, softcap: Optional[float] = None):
        self.weight_name, self.vocab_size, self.hidden_size = weight_name, vocab_size, hidden_size
        self.softcap = float(softcap) if softcap else None
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size), "embedding")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = _table(weights, rt, self.weight_name, self.hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.rt.ops.linear(x, self.weight, torch.float32)
        return self.rt.ops.softcap_(logits, self.softcap) if self.softcap else logits
