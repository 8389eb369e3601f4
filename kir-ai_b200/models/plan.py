"""A model as data: parts, and the order in which the blocks run.

``ModelPlan`` holds an embedding, a list of blocks, the ``order`` (a list of
``LayerCall``), a final norm and an output head.  The order may name a block
twice (weights shared between depths; each call then has a cache of its own)
and a call may read the cache that an earlier call filled (``write`` false).
``DecoderModel`` runs a plan on a batch; it knows nothing of any architecture.

The reference hard-codes the loop over ``spec.num_hidden_layers``
(crates/llm-backend/src/core/qwen/ops/decoder.rs:481-515 prefill, :526-566 decode).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..parts.base import Norm, NormedSum, Runtime, ScaledSum, StreamCopy, WeightSpec
from ..parts.block import Block
from ..parts.embedding import Embedding, OutputHead


@dataclass(frozen=True)
class LayerCall:
    """Run ``block`` with cache layer ``cache`` (None: the mixer keeps nothing; a tuple of cache layers for a mixer
    whose ``cache_need()`` is a tuple of needs, as two mixers side by side of which one keeps pages and one a state);
    ``write`` false reads what an earlier call wrote in the same step.  ``shift_cache`` is the cache layer of the
    block's token shift, where it has one (a state slot per request; every call has its own).  ``enter`` = (index
    into the plan's ``entries``, row of its bias table): ahead of this call the stream starts over from itself and the
    embedding's rows (``parts.merge.StreamMerge``), as at the head of every pass of a looped stretch."""

    block: int
    cache: object = None
    write: bool = True
    shift_cache: Optional[int] = None
    enter: Optional[tuple] = None


class PlanError(ValueError):
    pass


@dataclass
class ModelPlan:
    embedding: Embedding
    blocks: List[Block]
    order: List[LayerCall]
    final_norm: Norm
    head: OutputHead
    vocab_size: int
    hidden_size: int
    max_positions: Optional[int] = None
    ignorable_weights: List[str] = field(default_factory=list)  # tensors a folder may hold that no part wants
    cache_needs: List[object] = field(default_factory=list)  # filled by validate(): one need per cache layer
    entries: List[object] = field(default_factory=list)  # parts that stand between blocks (``LayerCall.enter``)

    def validate(self) -> "ModelPlan":
        """Checks the order against the blocks and derives the need of every cache layer."""
        needs: Dict[int, object] = {}
        for step, call in enumerate(self.order):
            if not 0 <= call.block < len(self.blocks):
                raise PlanError(f"order[{step}] names block {call.block}, but there are {len(self.blocks)} blocks")
            if call.enter is not None and not 0 <= call.enter[0] < len(self.entries):
                raise PlanError(f"order[{step}] enters through part {call.enter[0]}, but there are {len(self.entries)} such parts")
            shift_need = getattr(self.blocks[call.block], "shift_need", lambda: None)()
            if (shift_need is None) != (call.shift_cache is None):
                raise PlanError(f"order[{step}]: block {call.block} {'needs' if shift_need is not None else 'has no use for'} a cache layer for its token shift")
            if shift_need is not None:
                if call.shift_cache in needs:
                    raise PlanError(f"order[{step}]: cache layer {call.shift_cache} is written by two calls")
                needs[call.shift_cache] = shift_need
            need = self.blocks[call.block].mixer.cache_need()
            if need is None:
                if call.cache is not None:
                    raise PlanError(f"order[{step}]: block {call.block}'s mixer keeps nothing, yet cache {call.cache} is named")
                continue
            if call.cache is None:
                raise PlanError(f"order[{step}]: block {call.block}'s mixer needs a cache layer")
            if isinstance(need, tuple):
                # several needs: every one a cache layer of its own, written by this call
                if not isinstance(call.cache, tuple) or len(call.cache) != len(need) or not call.write:
                    raise PlanError(f"order[{step}]: block {call.block}'s mixer needs {len(need)} cache layers that it writes")
                for layer, one in zip(call.cache, need):
                    if layer in needs:
                        raise PlanError(f"order[{step}]: cache layer {layer} is written by two calls")
                    needs[layer] = one
                continue
            if isinstance(call.cache, tuple):
                raise PlanError(f"order[{step}]: block {call.block}'s mixer needs one cache layer, {call.cache} are named")
            if call.write:
                if call.cache in needs:
                    raise PlanError(f"order[{step}]: cache layer {call.cache} is written by two calls")
                needs[call.cache] = need
            else:
                if call.cache not in needs:
                    raise PlanError(f"order[{step}]: cache layer {call.cache} is read before any call wrote it")
                if needs[call.cache] != need:
                    raise PlanError(f"order[{step}]: reader needs {need}, cache layer {call.cache} holds {needs[call.cache]}")
        if sorted(needs) != list(range(len(needs))):
            raise PlanError(f"cache layers must be numbered 0..n-1 without gaps, got {sorted(needs)}")
        self.cache_needs = [needs[i] for i in range(len(needs))]
        return self

    def parts(self):
        return [self.embedding, *self.entries, *self.blocks, self.final_norm, self.head]

    def capture_safe(self) -> bool:
        """Whether a step of single tokens may be recorded into a CUDA graph: every part promises it
        (``Part.capture_safe``)."""
        return all(bool(getattr(part, "capture_safe", False)) for part in self.parts())

    def kernels_only(self) -> bool:
        """Whether products may be held back and launched together: every part promises to touch activations
        through the kernels only (``Part.kernels_only``)."""
        return all(bool(getattr(part, "kernels_only", False)) for part in self.parts())

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self.parts():
            for name, spec in part.weight_specs().items():
                if name in specs and specs[name].shape != spec.shape:
                    raise PlanError(f"tensor {name} is wanted with shapes {specs[name].shape} and {spec.shape}")
                specs[name] = spec
        return specs


class DecoderModel:
    """Runs a plan: embedding, the blocks in ``order``, and logits at chosen rows."""

    def __init__(self, plan: ModelPlan, rt: Runtime):
        self.plan = plan.validate()
        self.rt = rt
        # with parts that touch activations through the kernels only, a step's small products are launched together
        self._kernels_only = plan.kernels_only() and hasattr(rt.ops, "chained_products")
        self._entered = sorted({call.enter[0] for call in plan.order if call.enter is not None})
        self.nvtx = False  # True: every layer call is an NVTX range (the reference counts attempts and fallbacks per
        # kernel instead, crates/llm-native-runtime/src/native_metrics.rs:7-70; here ops.launch_counts does that)

    def load(self, weights) -> "DecoderModel":
        for part in self.plan.parts():
            part.load(weights, self.rt)
        return self

    def forward(self, batch, cache) -> tuple:
        """The residual stream [T, H] (32-bit) and the last block's not-yet-added output."""
        nvtx = torch.cuda.nvtx if self.nvtx else None  # ranges around the layer calls, for a timeline tool
        with self.rt.ops.chained_products(self._kernels_only):
            embedding, order, delta = self.plan.embedding, self.plan.order, None
            first = self.plan.blocks[order[0].block] if order else None
            if getattr(first, "reads_stream", False) and hasattr(embedding, "forward_with_copy"):
                # the first block reads the stream itself: its runtime-dtype copy is written with it
                resid, copy = embedding.forward_with_copy(batch.token_ids, batch.positions)
                delta = StreamCopy(copy) if copy is not None else None
            elif getattr(embedding, "uses_positions", False):
                resid = embedding.forward(batch.token_ids, batch.positions)
            else:
                resid = embedding.forward(batch.token_ids)
            # every part that stands between blocks takes the embedding's rows now, before a block changes the stream
            pairs = {index: self.plan.entries[index].begin(resid) for index in self._entered}
            for i, call in enumerate(order):
                if call.enter is not None:
                    resid, delta = self.plan.entries[call.enter[0]].forward(resid, delta, pairs[call.enter[0]], call.enter[1])
                if isinstance(call.cache, tuple):
                    view = tuple(cache.layer_view(layer) for layer in call.cache)
                else:
                    view = cache.layer_view(call.cache) if call.cache is not None else None
                following = self.plan.blocks[order[i + 1].block] if i + 1 < len(order) else None
                if nvtx:
                    nvtx.range_push(f"layer call {i}: block {call.block}, {batch.num_tokens} tokens")
                if call.shift_cache is not None:
                    resid, delta = self.plan.blocks[call.block].forward(resid, delta, batch, view, call.write, following,
                                                                        shift_cache=cache.layer_view(call.shift_cache))
                else:
                    resid, delta = self.plan.blocks[call.block].forward(resid, delta, batch, view, call.write, following)
                if nvtx:
                    nvtx.range_pop()
        return resid, delta

    def logits(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """32-bit logits [len(rows), V] of the token rows ``rows`` (int32, on the device)."""
        if isinstance(delta, StreamCopy):
            delta = None  # the last block left the stream complete
        if isinstance(delta, NormedSum) and not getattr(self.plan.final_norm, "takes_normed_sum", False):
            delta.settle(resid, self.rt.ops)
            delta = None
        if isinstance(delta, ScaledSum) and not getattr(self.plan.final_norm, "takes_scaled_sum", False):
            self.rt.ops.add_scaled_into_residual(resid, delta.rows, delta.factor)
            delta = None
        with self.rt.ops.chained_products(self._kernels_only):
            normed = self.plan.final_norm.add_forward_rows(resid, delta, rows)
            logits = self.plan.head.forward(normed)
        return logits
