"""A feed-forward made of small experts, of which every token uses a few.

Router logits z = W_router x in 32-bit; the ``top`` experts with the largest
logits are chosen and weighted by the softmax over the chosen logits alone;
an expert is down(act(up x)) without biases, act(z) = relu(z)^2; the result is
the weighted sum of the chosen experts' outputs.

How it runs: the experts' up matrices are stacked along the output axis and
their down matrices laid side by side along the input axis at load.  One
product gives every expert's hidden rows, one kernel applies the activation
and multiplies by the token's routing weight of the column's expert (zero for
an expert that was not chosen), and the down product then sums the chosen
experts' outputs in its own accumulation.  Nothing depends on how many tokens
an expert drew, so a step of single tokens can be captured in a graph; the
price is that every expert's rows are computed for every token, experts / top
times the arithmetic that the chosen experts alone would need.  For a step of
few tokens that price is none: the products are bound by reading the weights,
and a handful of tokens between them choose most experts anyway.

Steps of many tokens (``GROUPED_MIN_ROWS`` pairs of token and chosen expert, in
bfloat16, expert and model width multiples of 128) sort their pairs by expert
on the device instead: a plan kernel gives every pair a row in a buffer whose
experts' stretches are padded to tiles of 128 rows, the rows are gathered, two
grouped products (the first with relu^2 in its epilogue) multiply every tile
with its expert's matrices, and a combine kernel sums each token's rows with
its routing weights in 32-bit.  Only the chosen experts' arithmetic is done.
This path keeps a second copy of the down matrices, stacked along the output
axis.  Neither path waits for the host.

Options.  ``activation="silu_gated"``: an expert is down(silu(gate x) * (up x)) with a gate matrix of its own; the
experts' gate and up matrices are stacked expert by expert ([gate_e; up_e]; where the expert size is a multiple of 8, with
the rows of each in turns of eight, the order of the tensor-core product's gated epilogue), the few-token kernel applies
the gated activation and the routing weight together, and the many-token path runs the grouped product with the
activation in its epilogue (other expert sizes: without an epilogue, then the framework's gated-activation kernel).  ``scoring="softmax_all"``: the weights are the chosen experts'
shares of the softmax over ALL experts' logits, not renormalised (the choice is the same: the largest logits).
``shared``: a feed-forward that runs for every token beside the routed experts; its output is added (``forward_terms``
hands both terms to whoever adds them into the stream).

``activation="clamped_gated"`` (with ``limit`` L and ``slope`` a): an expert is down(g sigmoid(a g) (u + 1)) with
g = min(gate x, L) and u = clamp(up x, -L, L); laid out and run like ``silu_gated``.  ``scoring="sigmoid"``: an
expert's score is sigmoid(z).  The choice looks at score + ``correction`` (a stored vector [experts], named by
``names["correction"]``; None: no correction), and, with ``groups`` = (count, keep), only at experts of the ``keep``
groups (of ``count`` equal groups of neighbouring experts) whose two largest choice scores sum highest.  The weights
are the chosen experts' scores without the correction, not renormalised.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FeedForward, Runtime, WeightSpec
from .linear import Linear

ACTIVATIONS = ("relu2", "silu_gated", "clamped_gated")
SCORINGS = ("softmax_chosen", "softmax_all", "sigmoid")
GROUPED_MIN_ROWS = 512  # pairs of (token, chosen expert) from which a step sorts them by expert


class RoutedExperts(FeedForward):
    capture_safe = True
    kernels_only = True

    def __init__(self, prefix: str, hidden_size: int, expert_size: int, experts: int, top: int, *,
                 activation: str = "relu2", names: Optional[Dict[str, str]] = None,
                 out_dtype: Optional[torch.dtype] = None, scoring: str = "softmax_chosen", shared: Optional[FeedForward] = None,
                 limit: Optional[float] = None, slope: float = 1.0, correction: bool = False, groups: Optional[tuple] = None):
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown expert activation {activation!r}; known: {ACTIVATIONS}")
        if scoring not in SCORINGS:
            raise ValueError(f"unknown router scoring {scoring!r}; known: {SCORINGS}")
        self.gated = activation in ("silu_gated", "clamped_gated")
        self.gate_act = "clamped" if activation == "clamped_gated" else "silu"
        if (activation == "clamped_gated") != (limit is not None) or (limit is not None and not limit > 0.0):
            raise ValueError("the clamped activation, and it alone, takes a positive limit")
        self.limit, self.slope = float(limit or 0.0), float(slope)
        self.over_all = scoring == "softmax_all"
        self.scored = scoring == "sigmoid"
        if (correction or groups is not None) and not self.scored:
            raise ValueError("a correction on the choice and a choice among groups go with sigmoid scores")
        count, keep = groups if groups is not None else (1, 1)
        if experts % count or not 0 < keep <= count or top > keep * (experts // count):
            raise ValueError(f"{experts} experts in {count} equal groups of which {keep} stay open do not give {top} experts a token")
        self.groups = (int(count), int(keep))
        self.has_correction = bool(correction)
        self.correction: Optional[torch.Tensor] = None
        self.rule: Optional[dict] = None
        self.shared = shared
        if not 0 < top <= experts:
            raise ValueError(f"every token uses {top} of {experts} experts")
        n = {"router": "router.weight", "up": "experts.{e}.up_proj.weight", "down": "experts.{e}.down_proj.weight",
             "gate": "experts.{e}.gate_proj.weight", "correction": "router.correction"}
        n.update(names or {})
        self.correction_name = prefix + n["correction"]
        self.hidden_size, self.expert_size, self.experts, self.top = hidden_size, expert_size, experts, top
        self.activation = activation
        self.out_dtype = out_dtype
        self.router_name = prefix + n["router"]
        self.interleaved = self.gated and expert_size % 8 == 0
        if self.gated:
            # expert by expert: its gate rows, then its up rows; where the expert size allows, in the order of the
            # tensor-core product's gated epilogue instead: 8 gate rows, their 8 up rows, 8 gate rows, ...
            order = None
            if self.interleaved:
                block = torch.arange(expert_size).view(expert_size // 8, 1, 8)
                one = torch.cat([block, block + expert_size], dim=1).reshape(-1)  # of one expert's 2 * expert_size rows
                order = (torch.arange(experts)[:, None] * (2 * expert_size) + one[None, :]).reshape(-1)
            self.up = Linear([(prefix + n[kind].format(e=e), expert_size) for e in range(experts) for kind in ("gate", "up")],
                             hidden_size, row_order=order)
        else:
            self.up = Linear([(prefix + n["up"].format(e=e), expert_size) for e in range(experts)], hidden_size)
        self.down = Linear([(prefix + n["down"].format(e=e), expert_size) for e in range(experts)], hidden_size,
                           side_by_side=True)
        self.down_stacked = Linear([(prefix + n["down"].format(e=e), hidden_size) for e in range(experts)], expert_size)
        self.router: Optional[torch.Tensor] = None
        self.router_product: Optional[Linear] = None
        self.grouped = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        shared = self.shared.weight_specs() if self.shared is not None else {}
        correction = {self.correction_name: WeightSpec((self.experts,), "bias")} if self.has_correction else {}
        return {self.router_name: WeightSpec((self.experts, self.hidden_size), "linear"), **correction,
                **self.up.weight_specs(), **self.down.weight_specs(), **shared}

    @property
    def capture_safe(self) -> bool:
        return self.shared is None or bool(getattr(self.shared, "capture_safe", False))

    @property
    def kernels_only(self) -> bool:
        return self.shared is None or bool(getattr(self.shared, "kernels_only", False))

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.router = weights.on_device(self.router_name, torch.float32)
        if self.has_correction:
            self.correction = weights.on_device(self.correction_name, torch.float32)
        if self.scored:
            self.rule = {"correction": self.correction, "groups": self.groups[0], "keep": self.groups[1]}
        self.up.load(weights, rt)
        self.down.load(weights, rt)
        if self.shared is not None:
            self.shared.load(weights, rt)
        # sorting by expert pays only where a token uses a part of the experts, and needs whole 128-row boxes per expert
        self.grouped = (rt.dtype == torch.bfloat16 and self.top < self.experts and self.expert_size % 128 == 0
                        and self.hidden_size % 128 == 0 and hasattr(rt.ops, "linear_grouped"))
        if self.grouped:
            self.down_stacked.load(weights, rt)
        # A router stored in bfloat16 times bfloat16 rows with 32-bit accumulation IS the 32-bit product of those
        # values, so steps of many tokens take the tensor-core product for the logits and a kernel for the choice alone.
        if rt.dtype == torch.bfloat16 and weights.stored(self.router_name).dtype == torch.bfloat16 and self.hidden_size % 8 == 0:
            self.router_product = Linear([(self.router_name, self.experts)], self.hidden_size)
            self.router_product.load(weights, rt)

    ROUTER_PRODUCT_MIN_ROWS = 128

    def _route(self, x: torch.Tensor, want_chosen: bool):
        ops = self.rt.ops
        if self.router_product is not None and x.shape[0] >= self.ROUTER_PRODUCT_MIN_ROWS:
            return ops.router_choose_(self.router_product.forward(x, torch.float32), self.top, want_chosen, over_all=self.over_all,
                                      rule=self.rule)
        return ops.router_gates(x, self.router, self.top, want_chosen, over_all=self.over_all, rule=self.rule)

    def _sorts(self, rows: int) -> bool:
        return self.grouped and rows * self.top >= GROUPED_MIN_ROWS

    def _sorted_rows(self, x: torch.Tensor):
        """The many-token path up to the experts' outputs: (y [slots, E] bfloat16, slot_of, routing weights)."""
        ops = self.rt.ops
        _, ids, mix = self._route(x, True)
        tile_group, slot_of, row_of_slot = ops.route_plan(ids, self.experts)
        rows = ops.route_gather(x, row_of_slot)
        if self.gated and self.interleaved:
            hidden = ops.linear_grouped(rows, self.up.weight, self.experts, tile_group, gated=(self.gate_act, self.limit, self.slope))
        elif self.gated:
            hidden = ops.gated_activation(ops.linear_grouped(rows, self.up.weight, self.experts, tile_group), self.gate_act,
                                          self.limit, self.slope)
        else:
            hidden = ops.linear_grouped(rows, self.up.weight, self.experts, tile_group, relu2=True)
        return ops.linear_grouped(hidden, self.down_stacked.weight, self.experts, tile_group), slot_of, mix

    def adds_normed(self, rows: int) -> bool:
        """Optional, for a block that norms this part's OUTPUT: whether, for a batch of ``rows`` tokens, the part has
        ``forward_add_normed(x, batch, resid, spec)``, which adds the normed output into the 32-bit stream itself (the
        weighted sum of a token's expert rows is then never written out) and returns the stream's runtime-dtype copy."""
        return self.shared is None and self._sorts(rows) and self.rt.ops.route_combine_norm_add_takes(self.hidden_size)

    def forward_add_normed(self, x: torch.Tensor, batch, resid: torch.Tensor, spec):
        y, slot_of, mix = self._sorted_rows(x)
        return self.rt.ops.route_combine_norm_add(resid, y, slot_of, mix, spec.weight, spec.eps, self.rt.dtype)

    def forward_terms(self, x: torch.Tensor, batch=None) -> list:
        """[the routed experts' weighted sum] and, with a shared branch, [.., its output]."""
        routed = self._forward_routed(x, batch)
        return [routed] if self.shared is None else [routed, self.shared.forward(x, batch)]

    def forward(self, x: torch.Tensor, batch=None) -> torch.Tensor:
        if self.shared is None:
            return self._forward_routed(x, batch)
        if self.out_dtype != torch.float32:
            raise ValueError("experts with a shared branch leave 32-bit rows (out_dtype=torch.float32), which are added in 32-bit")
        routed, shared = self.forward_terms(x, batch)
        return self.rt.ops.add_scaled_into_residual(routed, [shared if shared.dtype == torch.float32 else shared.float()], 1.0)

    def _forward_routed(self, x: torch.Tensor, batch=None) -> torch.Tensor:
        ops = self.rt.ops
        if self._sorts(x.shape[0]):
            y, slot_of, mix = self._sorted_rows(x)
            out = ops.route_combine(y, slot_of, mix)
            return out if self.out_dtype == torch.float32 else ops.round_rows(out)
        gates = self._route(x, False)
        hidden = self.up.forward(x)
        if self.gated:
            hidden = ops.gated_expert_gate(hidden, gates, self.expert_size, self.gate_act, self.limit, self.slope,
                                           interleaved=self.interleaved)
        else:
            ops.relu2_gate_(hidden, gates, self.expert_size)
        return self.down.forward(hidden, self.out_dtype)
