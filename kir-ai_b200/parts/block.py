"""A block: two norms, a mixer and a feed-forward, and how they are arranged.

The residual stream is 32-bit; what a sub-layer produces (``delta``, in the
runtime dtype) is added into it by the next norm, so that sum and norm are one
pass over the row.  ``pre_norm`` is the reference's order
(crates/llm-backend/src/core/qwen/ops/decoder.rs:210-314): n1 = norm1(h);
a = mixer(n1); n2 = norm2(h + a); m = ffn(n2); out = h + a + m.  ``parallel``
feeds one norm to both sub-layers: out = h + mixer(n) + ffn(n).  ``out_norm``
norms what a sub-layer produced, not what it reads: h' = h + norm1(mixer(h));
out = h' + norm2(ffn(h')), the sub-layers reading the stream itself (rounded to
the runtime dtype); such a block may have no feed-forward (``ffn`` and ``norm2``
None), and it asks its sub-layers for 32-bit outputs (``out_dtype``), which the
norm kernel reads.

Where the parts on both sides offer it, a norm is not a kernel of its own: the product before it adds into the
stream and writes the norm's rows without their 1 / rms factor (``forward_into_norm``), and the product after it
applies that factor to its result (``takes_unscaled``); see ``UnscaledNorm``.  The block asks the parts and falls
back to the separate norm kernel when either side declines, so a part without these methods still fits.

A ``pre_norm`` block may carry a ``shift`` (``parts.shift.TokenShift``): what the mixer reads, norm1's rows, is first
mixed with the row of the token before.  The shift keeps a request's last row in a state slot of its own (the
layer call's ``shift_cache``), the norm hands it 32-bit rows, and the first norm then stays a kernel.  A mixer whose
output projection has a bias may leave it to the norm that adds its output into the stream (``deferred_bias``).

``sandwich`` norms both what a sub-layer reads and what it produced: h' = h + post1(mixer(norm1(h)));
out = h' + post2(ffn(norm2(h'))), with the norms on the outputs given as ``post_norm1`` and ``post_norm2``; the
feed-forward with its two norms may be missing.  The sub-layers leave 32-bit rows.  The norm on an output and the norm
that reads the stream next are one pass over the row: the block hands what is left to add on as a ``NormedSum``, which
a norm that ``takes_normed_sum`` adds while it norms (the next sub-layer's, the next block's first, or the model's
last); any other reader has it settled into the stream first.

``residual_scale`` m (``pre_norm`` only) multiplies what every sub-layer adds: h <- h + m * mixer(norm1(h)), then
h <- h + m * ffn(norm2(h)).  The sub-layers then leave 32-bit rows (a feed-forward may leave several terms,
``FeedForward.forward_terms``), which travel to the next norm as a ``ScaledSum``; a norm that ``takes_scaled_sum`` adds
them in its own pass, for any other a kernel adds them first.  No norm is folded into a product on this path.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from .base import FeedForward, FusedNormSpec, Mixer, Norm, NormedSum, Part, Runtime, ScaledSum, StreamCopy, UnscaledNorm, WeightSpec

ARRANGEMENTS = ("pre_norm", "parallel", "out_norm", "sandwich")


def _offers(part, method: str, rows: int) -> bool:
    """Whether a part has the optional ``method`` and answers yes for a batch of ``rows`` tokens; a part
    written without it declines."""
    fn = getattr(part, method, None)
    return bool(fn is not None and fn(rows))


class Block(Part):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], arrangement: str = "pre_norm",
                 shift: Optional[Part] = None, residual_scale: Optional[float] = None, post_norm1: Optional[Norm] = None,
                 post_norm2: Optional[Norm] = None):
        if (arrangement == "sandwich") != (post_norm1 is not None) or (post_norm2 is not None) != (arrangement == "sandwich" and ffn is not None):
            raise ValueError("the sandwich arrangement, and it alone, has a norm on every sub-layer's output")
        if arrangement == "sandwich" and ((ffn is None) != (norm2 is None) or shift is not None):
            raise ValueError("the sandwich arrangement has its second pair of norms exactly when it has a feed-forward, and no token shift")
        self.post_norm1, self.post_norm2 = post_norm1, post_norm2
        if residual_scale is not None and (arrangement != "pre_norm" or shift is not None):
            raise ValueError("a factor on the sub-layers' outputs is built for the pre_norm arrangement without a token shift")
        self.residual_scale = None if residual_scale is None else float(residual_scale)
        if shift is not None and arrangement != "pre_norm":
            raise ValueError("a token shift is built for the pre_norm arrangement only")
        if arrangement not in ARRANGEMENTS:
            raise ValueError(f"unknown block arrangement {arrangement!r}; known: {ARRANGEMENTS}")
        if arrangement == "pre_norm" and (ffn is None) != (norm2 is None):
            raise ValueError("the pre_norm arrangement has a second norm exactly when it has a feed-forward")
        if ffn is None and arrangement == "parallel":
            raise ValueError(f"the {arrangement} arrangement needs a feed-forward")
        if arrangement == "out_norm" and (ffn is None) != (norm2 is None):
            raise ValueError("the out_norm arrangement has a second norm exactly when it has a feed-forward")
        self.norm1, self.mixer, self.norm2, self.ffn, self.arrangement = norm1, mixer, norm2, ffn, arrangement
        self.shift = shift
        # a bias on the mixer's output is added by the second norm's kernel where both sides can
        self._bias_to_norm2 = bool(arrangement == "pre_norm" and ffn is not None and getattr(norm2, "takes_delta_bias", False)
                                   and hasattr(mixer, "deferred_bias"))
        if self._bias_to_norm2:
            mixer.defer_output_bias = True

    def _parts(self):
        return [p for p in (self.norm1, self.shift, self.mixer, self.post_norm1, self.norm2, self.ffn, self.post_norm2) if p is not None]

    def shift_need(self):
        """What the block's token shift keeps per request (None without one)."""
        return self.shift.cache_need() if self.shift is not None else None

    @property
    def reads_stream(self) -> bool:
        """Whether the block's first sub-layer reads the stream itself (rounded to the runtime dtype) and not a norm
        of it: whoever made the stream may then hand its runtime-dtype copy along as a ``StreamCopy``."""
        return self.arrangement == "out_norm"

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(part, "capture_safe", False)) for part in self._parts())

    @property
    def kernels_only(self) -> bool:
        return all(bool(getattr(part, "kernels_only", False)) for part in self._parts())

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self._parts():
            specs.update(part.weight_specs())
        return specs

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        for part in self._parts():
            part.load(weights, rt)

    def entry_spec(self, rows: int) -> Optional[FusedNormSpec]:
        """What the block before needs to take over this block's first norm for a batch of ``rows`` tokens;
        None if the norm stays a kernel."""
        if (self.arrangement != "pre_norm" or self.shift is not None or self.residual_scale is not None
                or not _offers(self.mixer, "takes_unscaled", rows)):
            return None
        return self._spec(self.norm1)

    @staticmethod
    def _spec(norm) -> Optional[FusedNormSpec]:
        fn = getattr(norm, "fused_spec", None)
        return fn() if fn is not None else None

    def forward(self, resid: torch.Tensor, delta, batch, cache, write_cache: bool = True,
                following: Optional["Block"] = None, shift_cache=None) -> Tuple[torch.Tensor, object]:
        """Takes the stream and what the block before left: its not-yet-added output, or (if this block's
        ``entry_spec`` was offered to it as ``following``) the ``UnscaledNorm`` of the first norm.  Returns the
        stream and what this block leaves, in the same two forms."""
        rows = resid.shape[0]
        if isinstance(delta, StreamCopy) and self.arrangement != "out_norm":
            delta = None  # the block before left nothing to add
        if isinstance(delta, ScaledSum) and (self.arrangement != "pre_norm" or self.shift is not None
                                             or not getattr(self.norm1, "takes_scaled_sum", False)):
            self.rt.ops.add_scaled_into_residual(resid, delta.rows, delta.factor)
            delta = None
        if isinstance(delta, NormedSum) and (self.arrangement != "sandwich" or not getattr(self.norm1, "takes_normed_sum", False)):
            delta.settle(resid, self.rt.ops)
            delta = None
        if self.arrangement == "sandwich":
            return self._forward_sandwich(resid, delta, batch, cache, write_cache)
        if self.residual_scale is not None:
            return self._forward_scaled(resid, delta, batch, cache, write_cache)
        if self.arrangement == "out_norm":
            return self._forward_out_norm(resid, delta, batch, cache, write_cache)
        if self.arrangement == "pre_norm":
            if self.shift is not None:
                if isinstance(delta, UnscaledNorm):
                    raise ValueError("a block with a token shift cannot follow a block that folded its first norm into a product")
                if batch.max_query_len == 1 and getattr(self.norm1, "fuses_shift", False) and hasattr(self.shift, "fused_args"):
                    # every request brings one token: the shift runs inside the norm's kernel
                    n1 = self.norm1.add_forward(resid, delta, shift=self.shift.fused_args(batch, shift_cache))
                else:
                    n1 = self.shift.forward(self.norm1.add_forward(resid, delta, wide=True), batch, shift_cache)
            else:
                n1 = delta if isinstance(delta, UnscaledNorm) else self.norm1.add_forward(resid, delta)
            if self.ffn is None:
                return resid, self.mixer.forward(n1, batch, cache, write_cache)  # the next norm adds it
            spec2 = self._spec(self.norm2) if _offers(self.mixer, "fuses_into_norm", rows) and _offers(self.ffn, "takes_unscaled", rows) else None
            if spec2 is not None:
                n2 = self.mixer.forward_into_norm(n1, batch, cache, write_cache, resid, spec2)
            elif self._bias_to_norm2:
                n2 = self.norm2.add_forward(resid, self.mixer.forward(n1, batch, cache, write_cache), delta_bias=self.mixer.deferred_bias())
            else:
                n2 = self.norm2.add_forward(resid, self.mixer.forward(n1, batch, cache, write_cache))
            spec_next = following.entry_spec(rows) if following is not None and _offers(self.ffn, "fuses_into_norm", rows) else None
            if spec_next is not None:
                return resid, self.ffn.forward_into_norm(n2, batch, resid, spec_next)
            return resid, self.ffn.forward(n2, batch)
        n = self.norm1.add_forward(resid, delta)
        a = self.mixer.forward(n, batch, cache, write_cache)
        m = self.ffn.forward(n, batch)
        self.norm1.rt.ops.add_into_residual(resid, a)
        return resid, m

    def _forward_sandwich(self, resid, delta, batch, cache, write_cache):
        """A norm before and after each sub-layer; what the last norm makes is left to the next reader of the stream."""
        if isinstance(delta, UnscaledNorm):
            raise ValueError("a sandwich block cannot follow a block that folded this block's norm into its product")
        if isinstance(delta, ScaledSum):
            self.rt.ops.add_scaled_into_residual(resid, delta.rows, delta.factor)
            delta = None
        n1 = self.norm1.add_forward(resid, delta)
        left = self._left_to_add(self.post_norm1, self.mixer.forward(n1, batch, cache, write_cache), resid)
        if self.ffn is None:
            return resid, left
        n2 = self.norm2.add_forward(resid, left)
        return resid, self._left_to_add(self.post_norm2, self.ffn.forward(n2, batch), resid)

    def _left_to_add(self, norm, y, resid):
        """norm(y) as something the next norm adds in its own pass, where both sides can; else it is added here."""
        if hasattr(norm, "normed_sum") and os.environ.get("KIRAI_FUSE_NORMS", "1") != "0":
            return norm.normed_sum(y)
        norm.add_normed(resid, y)
        return None

    def _forward_scaled(self, resid, delta, batch, cache, write_cache):
        """pre_norm with a factor on what the sub-layers add; their outputs are 32-bit rows."""
        ops, scale = self.rt.ops, self.residual_scale
        n1 = self.norm1.add_forward(resid, delta)
        left = ScaledSum(self._wide([self.mixer.forward(n1, batch, cache, write_cache)]), scale)
        if self.ffn is None:
            return resid, left
        if getattr(self.norm2, "takes_scaled_sum", False):
            n2 = self.norm2.add_forward(resid, left)
        else:
            ops.add_scaled_into_residual(resid, left.rows, left.factor)
            n2 = self.norm2.add_forward(resid, None)
        return resid, ScaledSum(self._wide(self.ffn.forward_terms(n2, batch)), scale)

    @staticmethod
    def _wide(rows):
        return [r if r.dtype == torch.float32 else r.float() for r in rows]

    def _forward_out_norm(self, resid, delta, batch, cache, write_cache):
        ops, narrow, rows = self.rt.ops, self.rt.dtype != torch.float32, resid.shape[0]
        if isinstance(delta, UnscaledNorm):
            raise ValueError("an out_norm block cannot follow a block that folded this block's norm into its product")
        if isinstance(delta, StreamCopy):
            x = delta.rows
        else:
            if delta is not None:
                ops.add_into_residual(resid, delta)
            x = None
        if x is None:
            x = ops.round_rows(resid) if narrow else resid
        x = self.norm1.add_normed(resid, self.mixer.forward(x, batch, cache, write_cache))
        if self.ffn is not None:
            # a feed-forward may take the norm on its output over (``adds_normed``), as products take over the norms
            # around them in the pre_norm arrangement
            spec = self._spec(self.norm2) if _offers(self.ffn, "adds_normed", rows) else None
            if spec is not None:
                x = self.ffn.forward_add_normed(x, batch, resid, spec)
            else:
                x = self.norm2.add_normed(resid, self.ffn.forward(x if narrow else resid, batch))
        return resid, StreamCopy(x if narrow else None)
