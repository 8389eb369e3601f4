"""Causal grouped-query attention over the paged cache.

Order of operations as in the reference
(crates/llm-backend/src/core/qwen/ops/attention_full.rs:197-309): project q, k, v;
optional per-head RMSNorm of q and k with one weight [d] shared by the heads,
before the position encoding (:252-287); rotate q and k at the absolute
position; append k, v to the cache before attending, so a token sees itself
(crates/llm-backend/src/core/native_attention.rs:307-309); scores q.k * scale over the
visible rows, softmax, weighted sum of v (:731-764); output projection.  Query
head h reads kv head h // (q_heads / kv_heads) (:732).  A window W makes row i
see rows [i - W + 1, i].

Every size and constant is a constructor argument; the position encoding is a
part of its own.  A layer built with ``reads_only`` has no k and v projections:
it projects q alone and reads a cache that another layer filled.

Three further options, each a constructor argument: ``value_dim`` (values of
another width than queries and keys; the output projection then reads
heads * value_dim columns), ``bias`` (q, k and v carry biases, added with the
projection), and ``qk_norm_over="projection"``: the RMS norm runs over ALL
columns of a token's q (and of its k) at once, before the split into heads,
with one weight per column, where ``"head"`` norms each head with a shared
weight [d].  A layer with any of the three takes one preparation kernel (bias,
norm, queries out, keys and values to their pages) and then the same attention
kernels; cache rows are max(head_dim, value_dim) wide, rounded up to 8, the
unused columns zero, and the output projection's matrix gets zero columns where
a head's output is padding.  ``out_dtype`` is the dtype of the mixer's result
(default: the runtime's).

Further options, again constructor arguments.  With biases or a value width of its own and NO norm over the
projection the layer may have a ``RotaryEmbedding`` (any part of a head, any frequency table): a second preparation
kernel adds the biases, rotates, and writes queries, keys and values.  ``head_factor`` names a tensor [q_heads] by
which each head's scores are multiplied (folded into the queries in 32-bit before they are rounded); ``softcap`` c
turns a score s into c tanh(s / c) before the softmax; ``chunk`` C lets position i see j <= i only when both lie in
the same run of C positions counted from the sequence's start (all keys stay cached); ``gate`` names a matrix
[q_heads * value_dim, hidden]: the concatenated heads are multiplied by sigmoid(gate x) before the output
projection (the matrix rides in the stacked q, k, v product); ``out_bias`` names a bias of the output projection.
``head_gate`` names a matrix [q_heads, hidden] instead: ONE number per head, sigmoid(head_gate x)_h, multiplies head
h's output (it rides in the stacked product too).  ``keep_first`` F goes with a ``window`` W: position i sees j <= i
when i - j < W or j < F, so a sequence's first F keys stay visible at their true positions (the cache keeps their
pages when the window gives the others back).  A ``RotaryEmbedding`` whose cosine and sine carry a factor
(``amplitude``) is applied with it by the preparation kernel.  A ``RotaryEmbedding`` that pairs neighbouring columns
has the rows of the q and k matrices (and biases) put in its ``head_order`` at load; scores do not change with the
order of a head's columns, as long as queries and keys share it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import KVCacheNeed, Mixer, PositionEncoding, Runtime, WeightSpec
from .linear import Linear
from .rope import RotaryEmbedding


class GQAttention(Mixer):
    def __init__(self, prefix: str, hidden_size: int, q_heads: int, kv_heads: int, head_dim: int,
                 position: Optional[PositionEncoding], *, window: Optional[int] = None,
                 qk_norm_eps: Optional[float] = None, scale: Optional[float] = None, reads_only: bool = False,
                 names: Optional[Dict[str, str]] = None, value_dim: Optional[int] = None, bias: bool = False,
                 qk_norm_over: str = "head", out_dtype: Optional[torch.dtype] = None, head_factor: Optional[str] = None,
                 softcap: Optional[float] = None, chunk: Optional[int] = None, gate: Optional[str] = None,
                 out_bias: Optional[str] = None, head_gate: Optional[str] = None, keep_first: int = 0):
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads are not a multiple of {kv_heads} kv heads")
        if qk_norm_over not in ("head", "projection"):
            raise ValueError(f"qk_norm_over must be 'head' or 'projection', got {qk_norm_over!r}")
        n = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight",
             "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias"}
        n.update(names or {})
        self.prefix = prefix
        self.hidden_size, self.q_heads, self.kv_heads, self.head_dim = hidden_size, q_heads, kv_heads, head_dim
        self.value_dim = head_dim if value_dim is None else value_dim
        self.window = window
        self.qk_norm_eps = qk_norm_eps
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.position = position
        self.reads_only = reads_only
        self.bias = bias
        self.out_dtype = out_dtype
        # the preparation that takes biases, a norm over the whole projection and values of their own width
        self.softcap = float(softcap) if softcap else None
        self.chunk = int(chunk) if chunk else None
        if self.chunk and window:
            raise ValueError("a layer has a window or a chunked mask, not both")
        if (self.softcap or self.chunk) and reads_only:
            raise ValueError("a soft cap or a chunked mask is not built for a layer that reads another layer's cache")
        self.head_factor_name = prefix + head_factor if head_factor else None
        self.gate_name = prefix + gate if gate else None
        self.head_gate_name = prefix + head_gate if head_gate else None
        self.keep_first = int(keep_first or 0)
        if self.keep_first and not window:
            raise ValueError("kept first keys go with a window")
        if gate and head_gate:
            raise ValueError("an output gate has a number per column or a number per head, not both")
        if (self.keep_first or head_gate) and reads_only:
            raise ValueError("kept first keys or a gate per head are not built for a layer that reads another layer's cache")
        self.out_bias_name = prefix + out_bias if out_bias else None
        self.head_factor = self.out_bias = None
        self.defer_output_bias = False  # a block whose next norm adds the bias sets this
        shifted_rotation = isinstance(position, RotaryEmbedding) and (position.offset != 0 or position.amplitude != 1.0
                                                                      or position.pairing != "halves")
        self.wide = (head_gate is not None or self.keep_first > 0 or bias or self.value_dim != head_dim or (qk_norm_eps is not None and qk_norm_over == "projection")
                     or head_factor is not None or gate is not None or shifted_rotation or self.softcap is not None
                     or self.chunk is not None or out_bias is not None)
        self.norm_over_projection = qk_norm_eps is not None and qk_norm_over == "projection"
        self.pad_dim = head_dim
        if self.wide:
            if position is not None and (self.norm_over_projection or not isinstance(position, RotaryEmbedding)):
                raise ValueError("with biases, a value width of its own, a head factor or a gate, queries and keys take a "
                                 "RotaryEmbedding or no position encoding, and none together with a norm over the projection")
            if self.norm_over_projection and (head_factor or gate):
                raise ValueError("a head factor or an output gate is not built together with a norm over the projection")
            if qk_norm_eps is not None and qk_norm_over == "head":
                raise ValueError("a per-head q/k norm is not built together with biases or values of their own width")
            self.pad_dim = -(-max(head_dim, self.value_dim) // 8) * 8
        sources = [(prefix + n["q"], q_heads * head_dim)]
        if not reads_only:
            sources += [(prefix + n["k"], kv_heads * head_dim), (prefix + n["v"], kv_heads * self.value_dim)]
        if self.gate_name:
            sources.append((self.gate_name, q_heads * self.value_dim))
        if self.head_gate_name:
            sources.append((self.head_gate_name, q_heads))
        # a rotation that pairs neighbouring columns: queries and keys are projected with their columns in the kernels' order
        self.q_order = self.k_order = None
        stacked_order = None
        if isinstance(position, RotaryEmbedding) and position.head_order() is not None:
            if not self.wide:
                raise ValueError("a rotation of neighbouring columns is built for the preparation that takes biases and partial rotations")
            self.q_order = position.row_order(q_heads)
            self.k_order = None if reads_only else position.row_order(kv_heads)
            total = sum(rows for _, rows in sources)
            stacked_order = torch.arange(total)
            stacked_order[: q_heads * head_dim] = self.q_order
            if self.k_order is not None:
                stacked_order[q_heads * head_dim : (q_heads + kv_heads) * head_dim] = q_heads * head_dim + self.k_order
        self.qkv = Linear(sources, hidden_size, row_order=stacked_order)
        self.out = Linear([(prefix + n["o"], hidden_size)], q_heads * self.value_dim,
                          column_groups=(q_heads, self.value_dim, self.pad_dim) if self.wide else None)
        self.q_norm_name, self.k_norm_name = prefix + n["q_norm"], prefix + n["k_norm"]
        self.bias_names = (prefix + n["q_bias"], prefix + n["k_bias"], prefix + n["v_bias"])
        self.q_norm_weight = self.k_norm_weight = None
        self.q_bias = self.k_bias = self.v_bias = None

    def cache_need(self):
        if self.wide:
            return KVCacheNeed(self.kv_heads, self.pad_dim, self.window, key_dim=self.head_dim, value_dim=self.value_dim,
                               keep_first=self.keep_first)
        return KVCacheNeed(self.kv_heads, self.head_dim, self.window)

    @property
    def capture_safe(self) -> bool:
        """The kernels read positions, lengths and block tables on the device; the position encoding is a part of
        its own and answers for itself."""
        return self.position is None or bool(self.position.capture_safe)

    @property
    def kernels_only(self) -> bool:
        return self.position is None or bool(self.position.kernels_only)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {**self.qkv.weight_specs(), **self.out.weight_specs()}
        if self.qk_norm_eps is not None:
            over = (self.q_heads, self.kv_heads) if self.norm_over_projection else (1, 1)
            specs[self.q_norm_name] = WeightSpec((over[0] * self.head_dim,), "norm")
            if not self.reads_only:
                specs[self.k_norm_name] = WeightSpec((over[1] * self.head_dim,), "norm")
        if self.bias:
            specs[self.bias_names[0]] = WeightSpec((self.q_heads * self.head_dim,), "bias")
            if not self.reads_only:
                specs[self.bias_names[1]] = WeightSpec((self.kv_heads * self.head_dim,), "bias")
                specs[self.bias_names[2]] = WeightSpec((self.kv_heads * self.value_dim,), "bias")
        if self.head_factor_name:
            specs[self.head_factor_name] = WeightSpec((self.q_heads,), "norm")
        if self.out_bias_name:
            specs[self.out_bias_name] = WeightSpec((self.hidden_size,), "bias")
        if self.position is not None:
            specs.update(self.position.weight_specs())
        return specs

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.qkv.load(weights, rt)
        self.out.load(weights, rt)
        if self.qk_norm_eps is not None:
            self.q_norm_weight = weights.on_device(self.q_norm_name, torch.float32)
            if not self.reads_only:
                self.k_norm_weight = weights.on_device(self.k_norm_name, torch.float32)
        if self.bias:
            self.q_bias = weights.on_device(self.bias_names[0], torch.float32)
            if self.q_order is not None:
                self.q_bias = self.q_bias[self.q_order.to(rt.device)].contiguous()
            if not self.reads_only:
                self.k_bias = weights.on_device(self.bias_names[1], torch.float32)
                if self.k_order is not None:
                    self.k_bias = self.k_bias[self.k_order.to(rt.device)].contiguous()
                self.v_bias = weights.on_device(self.bias_names[2], torch.float32)
        if self.head_factor_name:
            self.head_factor = weights.on_device(self.head_factor_name, torch.float32)
        if self.out_bias_name:
            self.out_bias = weights.on_device(self.out_bias_name, torch.float32)
        if self.position is not None:
            self.position.load(weights, rt)

    def deferred_bias(self) -> Optional[torch.Tensor]:
        """The output projection's bias, for whoever adds this mixer's output into the stream, when the block said
        that it will (``defer_output_bias``)."""
        return self.out_bias if self.defer_output_bias else None

    def takes_unscaled(self, rows: int) -> bool:
        return not self.wide and self.qkv.fuses_norms(rows)

    def fuses_into_norm(self, rows: int) -> bool:
        return self.out_bias is None and self.out.fuses_norms(rows)

    def forward(self, x, batch, cache, write_cache: bool = True) -> torch.Tensor:
        result = self.out.forward(self._mix(x, batch, cache, write_cache), self.out_dtype)
        if self.out_bias is not None and not self.defer_output_bias:
            self.rt.ops.add_bias_(result, self.out_bias)
        return result

    def _mix_wide(self, x, batch, cache, write_cache: bool) -> torch.Tensor:
        """[T, q_heads * pad_dim]: the stacked product in 32-bit, one preparation kernel, the attention kernels."""
        ops = self.rt.ops
        nkv = 0 if self.reads_only else self.kv_heads
        if nkv and not write_cache:
            raise ValueError("an attention layer with k and v projections of its own must fill its cache")
        table = batch.block_tables[cache.group]
        qkv = self.qkv.forward(x, torch.float32)
        if not self.norm_over_projection:
            rot = self.position
            q = ops.qkv_rope_write(qkv, self.q_heads, nkv, self.head_dim, self.value_dim, self.pad_dim, self.q_bias, self.k_bias,
                                   self.v_bias, self.head_factor, rot.inv_freq if rot is not None else None,
                                   rot.offset if rot is not None else 0, rot.rotary_dim if rot is not None else 0,
                                   cache.kv, table, batch.request_of_token, batch.positions, self.rt.dtype,
                                   rot_amplitude=rot.amplitude if rot is not None else 1.0)
            mixed = ops.paged_attention(q, cache.kv, table, batch, self.window, self.scale, chunk=self.chunk, softcap=self.softcap,
                                        keep_first=self.keep_first)
            gate_at = self.q_heads * self.head_dim + nkv * (self.head_dim + self.value_dim)
            if self.gate_name:
                ops.sigmoid_gate_(mixed, qkv[:, gate_at:], self.q_heads, self.value_dim, self.pad_dim)
            if self.head_gate_name:
                ops.head_gate_(mixed, qkv[:, gate_at : gate_at + self.q_heads], self.q_heads, self.value_dim, self.pad_dim)
            return mixed
        q = ops.qkv_wide_norm_write(qkv, self.q_heads, nkv, self.head_dim, self.value_dim, self.pad_dim, self.q_bias,
                                    self.k_bias, self.v_bias, self.q_norm_weight, self.k_norm_weight, self.qk_norm_eps or 0.0,
                                    cache.kv, table, batch.request_of_token, batch.positions, self.rt.dtype)
        return ops.paged_attention(q, cache.kv, table, batch, self.window, self.scale)

    def forward_into_norm(self, x, batch, cache, write_cache, resid, spec):
        return self.out.forward_into_norm(self._mix(x, batch, cache, write_cache), resid, spec)

    def _mix(self, x, batch, cache, write_cache: bool) -> torch.Tensor:
        """Everything before the output projection: [T, q_heads * head_dim]."""
        ops = self.rt.ops
        nq, d = self.q_heads, self.head_dim
        nkv = 0 if self.reads_only else self.kv_heads  # kv heads that this layer projects
        if write_cache and self.reads_only:
            raise ValueError("a reads_only attention layer cannot fill a cache")
        if self.wide:
            return self._mix_wide(x, batch, cache, write_cache)
        table = batch.block_tables[cache.group]
        qkv = self.qkv.forward(x)  # [T, (nq + 2 nkv) d]
        fused_table = self.position.fused_table() if isinstance(self.position, RotaryEmbedding) else None
        q = qkv[:, : nq * d].unflatten(1, (nq, d))
        if ((self.position is None or fused_table is not None) and write_cache and nkv == self.kv_heads
                and getattr(ops, "decode_prepares_qk", None) is not None
                and ops.decode_prepares_qk(qkv, cache.kv, batch, nq, nkv, d)):
            # every request brings one token: norm, rotation and the cache write happen inside the attention kernel
            return ops.attention_decode_qk(qkv, nq, nkv, d, self.q_norm_weight, self.k_norm_weight, fused_table,
                                           self.qk_norm_eps or 0.0, cache.kv, table, batch, self.window, self.scale)
        if self.position is None or fused_table is not None:
            ops.qk_norm_rope_kv_write_(qkv, nq, nkv, d, self.q_norm_weight, self.k_norm_weight, fused_table,
                                       self.qk_norm_eps or 0.0, cache.kv if write_cache else None, table,
                                       batch.request_of_token, batch.positions, write_cache)
        else:
            k = qkv[:, nq * d : (nq + nkv) * d].unflatten(1, (nkv, d))
            v = qkv[:, (nq + nkv) * d :].unflatten(1, (nkv, d))
            if self.qk_norm_eps is not None:
                ops.head_rmsnorm_(q, self.q_norm_weight, self.qk_norm_eps)
                if nkv:
                    ops.head_rmsnorm_(k, self.k_norm_weight, self.qk_norm_eps)
            self.position.apply(q, k, batch.positions)
            if write_cache:
                ops.kv_write(k, v, cache.kv, table, batch.request_of_token, batch.positions)
        return ops.paged_attention(q, cache.kv, table, batch, self.window, self.scale)
