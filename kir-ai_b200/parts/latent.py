"""Latent attention: keys and values of all heads are read out of one small cached row per token.

Per token the layer makes a query latent c_q = rms(W_dq h) * w_q and, from W_dkv h, a key/value latent
c = rms(first kv_rank columns) * w_kv and one rotated key part r (the last rot_dim columns, not normed) that all
heads share.  Head i has the query [q_i (dim columns), q'_i (rot_dim columns, rotated)] = rows of W_uq c_q, the key
[W_uk,i c, r] and the value W_uv,i c; scores are (q_i . W_uk,i c + q'_i . r) * scale, causal softmax, and the heads'
values go through W_o.

Only [c, r] is cached: kv_rank + rot_dim numbers a token, whatever the number of heads.  The layer attends in the
latent's own space, which the two identities q_i . (W_uk,i c) = (W_uk,i^T q_i) . c and
sum_j p_j W_uv,i c_j = W_uv,i (sum_j p_j c_j) allow: at load W_uk is folded into the query up-projection
(rows W_uk,i^T W_uq,i) and W_uv into the output projection (columns W_o,i W_uv,i), both worked out in 64-bit and
rounded once.  What runs is then attention of ``heads`` query heads over ONE key/value head whose key row is [c, r]
and whose value row is c, on the framework's attention kernels (cache rows are kv_rank + rot_dim wide, rounded up to
8; the value row repeats c).  Against attention over per-head keys and values this reads kv_rank + rot_dim columns
a key instead of heads * (dim + rot_dim + vdim), and multiplies with queries of kv_rank + rot_dim columns instead
of dim + rot_dim.

With ``gate`` (the name of a matrix [heads * value_dim, hidden]) the concatenated heads' values are multiplied by
sigmoid(gate x) ahead of the output projection.  A gate stands between W_uv and W_o, so W_uv is then NOT folded into
the output projection: the attention's sums of latents go through a product per head (``ops.head_linear_gate``, the
gate in the same kernel) and W_o reads heads * value_dim columns as stored; the gate's matrix rides in the stacked down
projection.  A rotation that pairs neighbouring columns (``RotaryEmbedding(pairing="neighbours")``) has the rows that
make the rotated query columns and the shared key part put in its ``head_order`` at load; a rotation with an
``amplitude`` is applied with it by both preparation kernels.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import KVCacheNeed, Mixer, Runtime, WeightSpec
from .linear import Linear
from .rope import RotaryEmbedding


class LatentAttention(Mixer):
    kernels_only = True

    def __init__(self, prefix: str, hidden_size: int, heads: int, dim: int, rot_dim: int, value_dim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, rotary: RotaryEmbedding, names: Optional[Dict[str, str]] = None,
                 out_dtype: Optional[torch.dtype] = None, gate: Optional[str] = None):
        n = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}
        n.update(names or {})
        self.gate_name = prefix + gate if gate else None
        if rotary.head_dim != rot_dim or rotary.rotary_dim != rot_dim or rotary.offset != 0:
            raise ValueError("the rotation of latent attention covers the whole shared key part")
        self.hidden_size, self.heads, self.dim, self.rot_dim, self.value_dim = hidden_size, heads, dim, rot_dim, value_dim
        self.q_rank, self.kv_rank, self.scale, self.eps, self.rotary, self.out_dtype = q_rank, kv_rank, float(scale), float(eps), rotary, out_dtype
        self.row = kv_rank + rot_dim                 # a cached key row, and a query head in the latent's space
        self.pad_dim = -(-self.row // 8) * 8
        self.names = {key: prefix + value for key, value in n.items()}
        self.order = rotary.head_order()  # of the rotated columns, where the rotation pairs neighbours
        sources = [(self.names["dq"], q_rank), (self.names["dkv"], kv_rank + rot_dim)]
        if self.gate_name:
            sources.append((self.gate_name, heads * value_dim))
        stacked_order = None
        if self.order is not None:
            stacked_order = torch.arange(sum(rows for _, rows in sources))
            stacked_order[q_rank + kv_rank : q_rank + kv_rank + rot_dim] = q_rank + kv_rank + self.order
        self.down = Linear(sources, hidden_size, row_order=stacked_order)
        self.up_q = Linear([("", heads * self.row)], q_rank)                 # filled from uq and uk at load
        if self.gate_name:
            self.out = Linear([(self.names["o"], hidden_size)], heads * value_dim)
        else:
            self.out = Linear([("", hidden_size)], heads * self.pad_dim)     # filled from o and uv at load
        self.up_v: Optional[torch.Tensor] = None                             # [heads, value_dim, kv_rank], with a gate
        self.up_v_padded: Optional[torch.Tensor] = None                      # [heads * value_dim, pad_dim], zero columns
        self.q_norm = self.kv_norm = None

    def cache_need(self) -> KVCacheNeed:
        return KVCacheNeed(1, self.pad_dim, None, key_dim=self.row, value_dim=self.kv_rank)

    @property
    def capture_safe(self) -> bool:
        return bool(self.rotary.capture_safe)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        return {**self.down.weight_specs(), **(self.out.weight_specs() if self.gate_name else {}),
                n["dq_norm"]: WeightSpec((self.q_rank,), "norm"), n["dkv_norm"]: WeightSpec((self.kv_rank,), "norm"),
                n["uq"]: WeightSpec((self.heads * (self.dim + self.rot_dim), self.q_rank)),
                n["uk"]: WeightSpec((self.heads * self.dim, self.kv_rank)),
                n["uv"]: WeightSpec((self.heads * self.value_dim, self.kv_rank)),
                n["o"]: WeightSpec((self.hidden_size, self.heads * self.value_dim))}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        n, H, d, r, dv, kr = self.names, self.heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank
        self.down.load(weights, rt)
        self.rotary.load(weights, rt)
        self.q_norm = weights.on_device(n["dq_norm"], torch.float32)
        self.kv_norm = weights.on_device(n["dkv_norm"], torch.float32)
        wide = dict(device=rt.device, dtype=torch.float64)
        uq = weights.stored(n["uq"]).to(**wide).view(H, d + r, self.q_rank)
        uk = weights.stored(n["uk"]).to(**wide).view(H, d, kr)
        uv = weights.stored(n["uv"]).to(**wide).view(H, dv, kr)
        o = weights.stored(n["o"]).to(**wide).view(self.hidden_size, H, dv)
        # query head i in the latent's space: [W_uk,i^T W_uq,i (kv_rank rows); the rotated rows of W_uq,i]
        rotated = uq[:, d:] if self.order is None else uq[:, d:][:, self.order.to(rt.device)]
        up_q = torch.cat([torch.einsum("hdk,hdq->hkq", uk, uq[:, :d]), rotated], dim=1)
        self.up_q.load_matrix(up_q.reshape(H * self.row, self.q_rank), rt)
        if self.gate_name:
            # the gate stands between W_uv and W_o: both stay as stored
            self.up_v = weights.stored(n["uv"]).to(device=rt.device, dtype=rt.dtype).view(H, dv, kr).contiguous()
            self.up_v_padded = None
            if rt.dtype == torch.bfloat16 and self.pad_dim % 8 == 0:
                # for steps of many tokens: the heads' matrices as the groups of one grouped product over padded rows
                self.up_v_padded = torch.zeros((H * dv, self.pad_dim), dtype=rt.dtype, device=rt.device)
                self.up_v_padded[:, :kr] = self.up_v.view(H * dv, kr)
            self.out.load(weights, rt)
            return
        # the output projection reads the heads' sums of latents: columns W_o,i W_uv,i, zero where a row is padding
        out = torch.zeros((self.hidden_size, H, self.pad_dim), **wide)
        out[:, :, :kr] = torch.einsum("ehv,hvk->ehk", o, uv)
        self.out.load_matrix(out.reshape(self.hidden_size, H * self.pad_dim), rt)

    def forward(self, x, batch, cache, write_cache: bool = True) -> torch.Tensor:
        if not write_cache:
            raise ValueError("a latent attention layer fills its own cache")
        ops = self.rt.ops
        table = batch.block_tables[cache.group]
        down = self.down.forward(x, torch.float32)
        amplitude = self.rotary.amplitude
        q_latent = ops.latent_prepare(down, self.q_rank, self.kv_rank, self.rot_dim, self.q_norm, self.kv_norm,
                                      self.rotary.inv_freq, self.eps, cache.kv, table, batch.request_of_token,
                                      batch.positions, self.rt.dtype, rot_amplitude=amplitude)
        q = ops.qkv_rope_write(self.up_q.forward(q_latent, torch.float32), self.heads, 0, self.row, self.row, self.pad_dim,
                               None, None, None, None, self.rotary.inv_freq, self.kv_rank, self.rot_dim, None, table,
                               batch.request_of_token, batch.positions, self.rt.dtype, rot_amplitude=amplitude)
        mixed = ops.paged_attention(q, cache.kv, table, batch, None, self.scale)
        if self.gate_name:
            gate = down[:, self.q_rank + self.kv_rank + self.rot_dim :]
            mixed = ops.head_linear_gate(mixed.view(mixed.shape[0], -1), self.up_v, self.heads, self.kv_rank, gate,
                                         padded_weight=self.up_v_padded)
        return self.out.forward(mixed, self.out_dtype)
