"""The Figalix decoder put together from parts.

Embedding rows as they are; pre-norm layers x <- x + m * mixer(norm1(x)), x <- x + m * ff(norm2(x)) with a constant m
on what the sub-layers add and Dynamic Tanh in the place of every norm (tanh(alpha x) * w + b, no statistics of the
row); two kinds of mixer, in whatever order the configuration lists them: a state-space mixer (short causal
convolution, a matrix state per head, a gate before a unit-RMS norm over parts of the row), and two mixers side by
side on the same rows, grouped-query attention (a rotated part of each head with frequencies stretched by their index,
a window under which a sequence's first keys stay visible, one sigmoid gate per head) next to a matrix memory with
exponential gates, whose outputs are each divided by their root mean square, weighted and averaged; a dense silu-gated
feed-forward, routed experts of that form with softmax weights over all experts and a shared branch, or none; the
model's norm, then the embedding table as output head and a soft cap on the logits.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2`` (each with ``.alpha`` and ``.b``), ``l<i>.mix.*`` (state space:
``in``, ``conv``, ``conv.b``, ``dt_bias``, ``A_log``, ``D``, ``norm``, ``o``; side by side: ``left.{q,k,v,g,o,out}``,
``right.{q,k,v,i,i.b,f,f.b,g,norm,o,out}``), ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router,e<j>.{gate,up,down},
shared.{gate,up,down}}``, ``final.norm``.
"""
from __future__ import annotations

import torch

from ..config.figalix import DenseMLP, FigalixConfig
from ..parts import (Block, DynamicTanh, Embedding, GatedMLP, GQAttention, MatrixMemory, OutputHead, RotaryEmbedding, RoutedExperts,
                     SideBySideMixer, StateSpaceMixer)
from .plan import LayerCall, ModelPlan

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o"}
_MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}
_EXPERT_NAMES = {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"}


def _rotary(head_dim: int, rot):
    if rot.dims == 0:
        return None
    scaling = None
    if rot.scaling is not None:
        scaling = {"factor": rot.scaling.factor, "original": rot.scaling.original, "fast": rot.scaling.fast, "slow": rot.scaling.slow}
    return RotaryEmbedding(head_dim, rot.base, rot.dims, scaling=scaling, precise=True)


def mixer_for_layer(cfg: FigalixConfig, layer, prefix: str):
    """The mixer of one configured layer, its tensors under ``prefix``; it leaves 32-bit rows."""
    m = layer.mixer
    if layer.kind == "mamba2":
        return StateSpaceMixer(prefix, cfg.width, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, cfg.norm_eps,
                               out_dtype=torch.float32)
    a, b = m.left, m.right
    left = GQAttention(prefix + "left.", cfg.width, a.heads, a.kv_heads, a.dim, _rotary(a.dim, a.rot), window=a.window,
                       scale=a.scale, value_dim=a.vdim, names=_ATTENTION_NAMES, head_gate="g",
                       keep_first=a.keep_first if a.window else 0, out_dtype=torch.float32)
    right = MatrixMemory(prefix + "right.", cfg.width, b.heads, b.dim, b.vdim, b.gate_cap, cfg.norm_eps, out_dtype=torch.float32)
    return SideBySideMixer(left, right, cfg.width, prefix + "left.out", prefix + "right.out", cfg.norm_eps)


def feed_forward_for_layer(cfg: FigalixConfig, layer, prefix: str):
    mlp = layer.mlp
    if mlp is None:
        return None
    if isinstance(mlp, DenseMLP):
        return GatedMLP(prefix, cfg.width, mlp.ff, "silu", names=_MLP_NAMES, out_dtype=torch.float32)
    shared = None
    if mlp.shared_ff is not None:
        shared = GatedMLP(prefix + "shared.", cfg.width, mlp.shared_ff, "silu", names=_MLP_NAMES, out_dtype=torch.float32)
    return RoutedExperts(prefix, cfg.width, mlp.ff, mlp.experts, mlp.top, activation="silu_gated", names=_EXPERT_NAMES,
                         out_dtype=torch.float32, scoring="softmax_all", shared=shared)


def build_figalix_plan(cfg: FigalixConfig) -> ModelPlan:
    blocks, order, next_cache = [], [], 0
    for index, layer in enumerate(cfg.layers):
        base = f"l{index}."
        ffn = feed_forward_for_layer(cfg, layer, base + "mlp.")
        norm2 = DynamicTanh(base + "norm2", cfg.width) if ffn is not None else None
        blocks.append(Block(DynamicTanh(base + "norm1", cfg.width), mixer_for_layer(cfg, layer, base + "mix."), norm2, ffn,
                            arrangement="pre_norm", residual_scale=cfg.residual_mult))
        if layer.kind == "parallel":
            # pages for the attention side, a state slot for the memory side
            order.append(LayerCall(block=index, cache=(next_cache, next_cache + 1), write=True))
            next_cache += 2
        else:
            order.append(LayerCall(block=index, cache=next_cache, write=True))
            next_cache += 1
    return ModelPlan(
        embedding=Embedding("embed", cfg.vocab, cfg.width),
        blocks=blocks,
        order=order,
        final_norm=DynamicTanh("final.norm", cfg.width),
        head=OutputHead("embed", cfg.vocab, cfg.width, softcap=cfg.logit_softcap),
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=None,
    ).validate()
