"""The Bikilix decoder put together from parts.

Embedding rows times a constant; layers with a norm before AND after each sub-layer, x <- x + norm1b(mixer(norm1(x))),
x <- x + norm2b(ff(norm2(x))), every norm an RMS norm whose stored tensor is the weight minus one (y = x / rms(x) * (1 + w));
two kinds of mixer, in whatever order the configuration lists them: grouped-query attention with biases on q, k and v,
a rotated leading part of every head (neighbouring columns paired) and a sliding window, and latent attention (one
small cached row per token for all heads, queries through a latent of their own, the shared key part rotated with
frequencies stretched by their index, a sigmoid gate on the heads' values); a dense relu^2 feed-forward, routed experts
(sigmoid scores, a correction on the choice, a choice among groups of experts, a clamped gated activation), or none;
a stretch of layers may run several times in a row with the same weights, every run with a cache of its own, and ahead
of every such pass the stream starts over as W [x; x0] + b_pass from itself and the embedding's rows x0; the model's
norm, then the embedding table as output head.

Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``,
``l<i>.mix.*`` (attention: ``q``, ``k``, ``v`` with ``.b`` biases, ``o``; latent attention: ``dq``, ``dq.norm``, ``uq``,
``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``g``, ``o``), ``l<i>.mlp.{up,down}`` or ``l<i>.mlp.{router,correction,
e<j>.{gate,up,down}}``, ``final.norm``.
"""
from __future__ import annotations

import torch

from ..config.bikilix import BikilixConfig, DenseMLP
from ..parts import (Block, Embedding, GQAttention, LatentAttention, OutputHead, PlainMLP, RMSNorm, RotaryEmbedding, RoutedExperts,
                     StreamMerge)
from .plan import LayerCall, ModelPlan

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}
_MLP_NAMES = {"up": "up", "down": "down"}
_EXPERT_NAMES = {"router": "router", "correction": "correction", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"}
EXPERT_SLOPE = 1.702  # the design's constant inside the experts' sigmoid


def _rotary(head_dim: int, rot) -> RotaryEmbedding:
    scaling = None
    if rot.scaling is not None:
        scaling = {"factor": rot.scaling.factor, "original": rot.scaling.original, "fast": rot.scaling.fast, "slow": rot.scaling.slow}
    return RotaryEmbedding(head_dim, rot.base, rot.dims, scaling=scaling, precise=True, pairing="neighbours")


def mixer_for_layer(cfg: BikilixConfig, layer, prefix: str):
    """The mixer of one configured layer, its tensors under ``prefix``; it leaves 32-bit rows."""
    m = layer.mixer
    if layer.kind == "attention":
        return GQAttention(prefix, cfg.width, m.heads, m.kv_heads, m.dim, _rotary(m.dim, m.rot) if m.rot.dims else None,
                           window=m.window, scale=m.scale, value_dim=m.vdim, bias=True, names=_ATTENTION_NAMES,
                           out_dtype=torch.float32)
    return LatentAttention(prefix, cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, cfg.norm_eps,
                           _rotary(m.rot_dim, m.rot), out_dtype=torch.float32, gate="g")


def feed_forward_for_layer(cfg: BikilixConfig, layer, prefix: str):
    mlp = layer.mlp
    if mlp is None:
        return None
    if isinstance(mlp, DenseMLP):
        return PlainMLP(prefix, cfg.width, mlp.ff, "relu2", names=_MLP_NAMES, out_dtype=torch.float32)
    return RoutedExperts(prefix, cfg.width, mlp.ff, mlp.experts, mlp.top, activation="clamped_gated", limit=mlp.limit,
                         slope=EXPERT_SLOPE, names=_EXPERT_NAMES, out_dtype=torch.float32, scoring="sigmoid", correction=True,
                         groups=(mlp.groups, mlp.keep))


def build_bikilix_plan(cfg: BikilixConfig) -> ModelPlan:
    def norm(name: str) -> RMSNorm:
        return RMSNorm(name, cfg.width, cfg.norm_eps, centre=1.0)

    blocks = []
    for index, layer in enumerate(cfg.layers):
        base = f"l{index}."
        ffn = feed_forward_for_layer(cfg, layer, base + "mlp.")
        blocks.append(Block(norm(base + "norm1"), mixer_for_layer(cfg, layer, base + "mix."),
                            norm(base + "norm2") if ffn is not None else None, ffn, arrangement="sandwich",
                            post_norm1=norm(base + "norm1b"), post_norm2=norm(base + "norm2b") if ffn is not None else None))
    entries = []
    if cfg.loop is not None:
        entries.append(StreamMerge("loop.in", cfg.width, "loop.step", cfg.loop.times))
    # every run of a layer has a cache layer of its own; a pass of the looped stretch enters through the merge
    order, next_cache = [], 0
    for number, indices in cfg.passes():
        for place, index in enumerate(indices):
            enter = (0, number) if number is not None and place == 0 else None
            order.append(LayerCall(block=index, cache=next_cache, write=True, enter=enter))
            next_cache += 1
    return ModelPlan(
        embedding=Embedding("embed", cfg.vocab, cfg.width, scale=cfg.embedding_scale),
        blocks=blocks,
        order=order,
        final_norm=norm("final.norm"),
        head=OutputHead("embed", cfg.vocab, cfg.width),
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=None,
        entries=entries,
    ).validate()
